"""``va_prefill_static``: the prefill for callers that are not allowed to allocate device memory
where the operator runs (a serving process whose memory pool belongs to another component, a
plugin inside someone else's stream-ordered region).  Its scratch is a fixed array inside the
library instead of a caller-provided workspace.

The GPU test drives the entry point through the C ABI twice in a row, with different inputs, and
requires the same output as ``va_prefill`` with an ordinary workspace: the second call finds the
first call's leftovers in the shared scratch and must not be disturbed by them.  The file name
makes pytest collect it last.
"""
import ctypes as C

import pytest
import torch


def _args(L, q, k, v, out, causal, chunk, counts=None):
    b, h, s, d = q.shape
    t4 = lambda t: L.Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return L.PrefillArgs(L.VA_BF16, b, h, k.shape[1], s, k.shape[2], d, 64, 16, 16, int(causal), chunk, 64,
                         t4(q), t4(k), t4(v), t4(out), 0.6931, None, 0, None, 0,
                         counts.data_ptr() if counts is not None else None, None, 0)


def test_static_scratch_limit_is_enforced_before_any_launch(built_library):
    """A problem whose scratch exceeds the built-in array is refused with a clear error; the
    check is pure host arithmetic, so it runs without a GPU."""
    from vecattention_b200 import _lib as L
    a = L.PrefillArgs()
    a.dtype, a.batch, a.heads, a.kv_heads, a.sq, a.sk, a.head_dim = 0, 1, 32, 32, 32768, 32768, 128
    a.pq, a.bk, a.group_k_block, a.causal, a.chunk_size, a.compat_bsq = 64, 16, 16, 0, 32768, 64
    need = C.c_size_t(0)
    assert L.lib().va_prefill_workspace_bytes(C.byref(a), C.byref(need)) == 0
    assert need.value > L.VA_STATIC_SCRATCH_BYTES
    rc = L.lib().va_prefill_static(C.byref(a), None)
    assert rc == -8
    assert "VA_STATIC_SCRATCH_BYTES" in L.status_string(rc)
    assert L.lib().va_prefill_static(None, None) == -1


@pytest.mark.gpu
def test_static_scratch_prefill_equals_workspace_prefill_twice(built_library):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from vecattention_b200 import _lib as L
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the third problem does not fit the built-in scratch in one pass, so it runs chunk by chunk there
    # while the workspace entry point runs it in one pass: both must agree
    for call, (seed, causal, s, chunk) in enumerate([(1, False, 2048, 1024), (2, True, 1200, 512), (3, True, 12288, 1024)]):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(1, 4, s, 128, generator=g).to(torch.bfloat16).cuda()
        k = torch.randn(1, 2, s, 128, generator=g).to(torch.bfloat16).cuda()
        v = torch.randn(1, 2, s, 128, generator=g).to(torch.bfloat16).cuda()
        k[:, :, ::19] *= 3.0
        nq = (s + 63) // 64
        # the existing entry point, workspace from the caller
        out_ws = torch.empty_like(q)
        cnt_ws = torch.empty(1, 4, nq, dtype=torch.int32, device="cuda")
        a = _args(L, q, k, v, out_ws, causal, chunk, cnt_ws)
        need = C.c_size_t(0)
        assert lib.va_prefill_workspace_bytes(C.byref(a), C.byref(need)) == 0
        # (the third problem needs more than the built-in array when run in one pass)
        assert (need.value <= L.VA_STATIC_SCRATCH_BYTES) == (call < 2)
        ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        a.workspace, a.workspace_bytes = ws.data_ptr(), need.value
        assert lib.va_prefill(C.byref(a), stream) == 0
        # the allocation-free entry point: same arguments, no workspace
        out_st = torch.full_like(q, float("nan"))
        cnt_st = torch.full_like(cnt_ws, -1)
        b = _args(L, q, k, v, out_st, causal, chunk, cnt_st)
        assert lib.va_prefill_static(C.byref(b), stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(cnt_st, cnt_ws), f"call {call}: selection counts differ"
        assert int(cnt_ws.sum()) > 0
        err = (out_st.float() - out_ws.float()).abs()
        assert torch.isfinite(out_st.float()).all()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, f"call {call}: {err.max().item()}"
        if call < 2:  # and against the CPU oracle (the third problem would take it minutes)
            import math
            from oracle import vecattn_oracle as O
            ref, sel = O.vecattention_prefill(q.cpu(), k.cpu(), v.cpu(), math.exp(-0.6931) - 1e-9, 64, 16, 16, causal, chunk,
                                              return_selection=True)
            ref_counts = torch.cat([c for c, _ in sel], dim=2)
            assert (cnt_st.cpu() - ref_counts).abs().sum() <= 2, f"call {call}: counts differ from the oracle"
            err = (out_st.float().cpu() - ref.float()).abs()
            assert err.max() <= 2e-2 and err.mean() <= 2e-3, f"call {call} vs oracle: {err.max().item()}"
