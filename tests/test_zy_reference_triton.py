"""The reference's own Triton kernels, compiled and run natively on the B200, against the CUDA
path on the same bf16/fp16 inputs.  Needs a B200 and the installed reference.

What this settles by measurement (the Triton CPU interpreter, which produced the committed
fixtures, can run neither bf16 nor the compiled kernels' 16-bit scaling, and handles the NaN-padded
key tail differently):

  * the pooled queries of ``average_vector(use_triton=True)`` (spattn/src/utils.py:340-351);
  * the selection of ``fuse_qk_softmax_minp_wo_causal`` (spattn/src/kernels/vecattention_kernels.py:
    59-181, kernels :206-345) in bf16 at the sizes of benchmark configurations 2-5 (one KV group, all
    query tiles, the operator's chunk loop), with a key length that is not a multiple of the key
    block (NaN-padded tail, :117-127), with per-head gaps (the second kernel) and in fp16;
  * the recall / sparsity measure of the threshold tuner, ``seg_pr_perHead``
    (spattn/threshold/model_tuner.py:118-226), against ``recall.selection_recall_sparsity``.

Both selections are given the reference's pooled queries, so the comparison isolates the selection
rule; sets must be equal except keys whose estimate lies within 1e-6 of the keep/drop boundary (the
reference's order across key-block groups depends on atomics, so lists are compared as sets).

The reference is read from ``baseline/_ref`` (``baseline/install_reference.sh`` puts it there);
its import of ``vllm_flash_attn`` (the sparse-attention fork, not part of the reference tree) is
satisfied by an empty stand-in, exactly as ``tests/golden/make_golden.py`` does.  A missing
install fails the tests: it must not go unnoticed.  The file name makes pytest collect these tests
after all others except the last file.
"""
import math
import os
import sys
import types

import pytest
import torch

from parity_util import boundary_band, membership

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


@pytest.fixture(scope="module")
def va(built_library):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import vecattention_b200 as va_mod
    return va_mod


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF_DIR, "spattn")):
        pytest.fail(f"{REF_DIR} does not hold the installed reference: run baseline/install_reference.sh")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    stub = types.ModuleType("vllm_flash_attn")

    def sparse_attn_func(*a, **k):
        raise RuntimeError("vllm_flash_attn.sparse_attn_func is not part of the reference tree")
    stub.sparse_attn_func = sparse_attn_func
    sys.modules.setdefault("vllm_flash_attn", stub)
    from spattn.src.kernels.vecattention_kernels import fuse_qk_softmax_minp_wo_causal
    from spattn.src.utils import average_vector
    return types.SimpleNamespace(average_vector=average_vector, select=fuse_qk_softmax_minp_wo_causal)


def _time_ms(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _compare_pooling(ours, theirs):
    """The association of the reference's fp32 sum (tl.sum) is not specified, so single results may
    round to the neighbouring 16-bit value; anything more is a different computation."""
    assert ours.dtype == theirs.dtype and ours.shape == theirs.shape
    diff = ours != theirs
    n = int(diff.sum())
    if n:
        a, b = ours[diff].float(), theirs[diff].float()
        ulp = torch.maximum(a.abs(), b.abs()) * (2.0 ** -7 if ours.dtype == torch.bfloat16 else 2.0 ** -10)
        assert bool(((a - b).abs() <= ulp * 1.01).all()), "pooled values differ by more than one rounding step"
    assert n <= max(2, int(3e-4 * ours.numel())), f"{n} of {ours.numel()} pooled values differ"
    return n


def _compare_selection(va, ref, avg, k, gap, causal, pq, bk, g, chunk_tiles, label):
    """Run both selections chunk by chunk on the same pooled queries; compare as sets."""
    b, h, nq, _ = avg.shape
    hkv, sk = k.shape[1], k.shape[2]
    k_ref = k if hkv == h else k.repeat_interleave(h // hkv, dim=1)  # the reference's callers repeat_kv first
    scale = torch.tensor(1.0 / math.sqrt(128), dtype=torch.float32, device=avg.device)
    qt = (avg.float() * scale).to(avg.dtype)
    lo = pq if causal else 0
    flips = total = 0
    t_ref = t_ours = 0.0
    for t0 in range(0, nq, chunk_tiles):
        a = avg[:, :, t0:t0 + chunk_tiles].contiguous()
        n = a.shape[2]
        cr, ir = ref.select(a, k_ref, t0, gap, causal, pq, bk, wo_initial=causal, group_k_block=g)
        cg, ig = va.fuse_qk_softmax_minp_wo_causal(a, k, t0, gap, causal, pq, bk, wo_initial=causal, group_k_block=g,
                                                   trim=False)
        t_ref += _time_ms(lambda: ref.select(a, k_ref, t0, gap, causal, pq, bk, wo_initial=causal, group_k_block=g), 2)
        t_ours += _time_ms(lambda: va.fuse_qk_softmax_minp_wo_causal(a, k, t0, gap, causal, pq, bk, wo_initial=causal,
                                                                     group_k_block=g, trim=False), 2)
        for bb in range(b):
            for hh in range(h):
                gp = float(gap[bb, hh]) if isinstance(gap, torch.Tensor) else gap
                m_ref = membership(cr[bb, hh], ir[bb, hh], sk)
                m_our = membership(cg[bb, hh], ig[bb, hh], sk)
                total += int(m_ref.sum())
                diff = m_ref ^ m_our
                rows = torch.nonzero(diff.any(dim=1)).flatten()
                for r0 in range(0, rows.numel(), 256):
                    rr = rows[r0:r0 + 256]
                    band = boundary_band(qt[bb, hh, t0:t0 + n][rr], k[bb, hh // (h // hkv)], gp, bk, g, lo)
                    bad = diff[rr] & ~band
                    assert not bool(bad.any()), (
                        f"{label}: head {hh}, tile {t0 + int(rr[torch.nonzero(bad.any(dim=1))[0, 0]])}: "
                        f"{int(bad.sum())} keys differ from the reference away from the boundary")
                flips += int(diff.sum())
        del cr, ir, cg, ig
    assert total > 0
    assert flips <= max(3, int(2e-5 * total)), f"{label}: {flips} boundary keys differ (of {total})"
    print(f"{label}: {total} selected (tile, key) pairs, {flips} differ inside the 1e-6 band; "
          f"selection time reference Triton {t_ref:.3f} ms, CUDA {t_ours:.3f} ms")
    return flips, total


@pytest.mark.parametrize("name", ["c2", "c3", "c4", "c5"])
def test_reference_triton_selection_at_config_sizes(va, ref, name):
    from vecattention_b200.synth import CONFIGS, calibrate_threshold, make_workload
    cfg = CONFIGS[name]
    rep = cfg["heads"] // cfg["kv_heads"]
    wl = make_workload(name, heads=range(0, rep))
    pq, bk, g, causal = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.causal
    ours = va.average_vector(wl.q, pq)
    theirs = ref.average_vector(wl.q, pq, use_triton=True)
    n = _compare_pooling(ours, theirs)
    print(f"{name}: pooled queries: {n} of {ours.numel()} values differ by one rounding step")

    def counts_at(th, hslice):
        cnt, _ = va.fuse_qk_softmax_minp_wo_causal(theirs[:, hslice].contiguous(), wl.k, 0, -math.log(th + 1e-9), causal,
                                                   pq, bk, wo_initial=causal, group_k_block=g, trim=False, capacity=4)
        return cnt
    gap = -math.log(calibrate_threshold(wl, counts_at) + 1e-9)
    _compare_selection(va, ref, theirs, wl.k, gap, causal, pq, bk, g, min(wl.chunk_size, wl.seq_len) // pq, name)


def _rand(shape, seed, dtype):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=gen, device="cuda").to(dtype)


@pytest.mark.parametrize("cfg", [
    dict(h=2, sq=1024, sk=4007, g=8192, causal=False, dtype=torch.bfloat16),   # Sk % 16 != 0: NaN-padded tail block
    dict(h=2, sq=1024, sk=4007, g=16, causal=False, dtype=torch.bfloat16),
    dict(h=2, sq=4288, sk=4288, g=16, causal=True, dtype=torch.bfloat16),      # 67 tiles: two Triton programs, ragged
    dict(h=2, sq=1024, sk=2048, g=4, causal=False, dtype=torch.float16),       # the 16-bit scaling in fp16
    dict(h=3, sq=1024, sk=2048, g=8192, causal=False, dtype=torch.bfloat16, per_head=True),
])
def test_reference_triton_selection_edge_cases(va, ref, cfg):
    dt = cfg["dtype"]
    q = _rand((1, cfg["h"], cfg["sq"], 128), 71, dt)
    k = _rand((1, cfg["h"], cfg["sk"], 128), 72, dt)
    k[:, :, ::41] *= 3.0
    theirs = ref.average_vector(q, 64, use_triton=True)
    _compare_pooling(va.average_vector(q, 64), theirs)
    if cfg.get("per_head"):
        gap = -torch.log(torch.tensor([[0.4, 0.6, 0.8]], device="cuda") + 1e-9)
    else:
        gap = -math.log(0.6 + 1e-9)
    _compare_selection(va, ref, theirs, k, gap, cfg["causal"], 64, 16, cfg["g"], 65536 // 64, str(cfg))


@pytest.mark.parametrize("causal", [False, True])
def test_reference_tuner_recall_and_sparsity(va, ref, causal):
    """The tuner's own ``seg_pr_perHead`` (dense softmax times the selection mask, in the input dtype) against
    the log-sum-exp route of this package.  The reference accumulates in bf16 (per-row recalls, the per-head
    sums and the sparsity), hence the tolerances."""
    from spattn.threshold.model_tuner import seg_pr_perHead
    from vecattention_b200.recall import selection_recall_sparsity
    h, s = 4, 1100
    q = _rand((1, h, s, 128), 91, torch.bfloat16)
    k = _rand((1, h, s, 128), 92, torch.bfloat16)
    k[:, :, ::17] *= 3.0
    thr = torch.tensor([0.3, 0.5, 0.7, 0.9], device="cuda")
    ref_recall, ref_sparsity = seg_pr_perHead(q, k, 64, 16, 16, thr, 512, causal)
    recall, sparsity = selection_recall_sparsity(q, k, 64, 16, 16, thr, 512, causal)
    print(f"causal={causal}: recall reference {ref_recall.float().tolist()} ours {recall.tolist()}; "
          f"sparsity reference {ref_sparsity.float().tolist()} ours {sparsity.tolist()}")
    assert (recall - ref_recall.float()).abs().max() <= 6e-3
    assert (sparsity - ref_sparsity.float()).abs().max() <= 1.5e-2


def test_reference_triton_rmsnorm(va, ref):
    """The reference's Triton RMSNorm (eval/DiTEvalKit/kernels/triton/rmsnorm.py) against the fused kernel's
    norm stage: equal except isolated results on the neighbouring 16-bit value (the sum of squares is
    associated differently)."""
    from eval.DiTEvalKit.kernels.triton.rmsnorm import triton_rmsnorm_forward
    from vecattention_b200.preattn import qk_norm_rope
    heads, s = 40, 777
    x = _rand((1, s, heads * 128), 95, torch.bfloat16)
    w = (1 + 0.1 * _rand((heads * 128,), 96, torch.float32)).to(torch.bfloat16)
    theirs = triton_rmsnorm_forward(x, w, 1e-6)
    theirs = theirs[0] if isinstance(theirs, tuple) else theirs
    ours, _ = qk_norm_rope(x, x, w, w, 1e-6, heads=heads)
    ours = ours.transpose(1, 2).reshape(1, s, heads * 128)
    diff = ours != theirs
    print(f"rmsnorm: {int(diff.sum())} of {ours.numel()} values differ from the reference Triton kernel")
    assert diff.float().mean() <= 2e-3
    step = theirs.float().abs().clamp_min(1e-3) * 2.0 ** -7
    assert bool(((ours.float() - theirs.float()).abs() <= 1.01 * step).all())
