"""Parity of the CUDA path (through the C ABI, via the Python host mirror) against the CPU
oracle on the same seeded inputs.  Needs a B200: run with ``-m gpu``.

Bars: pooling bit-exact; selected index sets identical except keys whose estimate lies within
1e-6 (relative to the magnitudes compared) of the keep/drop boundary; attention outputs within
max-abs 2e-2 and mean-abs 2e-3 in bf16 of the fp32 oracle.
"""
import math

import numpy as np
import pytest
import torch

import cases as C
from oracle import vecattn_oracle as O
from parity_util import MAX_ABS, MEAN_ABS, check_selection

pytestmark = pytest.mark.gpu



@pytest.fixture(scope="module")
def va(built_library):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import vecattention_b200 as va_mod
    return va_mod


def _rand(shape, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,pq", [((1, 2, 1008, 128), 64), ((2, 3, 384, 128), 128), ((1, 1, 50, 128), 64),
                                      ((1, 4, 2048, 128), 64)])
def test_pool_bit_exact(va, dtype, shape, pq):
    q = _rand(shape, 1, dtype)
    ref = O.pool_q(q, pq)
    out = va.average_vector(q.cuda(), pq)
    assert out.dtype == dtype and tuple(out.shape) == tuple(ref.shape)
    assert torch.equal(out.cpu(), ref)


def test_pool_strided_input(va):
    # (B,S,H,D) storage viewed as (B,H,S,D): addressed in place through the strides
    q = _rand((2, 640, 3, 128), 2, torch.bfloat16)
    out = va.average_vector(q.cuda().transpose(1, 2), 64)
    assert torch.equal(out.cpu(), O.pool_q(q.transpose(1, 2).contiguous(), 64))


# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["c1_g8192", "c1_g16", "ragged_nc", "ragged_causal", "sq_ne_sk_p128", "per_head",
                                  "fp16_nc", "causal_q1"])
def test_select_parity_golden_inputs(va, name):
    """The golden cases' seeded inputs in 16-bit: CUDA selection == oracle selection."""
    p = C.CASES[name]
    dt = torch.float16 if p["dtype"] == "fp16" else torch.bfloat16
    q, k, _ = C.make_inputs(p)
    q, k = q.to(dt), k.to(dt)
    g = np.load(f"{__import__('os').path.dirname(__file__)}/golden/{name}.npz")
    gap = g["gap"]
    gap = torch.from_numpy(gap).float() if gap.ndim else float(gap)
    avg = O.pool_q(q, p["pq"])
    cr, ir, amb = O.select_columns(avg, k, 0, gap, p["causal"], p["pq"], p["bk"], wo_initial=p["causal"],
                                   group_k_block=p["g"], return_ambiguous=True)
    gap_dev = gap.cuda() if isinstance(gap, torch.Tensor) else gap
    cg, ig = va.fuse_qk_softmax_minp_wo_causal(avg.cuda(), k.cuda(), 0, gap_dev, p["causal"], p["pq"], p["bk"],
                                               wo_initial=p["causal"], group_k_block=p["g"])
    check_selection(cg, ig, cr, ir, amb, p["h"], p["sk"])
    assert int(cr.sum()) > 0


@pytest.mark.parametrize("cfg", [
    dict(h=4, hkv=2, sq=768, sk=768, pq=64, bk=16, g=4, causal=True, toff=0, th=0.5),       # GQA causal
    dict(h=2, hkv=2, sq=512, sk=1000, pq=64, bk=16, g=8192, causal=False, toff=0, th=0.6),  # Sk % Bk != 0
    dict(h=2, hkv=1, sq=512, sk=1536, pq=128, bk=32, g=3, causal=False, toff=0, th=0.55),
    dict(h=1, hkv=1, sq=384, sk=2048, pq=64, bk=64, g=2, causal=False, toff=0, th=0.5),
    dict(h=1, hkv=1, sq=256, sk=2048, pq=128, bk=128, g=1, causal=False, toff=0, th=0.5),
    dict(h=2, hkv=2, sq=1536, sk=1536, pq=128, bk=128, g=1, causal=True, toff=0, th=0.5),   # the reference's default sizes
    dict(h=2, hkv=1, sq=1100, sk=1100, pq=128, bk=128, g=3, causal=True, toff=0, th=0.6),   # ragged, groups of 3 blocks
    dict(h=2, hkv=2, sq=1280, sk=1280, pq=128, bk=64, g=2, causal=True, toff=0, th=0.5),
    dict(h=2, hkv=2, sq=512, sk=2048, pq=64, bk=16, g=16, causal=True, toff=24, th=0.4),    # a later chunk
    dict(h=6, hkv=2, sq=4480, sk=4480, pq=64, bk=16, g=16, causal=True, toff=0, th=0.7),     # rows span CTAs/heads
])
def test_select_parity_more_shapes(va, cfg):
    q = _rand((1, cfg["h"], cfg["sq"], 128), 31, torch.bfloat16)
    k = _rand((1, cfg["hkv"], cfg["sk"], 128), 32, torch.bfloat16)
    k[:, :, ::37] *= 3.0
    gap = -math.log(cfg["th"] + 1e-9)
    avg = O.pool_q(q, cfg["pq"])
    kw = dict(wo_initial=cfg["causal"], group_k_block=cfg["g"])
    cr, ir, amb = O.select_columns(avg, k, cfg["toff"], gap, cfg["causal"], cfg["pq"], cfg["bk"],
                                   return_ambiguous=True, **kw)
    cg, ig = va.fuse_qk_softmax_minp_wo_causal(avg.cuda(), k.cuda(), cfg["toff"], gap, cfg["causal"], cfg["pq"],
                                               cfg["bk"], **kw)
    check_selection(cg, ig, cr, ir, amb, cfg["h"], cfg["sk"])
    # strict causal rule (no truncating-division quirk)
    if cfg["causal"]:
        cr2, ir2, amb2 = O.select_columns(avg, k, cfg["toff"], gap, True, cfg["pq"], cfg["bk"], compat_q1=False,
                                          return_ambiguous=True, **kw)
        cg2, ig2 = va.fuse_qk_softmax_minp_wo_causal(avg.cuda(), k.cuda(), cfg["toff"], gap, True, cfg["pq"],
                                                     cfg["bk"], compat_q1=False, **kw)
        check_selection(cg2, ig2, cr2, ir2, amb2, cfg["h"], cfg["sk"])


def test_select_capacity_overflow_is_reported(va):
    q = _rand((1, 1, 256, 128), 5, torch.bfloat16)
    k = _rand((1, 1, 1024, 128), 6, torch.bfloat16)
    avg = O.pool_q(q, 64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gap = 50.0  # keeps everything
    cnt, idx = va.fuse_qk_softmax_minp_wo_causal(avg.cuda(), k.cuda(), 0, gap, False, 64, 16, group_k_block=8192,
                                                 trim=False, capacity=100, status=status)
    assert int(status.item()) & 1
    assert torch.all(cnt == 1024)                      # counts stay exact
    assert torch.equal(idx[0, 0, 0].cpu(), torch.arange(100, dtype=torch.int32))


# ------------------------------------------------------------------------------------------------
ATTN_CASES = [
    dict(b=1, h=2, hkv=2, sq=512, sk=512, pq=64, causal=False, bk=16, g=8192, th=0.5),
    dict(b=2, h=2, hkv=2, sq=384, sk=1000, pq=128, causal=False, bk=16, g=4, th=0.6),
    dict(b=1, h=4, hkv=2, sq=1008, sk=1008, pq=64, causal=True, bk=16, g=16, th=0.5),
    dict(b=1, h=2, hkv=1, sq=1200, sk=1200, pq=128, causal=True, bk=32, g=16, th=0.4),
    dict(b=1, h=1, hkv=1, sq=50, sk=50, pq=64, causal=True, bk=16, g=16, th=0.5),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", ATTN_CASES)
def test_sparse_attention_parity(va, cfg, dtype):
    q = _rand((cfg["b"], cfg["h"], cfg["sq"], 128), 41, dtype)
    k = _rand((cfg["b"], cfg["hkv"], cfg["sk"], 128), 42, dtype)
    v = _rand((cfg["b"], cfg["hkv"], cfg["sk"], 128), 43, dtype)
    k[:, :, ::29] *= 3.0
    avg = O.pool_q(q, cfg["pq"])
    gap = -math.log(cfg["th"] + 1e-9)
    cc, ci = O.select_columns(avg, k, 0, gap, cfg["causal"], cfg["pq"], cfg["bk"], wo_initial=cfg["causal"],
                              group_k_block=cfg["g"])
    bc, bi = O.block_tables(cfg["b"], cfg["h"], cfg["sq"], cfg["pq"], cfg["causal"])
    ref = O.sparse_attention(q, k, v, cfg["pq"], bc, bi, cc, ci, cfg["causal"], out_dtype=torch.float32)
    # the reference's calling convention: (B,S,H,D) tensors
    out = va.sparse_attn_func(q.cuda().transpose(1, 2).contiguous(), k.cuda().transpose(1, 2).contiguous(),
                              v.cuda().transpose(1, 2).contiguous(), cfg["pq"], bc.cuda(), bi.cuda(), cc.cuda(),
                              ci.cuda(), causal=cfg["causal"])
    assert tuple(out.shape) == (cfg["b"], cfg["sq"], cfg["h"], 128)
    err = (out.transpose(1, 2).float().cpu() - ref).abs()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max().item(), err.mean().item())
    # block tables built on the device equal the reference construction
    bcg, big = va.block_tables(cfg["b"], cfg["h"], cfg["sq"], cfg["pq"], cfg["causal"], "cuda")
    assert torch.equal(bcg.cpu(), bc) and torch.equal(big.cpu(), bi)


def test_sparse_attention_empty_tile_gives_zeros(va):
    q = _rand((1, 1, 128, 128), 1, torch.bfloat16).cuda()
    k = _rand((1, 1, 256, 128), 2, torch.bfloat16).cuda()
    v = _rand((1, 1, 256, 128), 3, torch.bfloat16).cuda()
    cc = torch.tensor([[[0, 3]]], dtype=torch.int32, device="cuda")
    ci = torch.tensor([[[[0, 0, 0], [5, 17, 200]]]], dtype=torch.int32, device="cuda")
    out = va.sparse_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), 64, None, None, cc, ci,
                              causal=False).transpose(1, 2)
    assert torch.all(out[0, 0, :64] == 0)
    ref = O.sparse_attention(q.cpu(), k.cpu(), v.cpu(), 64, torch.zeros(1, 1, 2, dtype=torch.int32),
                             torch.zeros(1, 1, 2, 1, dtype=torch.int32), cc.cpu(), ci.cpu(), False,
                             out_dtype=torch.float32)
    assert (out.float().cpu() - ref).abs().max() <= MAX_ABS


# ------------------------------------------------------------------------------------------------
PREFILL_CASES = [
    dict(b=1, h=4, hkv=4, s=2048, pq=64, bk=16, g=8192, causal=False, chunk=1024, th=0.55),
    dict(b=1, h=2, hkv=2, s=1200, pq=64, bk=16, g=16, causal=True, chunk=512, th=0.5),
    dict(b=2, h=4, hkv=2, s=1008, pq=128, bk=32, g=4, causal=True, chunk=16384, th=0.6),
    dict(b=1, h=3, hkv=3, s=640, pq=64, bk=16, g=2, causal=False, chunk=256, th=(0.3, 0.5, 0.7)),
    dict(b=1, h=2, hkv=2, s=1500, pq=128, bk=128, g=1, causal=True, chunk=16384, th=0.5),  # the reference's defaults
]


@pytest.mark.parametrize("cfg", PREFILL_CASES)
def test_prefill_matches_oracle(va, cfg):
    q = _rand((cfg["b"], cfg["h"], cfg["s"], 128), 51, torch.bfloat16)
    k = _rand((cfg["b"], cfg["hkv"], cfg["s"], 128), 52, torch.bfloat16)
    v = _rand((cfg["b"], cfg["hkv"], cfg["s"], 128), 53, torch.bfloat16)
    k[:, :, ::31] *= 3.0
    th = torch.tensor(cfg["th"], dtype=torch.float32) if isinstance(cfg["th"], tuple) else cfg["th"]
    ref, sel = O.vecattention_prefill(q, k, v, th, cfg["pq"], cfg["bk"], cfg["g"], cfg["causal"], cfg["chunk"],
                                      return_selection=True)
    th_dev = th.cuda() if isinstance(th, torch.Tensor) else th
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, counts = va.VecAttention_prefill(q.cuda(), k.cuda(), v.cuda(), th_dev, cfg["pq"], cfg["bk"], cfg["g"],
                                          cfg["causal"], cfg["chunk"], return_selection=True, status=status)
    assert int(status.item()) == 0, "a kernel reported overflow or an internal timeout"
    ref_counts = torch.cat([c for c, _ in sel], dim=2)
    # a boundary key may flip a count by one; anything else is a bug
    assert (counts.cpu() - ref_counts).abs().sum() <= 2
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max().item(), err.mean().item())
    # dense-attention error of both implementations (reported, not asserted tightly)
    dense = O.dense_attention(q, k, v, cfg["causal"])
    e_ref = (ref.float() - dense).abs().mean().item()
    e_gpu = (out.float().cpu() - dense).abs().mean().item()
    print(f"mean |sparse - dense|: oracle {e_ref:.4e}  cuda {e_gpu:.4e}")
    assert abs(e_ref - e_gpu) <= MEAN_ABS


def test_prefill_error_behaviour(va):
    q = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):   # spattn/src/VecAttention.py:43
        va.VecAttention_prefill(q, q, q, 0.5, 64, 16, 16, False, chunk_size=100)
    with pytest.raises(AssertionError):   # :44
        va.VecAttention_prefill(q, q, q, 0.5, 32, 16, 16, False, chunk_size=1024)
    with pytest.raises(AssertionError):   # vecattention_kernels.py:129
        va.VecAttention_prefill(q, q, q, 0.5, 64, 128, 16, True, chunk_size=1024)
    with pytest.raises(RuntimeError):
        va.VecAttention_prefill(q.cpu(), q.cpu(), q.cpu(), 0.5, 64, 16, 16, False, chunk_size=1024)
    with pytest.raises((AssertionError, ValueError)):
        va.VecAttention_prefill(q.float(), q.float(), q.float(), 0.5, 64, 16, 16, False, chunk_size=1024)


# ------------------------------------------------------------------------------------------------
# Size-independent properties at benchmark-like sizes (the oracle would take minutes there)
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def big(va):
    from vecattention_b200.synth import make_workload
    return make_workload("c2", heads=range(0, 2))


def test_property_keep_everything_equals_dense(va, big):
    """With a vanishing threshold every key is selected, so the operator must equal dense
    attention (checked against torch's scaled_dot_product_attention on the same GPU)."""
    q, k, v = big.q[:, :, :8192], big.k[:, :, :8192], big.v[:, :, :8192]
    out, counts = va.VecAttention_prefill(q, k, v, 1e-30, 64, 16, 16, False, 32768, return_selection=True)
    assert torch.all(counts == 8192)
    dense = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    err = (out.float() - dense.float()).abs()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS


def test_property_selection_lists_sorted_unique_in_range_and_deterministic(va, big):
    avg = va.average_vector(big.q, 64)
    gap = -math.log(0.5)
    c1, i1 = va.fuse_qk_softmax_minp_wo_causal(avg, big.k, 0, gap, False, 64, 16, group_k_block=16, trim=False)
    c2, i2 = va.fuse_qk_softmax_minp_wo_causal(avg, big.k, 0, gap, False, 64, 16, group_k_block=16, trim=False)
    assert torch.equal(c1, c2)
    pos = torch.arange(i1.shape[-1], device="cuda").view(1, 1, 1, -1)
    valid = pos < c1.unsqueeze(-1)
    assert torch.equal(torch.where(valid, i1, 0), torch.where(valid, i2, 0))
    inc = (i1[..., 1:] > i1[..., :-1]) | ~valid[..., 1:]
    assert bool(inc.all())
    assert bool(((i1 >= 0) & (i1 < big.seq_len) | ~valid).all())
    # every 256-key group has at least its own maximum kept
    assert int(c1.min()) >= big.seq_len // 256


def test_property_chunk_size_does_not_change_noncausal_results(va, big):
    a = va.VecAttention_prefill(big.q, big.k, big.v, 0.6, 64, 16, 16, False, 32768)
    b = va.VecAttention_prefill(big.q, big.k, big.v, 0.6, 64, 16, 16, False, 4096)
    assert torch.equal(a, b)


def test_property_linear_in_v(va, big):
    q, k = big.q[:, :, :4096], big.k
    v1, v2 = big.v, torch.roll(big.v, 1, dims=2)
    o1 = va.VecAttention_prefill(q, k, v1, 0.6, 64, 16, 8192, False, 4096).float()
    o2 = va.VecAttention_prefill(q, k, v2, 0.6, 64, 16, 8192, False, 4096).float()
    o12 = va.VecAttention_prefill(q, k, (v1.float() + v2.float()).to(v1.dtype), 0.6, 64, 16, 8192, False, 4096).float()
    assert (o12 - (o1 + o2)).abs().max() <= 2 * MAX_ABS


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("slices", [1, 2, 5])
def test_host_buffer_pipeline_equals_device_call(va, slices, pinned):
    """VecAttention_prefill_host (host q/k/v, head slices pipelined over three streams) gives the
    bits of one device call on all heads: GQA, per-head thresholds, causal, two calls in a row
    sharing the staging buffers."""
    from vecattention_b200.hostio import VecAttention_prefill_host
    b, h, hkv, s = 1, 12, 4, 1500
    staging = {}
    for seed in (5, 6):
        q = _rand((b, h, s, 128), seed, torch.bfloat16)
        k = _rand((b, hkv, s, 128), seed + 10, torch.bfloat16)
        v = _rand((b, hkv, s, 128), seed + 20, torch.bfloat16)
        k[:, :, ::23] *= 3.0
        thr = torch.linspace(0.5, 0.9, h)
        ref = va.VecAttention_prefill(q.cuda(), k.cuda(), v.cuda(), thr.cuda(), 64, 16, 16, True, 512)
        hq, hk, hv = (t.pin_memory() if pinned else t for t in (q, k, v))
        got = VecAttention_prefill_host(hq, hk, hv, thr, 64, 16, 16, True, 512, slices=slices, staging=staging)
        assert not got.is_cuda and got.shape == q.shape
        assert torch.equal(got, ref.cpu())
    with pytest.raises(ValueError):
        VecAttention_prefill_host(q.cuda(), k, v, 0.5, 64, 16, 16, True, 512)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("vs,ve", [(37, 1900), (None, 1500), (200, None), (0, 2048), (64, 64), (130, 131), (1000, 1087)])
def test_vision_slice_composition_matches_oracle(va, vs, ve):
    """Dense text prefix / VecAttention up to the end of the vision span / dense text suffix
    (the reference dispatcher's composition), GQA, positions that are not tile multiples; the
    one-launch form and the three-launch form give the same bits."""
    b, h, hkv, s = 1, 4, 2, 2048
    q = _rand((b, h, s, 128), 31, torch.bfloat16)
    k = _rand((b, hkv, s, 128), 32, torch.bfloat16)
    v = _rand((b, hkv, s, 128), 33, torch.bfloat16)
    k[:, :, ::29] *= 3.0
    ref = O.vecattention_prefill_vision(q, k, v, 0.7, 64, 16, 16, 1024, vs, ve).float()
    got = va.VecAttention_prefill_vision(q.cuda(), k.cuda(), v.cuda(), 0.7, 64, 16, 16, True, 1024,
                                         vision_start_position=vs, vision_end_position=ve).float().cpu()
    three = va.VecAttention_prefill_vision(q.cuda(), k.cuda(), v.cuda(), 0.7, 64, 16, 16, True, 1024,
                                           vision_start_position=vs, vision_end_position=ve, fused=False).float().cpu()
    assert torch.equal(got, three), "one launch and three launches must agree bit for bit"
    err = (got - ref).abs()
    assert torch.isfinite(got).all()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max().item(), err.mean().item())
    with pytest.raises(ValueError):
        va.VecAttention_prefill_vision(q.cuda(), k.cuda(), v.cuda(), 0.7, 64, 16, 16, False, 1024, vision_start_position=3)


# ---------------------------------------------------------------------------------------------
def test_softmax_lse_output(va):
    """return_softmax_lse of the sparse attention entry point: log-sum-exp of the scaled scores over
    the keys each row visits; with every key listed it equals the dense value."""
    b, h, hkv, s = 1, 4, 2, 700
    q = _rand((b, s, h, 128), 41, torch.bfloat16).cuda()
    k = _rand((b, s, hkv, 128), 42, torch.bfloat16).cuda()
    v = _rand((b, s, hkv, 128), 43, torch.bfloat16).cuda()
    for pq in (64, 128):
        nq = math.ceil(s / pq)
        cnt = torch.full((b, h, nq), s, dtype=torch.int32, device="cuda")
        idx = torch.arange(s, dtype=torch.int32, device="cuda").expand(b, h, nq, s).contiguous()
        out, lse = va.sparse_attn_func(q, k, v, pq, None, None, cnt, idx, return_softmax_lse=True, causal=False)
        kk = k.float().repeat_interleave(h // hkv, dim=2)
        ref = torch.logsumexp(torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) / math.sqrt(128), dim=-1)
        assert lse.shape == (b, h, s) and lse.dtype == torch.float32
        assert (lse - ref).abs().max() <= 2e-3, (pq, (lse - ref).abs().max().item())


@pytest.mark.parametrize("causal", [False, True])
def test_selection_recall_and_sparsity_match_the_tuner_rule(va, causal):
    from vecattention_b200.recall import selection_recall_sparsity
    b, h, hkv, s = 1, 4, 4, 1100
    q = _rand((b, h, s, 128), 61, torch.bfloat16)
    k = _rand((b, hkv, s, 128), 62, torch.bfloat16)
    k[:, :, ::17] *= 3.0
    thr = torch.tensor([0.3, 0.5, 0.7, 0.9])
    ref_recall, ref_sparsity = O.seg_pr_per_head(q, k, 64, 16, 16, thr, 512, causal)
    recall, sparsity = selection_recall_sparsity(q.cuda(), k.cuda(), 64, 16, 16, thr.cuda(), 512, causal)
    assert recall.shape == (h,) and sparsity.shape == (h,)
    assert (recall.cpu().double() - ref_recall).abs().max() <= 2e-3, (recall, ref_recall)
    assert (sparsity.cpu().double() - ref_sparsity).abs().max() <= 1e-3, (sparsity, ref_sparsity)
    assert (recall.cpu()[1:] <= recall.cpu()[:-1] + 1e-3).all()  # a higher threshold keeps less mass


# ---------------------------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_the_context_stays_usable(va):
    """A wait that nothing completes gives up after its poll limit, the kernel returns normally
    with VA_STATUS_TIMEOUT in the status word, and the next ordinary launch is correct."""
    import ctypes as C
    from vecattention_b200 import _lib as L
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.lib().va_selftest_wait_timeout(status.data_ptr(), 200, stream) == 0
    torch.cuda.synchronize()                         # returns: the wait was bounded
    assert int(status.item()) == L.VA_STATUS_TIMEOUT
    q = _rand((1, 2, 1008, 128), 1, torch.bfloat16)
    assert torch.equal(va.average_vector(q.cuda(), 64).cpu(), O.pool_q(q, 64))
    status.zero_()
    k = _rand((1, 2, 1008, 128), 2, torch.bfloat16)
    out = va.VecAttention_prefill(q.cuda(), k.cuda(), k.cuda(), 0.5, 64, 16, 16, False, 512, status=status)
    ref = O.vecattention_prefill(q, k, k, 0.5, 64, 16, 16, False, 512)
    assert int(status.item()) == 0
    assert (out.float().cpu() - ref.float()).abs().max() <= MAX_ABS


# ---------------------------------------------------------------------------------------------
def test_dispatcher_with_config(va, tmp_path):
    """customize_prefill_attention: per-layer threshold tensor, vision positions from the configuration, the
    dense method on the same kernel, the latency record and the Q/K dump."""
    import types
    from vecattention_b200.dispatch import SPARSITY_RECORD
    b, h, hkv, s = 1, 4, 2, 1500
    q = _rand((b, h, s, 128), 81, torch.bfloat16).cuda()
    k = _rand((b, hkv, s, 128), 82, torch.bfloat16).cuda()
    v = _rand((b, hkv, s, 128), 83, torch.bfloat16).cuda()
    layer = types.SimpleNamespace(layer_idx=1)
    thr = torch.tensor([[0.3] * h, [0.6, 0.7, 0.8, 0.9], [0.9] * h], device="cuda")   # (layers, heads)
    cfg = va.FastPrefillConfig(metric="vecattention", threshold=thr, group_k_block=16, chunk_size=1024,
                               vision_start_position=100, vision_end_position=1300, dump_qk_dir=str(tmp_path))
    SPARSITY_RECORD.attention_latency_list = []
    got = va.customize_prefill_attention(layer, q, k, v, config=cfg)
    want = va.VecAttention_prefill_vision(q, k, v, thr[1], 64, 16, 16, True, 1024, vision_start_position=100,
                                          vision_end_position=1300)
    assert torch.equal(got, want)
    one = va.VecAttention_prefill(q, k, v, torch.tensor(0.7, device="cuda"), 64, 16, 16, True, 1024)   # a 0-d tensor
    assert torch.equal(one, va.VecAttention_prefill(q, k, v, torch.full((h,), 0.7, device="cuda"), 64, 16, 16, True, 1024))
    assert len(SPARSITY_RECORD.attention_latency_list) == 1
    torch.cuda.synchronize()
    e0, e1 = SPARSITY_RECORD.attention_latency_list[0]
    assert e0.elapsed_time(e1) > 0
    assert (tmp_path / "input" / "layer_1_qk.pt").exists()
    kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
    for causal in (True, False):
        dense = va.customize_prefill_attention(layer, q, k, v, causal=causal, config=va.FastPrefillConfig(metric="full"))
        ref = torch.nn.functional.scaled_dot_product_attention(q, kk, vv, is_causal=causal)
        err = (dense.float() - ref.float()).abs()
        assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (causal, err.max().item())
    with pytest.raises(NotImplementedError):
        va.customize_prefill_attention(layer, q, k, v, config=va.FastPrefillConfig(metric="anchor"))
    with pytest.raises(AssertionError):
        va.customize_prefill_attention(layer, q, k, v, causal=False, config=va.FastPrefillConfig(metric="flex"))
