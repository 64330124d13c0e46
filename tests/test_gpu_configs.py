"""Parity against the CPU oracle at the sizes of the benchmark configurations 2-5 (32 K, 75.6 K,
118.8 K tokens non-causal; 64 K tokens causal with 7:1 grouped-query heads).  Needs a B200.

One KV group of each configuration is generated on the GPU at full sequence length and copied to
the host, so that both sides see the same bits.  The CUDA path runs all query tiles; the oracle
runs a sample of them (the first tiles, the tiles around every prefill-chunk boundary, the rows
where the reference's causal quirk applies, the ragged last tile and a seeded random rest):

  * pooled queries of the sampled tiles: bit-exact;
  * selected index sets of the sampled tiles: identical except keys whose estimate lies within
    1e-6 of the keep/drop boundary;
  * attention outputs of the sampled tiles, computed from the CUDA path's own selection: within
    max-abs 2e-2 / mean-abs 2e-3 of the fp32 oracle;
  * the staged calls (pool, select, attention) and the whole operator agree bit for bit;
  * the dense-attention error of both implementations on the sampled tiles is printed.
"""
import math

import numpy as np
import pytest
import torch

from oracle import vecattn_oracle as O
from parity_util import MAX_ABS, MEAN_ABS, check_selection

pytestmark = pytest.mark.gpu

N_SAMPLES = 64


@pytest.fixture(scope="module")
def va(built_library):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import vecattention_b200 as va_mod
    return va_mod


def _sample_tiles(nq, chunk_tiles, causal, seed):
    fixed = {0, 1, 2, nq - 2, nq - 1}
    for c in range(chunk_tiles, nq, chunk_tiles):      # last tile of a chunk, first two of the next
        fixed |= {c - 1, c, c + 1}
    if causal:                                         # rows that lose 48 keys to the truncating division
        fixed |= {64, 65, 128, 960, 63}
    fixed = {t for t in fixed if 0 <= t < nq}
    rng = np.random.default_rng(seed)
    rest = [t for t in rng.permutation(nq).tolist() if t not in fixed]
    return sorted(fixed | set(rest[: max(0, N_SAMPLES - len(fixed))]))


@pytest.mark.parametrize("name", ["c2", "c3", "c4", "c5"])
def test_config_sampled_tiles_match_oracle(va, name):
    from vecattention_b200 import api
    from vecattention_b200.synth import CONFIGS, calibrate_threshold, make_workload
    cfg = CONFIGS[name]
    rep = cfg["heads"] // cfg["kv_heads"]
    wl = make_workload(name, heads=range(0, rep))       # one KV group, all tokens
    pq, bk, g, chunk, causal, s = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.chunk_size, wl.causal, wl.seq_len
    nq = wl.nq

    # ---- CUDA path, all tiles ----
    avg = va.average_vector(wl.q, pq)

    def counts_at(th, hslice):
        cnt, _ = va.fuse_qk_softmax_minp_wo_causal(avg[:, hslice].contiguous(), wl.k, 0, -math.log(th + 1e-9), causal, pq, bk,
                                                   wo_initial=causal, group_k_block=g, trim=False, capacity=4)
        return cnt
    thr = calibrate_threshold(wl, counts_at)
    gap = -math.log(thr + 1e-9)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the operator runs the selection per prefill chunk (the causal quirk restarts at chunk boundaries)
    chunk_tiles = min(chunk, s) // pq
    cnt_parts, idx_parts = [], []
    for t0 in range(0, nq, chunk_tiles):
        c, i = va.fuse_qk_softmax_minp_wo_causal(avg[:, :, t0:t0 + chunk_tiles].contiguous(), wl.k, t0, gap, causal, pq, bk,
                                                 wo_initial=causal, group_k_block=g, trim=False, status=status)
        cnt_parts.append(c)
        idx_parts.append(i)
    cnt = torch.cat(cnt_parts, dim=2)
    idx = torch.cat(idx_parts, dim=2)
    del cnt_parts, idx_parts
    bc, bi = va.block_tables(1, rep, s, pq, causal, "cuda")
    out = api._sparse_attn_bhsd(wl.q, wl.k, wl.v, pq, bc, bi, cnt, idx, causal, status=status)
    out_op, cnt_op = va.VecAttention_prefill(wl.q, wl.k, wl.v, thr, pq, bk, g, causal, chunk, return_selection=True,
                                             status=status)
    assert int(status.item()) == 0, "a kernel reported overflow or an internal timeout"
    assert torch.equal(cnt_op, cnt), "operator and staged selection counts differ"
    assert torch.equal(out_op, out), "operator and staged calls differ"
    kept = float(cnt.sum()) / (wl.eligible_pairs_per_head() * rep)
    assert abs(kept - wl.keep) < 0.02, kept

    # ---- the same bits on the host; oracle on the sampled tiles ----
    tiles = _sample_tiles(nq, chunk_tiles, causal, seed=11)
    q_h, k_h, v_h = wl.q.cpu(), wl.k.cpu(), wl.v.cpu()
    avg_h = torch.stack([O.pool_q(q_h[:, :, t * pq:(t + 1) * pq], pq)[:, :, 0] for t in tiles], dim=2)
    assert torch.equal(avg[:, :, tiles].cpu(), avg_h), "pooled queries differ"

    flips = total = 0
    for t0 in range(0, nq, chunk_tiles):
        sel = [t for t in tiles if t0 <= t < t0 + chunk_tiles]
        if not sel:
            continue
        pos = [tiles.index(t) for t in sel]
        cr, ir, amb = O.select_columns(avg_h[:, :, pos], k_h, t0, gap, causal, pq, bk, wo_initial=causal, group_k_block=g,
                                       return_ambiguous=True, rows=[t - t0 for t in sel])
        f, n = check_selection(cnt[:, :, sel], idx[:, :, sel], cr, ir, amb, rep, s)
        flips += f
        total += n
    print(f"{name}: threshold {thr:.4f}, kept {kept:.4f}; {len(tiles)} sampled tiles x {rep} heads: "
          f"{flips} boundary keys differ of {total}")

    ci_h = idx[:, :, tiles].cpu()
    cc_h = cnt[:, :, tiles].cpu()
    # tables of the sampled tiles placed at their own tile index, so that the oracle can be asked for those tiles only
    cc_full = torch.zeros(1, rep, nq, dtype=torch.int32)
    ci_full = torch.zeros(1, rep, nq, int(cc_h.max()), dtype=torch.int32)
    cc_full[:, :, tiles] = cc_h
    ci_full[:, :, tiles] = ci_h[..., : ci_full.shape[-1]]
    ref = O.sparse_attention(q_h, k_h, v_h, pq, bc.cpu(), bi.cpu(), cc_full, ci_full, causal, out_dtype=torch.float32,
                             tiles=tiles)
    rows = torch.cat([torch.arange(t * pq, min((t + 1) * pq, s)) for t in tiles])
    got = out[:, :, rows].float().cpu()
    err = (got - ref[:, :, rows]).abs()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max().item(), err.mean().item())

    # dense-attention error of both implementations on a few of the sampled tiles (reported)
    few = tiles[:: max(1, len(tiles) // 8)]
    e_ref, e_gpu, n = 0.0, 0.0, 0
    for t in few:
        r0, r1 = t * pq, min((t + 1) * pq, s)
        kk = k_h[:, :, :r1] if causal else k_h
        vv = v_h[:, :, :r1] if causal else v_h
        dense = O.dense_attention(q_h[:, :, r0:r1], kk, vv, causal, q_offset=r0)
        e_ref += (ref[:, :, r0:r1] - dense).abs().sum().item()
        e_gpu += (out[:, :, r0:r1].float().cpu() - dense).abs().sum().item()
        n += dense.numel()
    print(f"{name}: max|cuda - oracle| {err.max():.3e}, mean {err.mean():.3e}; "
          f"mean|sparse - dense| oracle {e_ref / n:.4e}, cuda {e_gpu / n:.4e}")
    assert abs(e_ref - e_gpu) / n <= MEAN_ABS


@pytest.mark.parametrize("causal,heads,kv_heads,nq,sk", [(False, 20, 20, 1024, 16384), (True, 12, 4, 256, 16384)])
def test_selection_launch_schedules_agree(va, causal, heads, kv_heads, nq, sk):
    """The selection kernel's grid depends on how many CTAs a launch has: key segments for few CTAs, the last
    partial wave of equally long walks cut into segments, causal row blocks of all heads handed out longest walk
    first.  One launch over all heads and one launch per KV group take different schedules and must produce the
    same lists (the per-group form is the one the oracle and the reference's kernels are compared with)."""
    from parity_util import membership
    g = torch.Generator(device="cuda").manual_seed(17)
    avg = torch.randn(1, heads, nq, 128, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(1, kv_heads, sk, 128, generator=g, device="cuda").to(torch.bfloat16)
    k[:, :, ::37] *= 3.0
    gap = -math.log(0.6)
    rep = heads // kv_heads
    kw = dict(wo_initial=causal, group_k_block=8192, trim=False)
    cnt_all, idx_all = va.fuse_qk_softmax_minp_wo_causal(avg, k, 0, gap, causal, 64, 16, **kw)
    assert int(cnt_all.sum()) > 0
    for kv in range(kv_heads):
        hs = slice(kv * rep, (kv + 1) * rep)
        cnt_g, idx_g = va.fuse_qk_softmax_minp_wo_causal(avg[:, hs].contiguous(), k[:, kv:kv + 1].contiguous(), 0, gap, causal,
                                                         64, 16, **kw)
        assert torch.equal(cnt_all[:, hs], cnt_g), f"KV group {kv}: counts differ between the two schedules"
        a = membership(cnt_all[0, hs].reshape(-1), idx_all[0, hs].reshape(rep * nq, -1), sk)
        b = membership(cnt_g[0].reshape(-1), idx_g[0].reshape(rep * nq, -1), sk)
        assert torch.equal(a, b), f"KV group {kv}: selected keys differ between the two schedules"
