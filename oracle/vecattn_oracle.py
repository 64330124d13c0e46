"""CPU oracle for the VecAttention prefill path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with plain PyTorch/NumPy tensor arithmetic, what the
reference computes on the path ``VecAttention_prefill`` -> ``average_vector`` ->
``fuse_qk_softmax_minp_wo_causal`` -> ``sparse_attn_func``.  It is the checker for the
CUDA kernels; nothing in the product package imports it.  Only the tests, the smoke
check and the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may call it.

Parity status
-------------
* Pooling and selection (``pool_q``, ``select_columns``, ``block_tables``): PINNED.  The
  committed fixtures under ``tests/golden/`` were produced by importing the reference's own
  ``average_vector`` and ``fuse_qk_softmax_minp_wo_causal`` (Triton kernels executed by the
  Triton CPU interpreter, fp32 inputs) and ``tests/test_oracle_golden.py`` checks this
  file against them.
* Sparse attention (``sparse_attention``): PARITY UNPINNED.  The reference calls
  ``vllm_flash_attn.sparse_attn_func`` from the package ``vllm-flash-attn 2.7.2.post1``
  (fork ``anminliu/vllm-flash-attention``, un-vendored git submodule, commit not recorded);
  its source is not part of the reference tree and the reference has no test or golden
  vector at that boundary.  The restatement follows the reference's only in-tree statement
  of the semantics, the mask rebuild in ``spattn/threshold/model_tuner.py:202-216``, plus
  the published vertical-slash flash-attention contract (softmax scale 1/sqrt(D), causal
  ``key <= query`` applied per element).

All citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

SPATTN_BLOCK_SIZE_K = 64  # spattn/src/VecAttention.py:45-46 (dense "slash" block width)
DEFAULT_BSQ = 64          # spattn/src/kernels/vecattention_kernels.py:51-53 and every causal pkl entry


# --------------------------------------------------------------------------------------
# A0: threshold -> gap, block tables
# --------------------------------------------------------------------------------------
def gap_from_threshold(threshold: Union[float, torch.Tensor]):
    """MinP threshold -> logit gap.  spattn/src/VecAttention.py:48-52."""
    if isinstance(threshold, torch.Tensor):
        return -torch.log(threshold + 1e-9)
    return -math.log(threshold + 1e-9, math.e)


def block_tables(batch: int, heads: int, seq_len: int, pq: int, causal: bool
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense-block tables.  spattn/src/VecAttention.py:62-92.

    Causal: each query tile gets the first ``pq`` keys (sink) and its own diagonal tile as
    64-wide blocks; non-causal: no dense blocks.
    """
    nq = math.ceil(seq_len / pq)
    if not causal:
        return (torch.zeros(batch, heads, nq, dtype=torch.int32),
                torch.zeros(batch, heads, nq, 1, dtype=torch.int32))
    n = pq // SPATTN_BLOCK_SIZE_K
    cnt = torch.full((batch, heads, nq), 2 * n, dtype=torch.int32)
    cnt[..., 0] = math.ceil(min(seq_len, pq) / SPATTN_BLOCK_SIZE_K)
    if seq_len > pq and seq_len % pq != 0:
        cnt[..., -1] = n + math.ceil((seq_len - (seq_len // pq) * pq) / SPATTN_BLOCK_SIZE_K)
    idx = torch.zeros(batch, heads, nq, 2 * n, dtype=torch.int32)
    offs = torch.arange(n, dtype=torch.int32) * SPATTN_BLOCK_SIZE_K
    idx[..., :n] = offs
    base = (torch.arange(nq, dtype=torch.int32) * pq).unsqueeze(-1)
    idx[..., n:] = base + offs
    return cnt, idx


# --------------------------------------------------------------------------------------
# A1: mean pooling of Q per query tile
# --------------------------------------------------------------------------------------
def _pairwise_tree_sum(x: torch.Tensor) -> torch.Tensor:
    """Sum over dim -2 (a power-of-two length) as a balanced binary tree of fp32 adds:
    level 0 adds rows (0,1),(2,3),...; level 1 adds those partial sums pairwise; and so on.
    The CUDA pooling kernel uses exactly this association, so both round identically."""
    n = x.shape[-2]
    assert n & (n - 1) == 0
    while n > 1:
        x = x[..., 0::2, :] + x[..., 1::2, :]
        n //= 2
    return x[..., 0, :]


def pool_q(q: torch.Tensor, pq: int) -> torch.Tensor:
    """Mean of every ``pq`` consecutive query rows, computed in fp32, returned in q.dtype.

    Follows spattn/src/utils.py:340-360 (``average_vector``) and the Triton pooling kernel
    spattn/src/utils.py:48,64 (a ragged last tile is divided by its real row count).  The
    reference does not specify the association of the fp32 sum (``tl.sum`` / ``mean``);
    here it is the balanced tree of ``_pairwise_tree_sum``.
    """
    b, h, s, d = q.shape
    nq = math.ceil(s / pq)
    x = q.float()
    pad = nq * pq - s
    if pad:
        x = torch.nn.functional.pad(x, (0, 0, 0, pad), value=0.0)
    x = x.view(b, h, nq, pq, d)
    tot = _pairwise_tree_sum(x)
    cnt = torch.full((nq,), float(pq), dtype=torch.float32)
    cnt[-1] = float(pq - pad)
    return (tot / cnt.view(1, 1, nq, 1)).to(q.dtype)


# --------------------------------------------------------------------------------------
# A2/A3: streaming MinP selection of key columns
# --------------------------------------------------------------------------------------
def scaled_pooled_q(avg_q: torch.Tensor, scale_in_dtype: bool = False) -> torch.Tensor:
    """q~ = round_to_dtype(fp32(q_bar) * fp32(1/sqrt(D))).
    spattn/src/kernels/vecattention_kernels.py:94,244-245.  Compiled Triton passes the run-time
    float argument ``sm_scale`` as an fp32 value, so a 16-bit tile times it is promoted to an
    fp32 product and rounded once (triton/language/semantic.py, ``computation_type_impl`` rule
    2; the PyTorch-like "scalar does not promote" rule applies to Python literals only).
    ``scale_in_dtype`` is what the Triton CPU *interpreter* does instead: there ``sm_scale``
    stays a Python number, is rounded to the tile's 16-bit type and multiplied in that type.
    It exists only so that the interpreter-generated 16-bit fixture can be checked."""
    d = avg_q.shape[-1]
    if scale_in_dtype:
        return avg_q * torch.tensor(1.0 / math.sqrt(d), dtype=avg_q.dtype)
    scale = torch.tensor(1.0 / math.sqrt(d), dtype=torch.float32)
    return (avg_q.float() * scale).to(avg_q.dtype)


def row_key_limits(nq: int, tile_offset: int, sk: int, pq: int, bk: int, causal: bool,
                   wo_initial: bool, bsq: int = DEFAULT_BSQ, compat_q1: bool = True,
                   rows: Optional[Sequence[int]] = None) -> Tuple[int, np.ndarray]:
    """Eligible key range [lo, hi[r]) of every pooled row of one chunk.

    spattn/src/kernels/vecattention_kernels.py:231-233,260.  ``lo``: with ``wo_init`` the
    first ``pq`` keys (the sink tile) are never selectable.  ``hi``: non-causal -> ``sk``;
    causal -> start of the row's own diagonal tile.  The reference evaluates the causal
    test with a truncating integer division relative to the first tile of the Triton
    program (``bsq`` pooled rows per program), which for the first row of each program
    also drops the key blocks starting inside the preceding tile, except its first one
    (``compat_q1``).  ``rows`` (optional) gives the position inside the chunk of each of the
    ``nq`` pooled rows when only a sample of the chunk's rows is evaluated.
    """
    lo = pq if wo_initial else 0
    pos = np.arange(nq, dtype=np.int64) if rows is None else np.asarray(rows, dtype=np.int64)
    assert pos.shape == (nq,)
    g = tile_offset + pos
    if not causal:
        return lo, np.full(nq, sk, dtype=np.int64)
    hi = np.minimum(sk, g * pq)
    if compat_q1:
        first = (pos % bsq) == 0
        hi = np.where(first, np.minimum(hi, (g - 1) * pq + bk), hi)
    return lo, np.maximum(hi, 0)


def select_columns(avg_q: torch.Tensor, k: torch.Tensor, tile_offset: int,
                   gap: Union[float, torch.Tensor], causal: bool, pq: int, bk: int,
                   wo_initial: bool = False, group_k_block: int = 1,
                   bsq: int = DEFAULT_BSQ, compat_q1: bool = True,
                   return_ambiguous: bool = False, rel_tol: float = 1e-6,
                   scale_in_dtype: bool = False, rows: Optional[Sequence[int]] = None):
    """Streaming MinP selection.  Restates ``fuse_qk_softmax_minp_wo_causal``
    (spattn/src/kernels/vecattention_kernels.py:59-181) and its Triton kernels (:206-345).

    For every pooled row and every group of ``group_k_block`` key blocks of ``bk`` keys:
    walk the blocks in order, ``m = max(m, max_j s[j])`` including the current block
    (:257), keep key ``j`` iff ``fp32(s[j] + gap) >= m`` (:258) and ``j`` lies in the row's
    eligible range.  Keys past ``sk`` (NaN padding in the reference, :117-127) never count.

    Returns ``(count[B,H,nq] int32, index[B,H,nq,max(1,max count)] int32)`` with each row's
    indices ascending (the reference's cross-group order depends on atomics; compare as
    sets).  With ``return_ambiguous`` also returns a list-of-lists of int64 arrays holding,
    per (b,h,row), the keys whose estimate lies within ``rel_tol`` (relative to the
    magnitudes compared) of the keep/drop boundary in fp64 arithmetic.  ``rows``: the pooled
    rows given are a sample of the chunk's rows, at these positions inside the chunk (the
    rule is per row; the position only enters the causal key limit).
    """
    b_, h_, nq, d = avg_q.shape
    hkv = k.shape[1]
    assert h_ % hkv == 0
    rep = h_ // hkv
    sk = k.shape[2]
    g_ = int(group_k_block)
    if wo_initial and pq % bk != 0:
        raise ValueError("wo_initial requires q_pooling_size % k_local_size == 0")
    if causal and pq % bk != 0:  # vecattention_kernels.py:129
        raise AssertionError("causal requires q_pooling_size % k_local_size == 0")
    qt = scaled_pooled_q(avg_q, scale_in_dtype)
    lo, hi = row_key_limits(nq, tile_offset, sk, pq, bk, causal, wo_initial, bsq, compat_q1, rows)
    hi_t = torch.from_numpy(hi).view(nq, 1)
    nblk = math.ceil(sk / bk)
    ngrp = math.ceil(nblk / g_)
    jj = torch.arange(nblk * bk).view(1, -1)
    in_range = (jj >= lo) & (jj < hi_t) & (jj < sk)
    blk_of_key = (torch.arange(nblk * bk) // bk)

    counts = torch.zeros(b_, h_, nq, dtype=torch.int32)
    rows = []
    amb_rows = []
    for b in range(b_):
        for h in range(h_):
            if isinstance(gap, torch.Tensor):
                # per-head kernel: gaps[b*H + h]  (vecattention_kernels.py:301-302)
                gap32 = gap.reshape(-1)[(b * h_ + h) % gap.numel()].to(torch.float32)
            else:
                gap32 = torch.tensor(float(gap), dtype=torch.float32)
            qh = qt[b, h].float()
            kh = k[b, h // rep].float()
            s = qh @ kh.t()                                   # fp32 accumulate (:256)
            sp = torch.full((nq, nblk * bk), float("-inf"), dtype=torch.float32)
            sp[:, :sk] = s
            bmax = sp.view(nq, nblk, bk).amax(-1)
            bmax[:, : lo // bk] = float("-inf")               # blocks before ``lo`` are not walked
            bm = torch.full((nq, ngrp * g_), float("-inf"), dtype=torch.float32)
            bm[:, :nblk] = bmax
            pm = torch.cummax(bm.view(nq, ngrp, g_), dim=-1).values.reshape(nq, ngrp * g_)[:, :nblk]
            m = pm[:, blk_of_key]
            keep = ((sp + gap32) >= m) & in_range
            counts[b, h] = keep.sum(-1).to(torch.int32)
            rows.append([torch.nonzero(keep[r]).flatten().to(torch.int32) for r in range(nq)])
            if return_ambiguous:
                s64 = qh.double() @ kh.double().t()
                sp64 = torch.full((nq, nblk * bk), float("-inf"), dtype=torch.float64)
                sp64[:, :sk] = s64
                bmax64 = sp64.view(nq, nblk, bk).amax(-1)
                bmax64[:, : lo // bk] = float("-inf")
                bm64 = torch.full((nq, ngrp * g_), float("-inf"), dtype=torch.float64)
                bm64[:, :nblk] = bmax64
                pm64 = torch.cummax(bm64.view(nq, ngrp, g_), dim=-1).values.reshape(nq, -1)[:, :nblk]
                m64 = pm64[:, blk_of_key]
                g64 = float(gap32)
                scale = torch.maximum(m64.abs(), sp64.abs() + abs(g64))
                near = ((sp64 + g64 - m64).abs() <= rel_tol * scale) & in_range
                amb_rows.append([torch.nonzero(near[r]).flatten() for r in range(nq)])
    maxc = max(1, min(sk, int(counts.max()) if counts.numel() else 0))
    index = torch.zeros(b_, h_, nq, maxc, dtype=torch.int32)
    for b in range(b_):
        for h in range(h_):
            for r, ids in enumerate(rows[b * h_ + h]):
                index[b, h, r, : ids.numel()] = ids
    if return_ambiguous:
        return counts, index, amb_rows
    return counts, index


# --------------------------------------------------------------------------------------
# A4: vector-sparse attention
# --------------------------------------------------------------------------------------
def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pq: int,
                     blk_count: torch.Tensor, blk_idx: torch.Tensor,
                     col_count: torch.Tensor, col_idx: torch.Tensor,
                     causal: bool, q_offset: int = 0, round_p: bool = False,
                     out_dtype: Optional[torch.dtype] = None,
                     compute_dtype: torch.dtype = torch.float32,
                     tiles: Optional[Sequence[int]] = None) -> torch.Tensor:
    """softmax(Q K_t^T / sqrt(D)) V_t per query tile over K_t = dense 64-key blocks at
    ``blk_idx[..., :blk_count]`` plus single keys ``col_idx[..., :col_count]``.

    Call contract: spattn/src/VecAttention.py:110-121.  Which (row, key) pairs take part:
    spattn/threshold/model_tuner.py:202-216 (64-wide slabs clipped to the key length, plus
    the listed columns, for all rows of the tile), intersected with ``key <= query`` when
    causal (:182-185 there: the dense softmax is causally masked before the sparse mask is
    applied).  ``q`` is (B,H,Sq,D) holding query rows ``q_offset ..``; ``k``/``v`` are
    (B,Hkv,Sk,D).  A tile with no key at all yields zeros (undefined in the reference).
    ``round_p`` rounds the unnormalised probabilities to the input dtype before the PV
    product, as flash-attention kernels do.  ``tiles`` restricts the work to these query
    tiles (the other rows of the result stay zero).
    """
    b_, h_, sq, d = q.shape
    hkv = k.shape[1]
    rep = h_ // hkv
    sk = k.shape[2]
    out_dtype = out_dtype or q.dtype
    out = torch.zeros(b_, h_, sq, d, dtype=out_dtype)
    scale = 1.0 / math.sqrt(d)
    nq = math.ceil(sq / pq)
    for b in range(b_):
        for h in range(h_):
            kh = k[b, h // rep].to(compute_dtype)
            vh = v[b, h // rep].to(compute_dtype)
            for t in (range(nq) if tiles is None else tiles):
                r0, r1 = t * pq, min((t + 1) * pq, sq)
                member = torch.zeros(sk, dtype=torch.bool)
                for off in blk_idx[b, h, t, : int(blk_count[b, h, t])].tolist():
                    member[off: min(off + SPATTN_BLOCK_SIZE_K, sk)] = True
                cols = col_idx[b, h, t, : int(col_count[b, h, t])].long()
                member[cols] = True
                keys = torch.nonzero(member).flatten()
                if keys.numel() == 0:
                    continue
                qt = q[b, h, r0:r1].to(compute_dtype)
                s = (qt @ kh[keys].t()) * scale
                if causal:
                    qpos = (q_offset + torch.arange(r0, r1)).view(-1, 1)
                    s = s.masked_fill(keys.view(1, -1) > qpos, float("-inf"))
                mx = s.amax(-1, keepdim=True)
                mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
                p = torch.exp(s - mx)
                l = p.sum(-1, keepdim=True)
                if round_p:
                    p = p.to(q.dtype).to(compute_dtype)
                o = (p @ vh[keys]) / torch.where(l > 0, l, torch.ones_like(l))
                out[b, h, r0:r1] = o.to(out_dtype)
    return out


def dense_attention(q, k, v, causal: bool, q_offset: int = 0,
                    compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Plain softmax attention (fp32/fp64), used to report the dense-attention error."""
    b_, h_, sq, d = q.shape
    rep = h_ // k.shape[1]
    kk = k.to(compute_dtype).repeat_interleave(rep, dim=1)
    vv = v.to(compute_dtype).repeat_interleave(rep, dim=1)
    s = (q.to(compute_dtype) @ kk.transpose(-1, -2)) / math.sqrt(d)
    if causal:
        qpos = (q_offset + torch.arange(sq)).view(-1, 1)
        s = s.masked_fill(torch.arange(k.shape[2]).view(1, -1) > qpos, float("-inf"))
    return torch.softmax(s, dim=-1) @ vv


# --------------------------------------------------------------------------------------
# A0: the whole operator
# --------------------------------------------------------------------------------------
def vecattention_prefill(q, k, v, threshold=None, q_pooling_size: int = 128,
                         k_local_size: int = 128, group_k_block: int = 1,
                         causal: bool = True, chunk_size: int = 16 * 1024,
                         bsq: int = DEFAULT_BSQ, compat_q1: bool = True,
                         round_p: bool = False, return_selection: bool = False):
    """The operator end to end.  spattn/src/VecAttention.py:10-123, with K/V of
    ``Hkv`` heads treated as the reference's callers treat them (``repeat_kv``,
    spattn/src/models/load_qwen2p5_vl.py:51-53)."""
    assert chunk_size % q_pooling_size == 0
    assert q_pooling_size in (64, 128)
    gap = gap_from_threshold(threshold)
    b_, h_, sq, d = q.shape
    pq = q_pooling_size
    blk_count, blk_idx = block_tables(b_, h_, sq, pq, causal)
    out = torch.empty(b_, h_, sq, d, dtype=q.dtype)
    sel = []
    for i in range(0, sq, chunk_size):
        qc = q[:, :, i: i + chunk_size]
        avg = pool_q(qc, pq)
        cc, ci = select_columns(avg, k, i // pq, gap, causal, pq, k_local_size,
                                wo_initial=causal, group_k_block=group_k_block,
                                bsq=bsq, compat_q1=compat_q1)
        t0, t1 = i // pq, (i + chunk_size) // pq
        kc = k[:, :, : i + chunk_size] if causal else k
        vc = v[:, :, : i + chunk_size] if causal else v
        out[:, :, i: i + chunk_size] = sparse_attention(
            qc, kc, vc, pq, blk_count[:, :, t0:t1], blk_idx[:, :, t0:t1], cc, ci,
            causal, q_offset=i, round_p=round_p)
        sel.append((cc, ci))
    if return_selection:
        return out, sel
    return out


# --------------------------------------------------------------------------------------
# The dispatcher's vision-slice composition around the operator
# --------------------------------------------------------------------------------------
def vecattention_prefill_vision(q, k, v, threshold, q_pooling_size, k_local_size, group_k_block, chunk_size,
                                vision_start, vision_end, bsq: int = DEFAULT_BSQ, compat_q1: bool = True):
    """The ``vecattention`` branch of customize_prefill_attention with vision positions set,
    spattn/src/models/utils.py:97-128 (causal): full attention on rows [0, vision_start), the
    operator on [0, vision_end), full attention over all keys on rows [vision_end, S)."""
    s = q.shape[2]
    end = s if vision_end is None else vision_end
    out_va = vecattention_prefill(q[:, :, :end], k[:, :, :end], v[:, :, :end], threshold, q_pooling_size,
                                  k_local_size, group_k_block, True, chunk_size, bsq=bsq, compat_q1=compat_q1)
    out_va = out_va.clone()
    if vision_start is not None:
        out_va[:, :, :vision_start] = dense_attention(q[:, :, :vision_start], k[:, :, :vision_start],
                                                      v[:, :, :vision_start], True)
    if vision_end is not None:
        after = dense_attention(q[:, :, end:], k, v, True, q_offset=end)
        return torch.cat([out_va, after.to(out_va.dtype)], dim=2)
    return out_va


# --------------------------------------------------------------------------------------
# The threshold tuner's inner loop
# --------------------------------------------------------------------------------------
def seg_pr_per_head(q, k, block_size_q, block_size_k=16, group_size_k=16, threshold=None,
                    chunk_size=8 * 1024, causal=False, bsq: int = DEFAULT_BSQ, round_probs: bool = False):
    """Recall and sparsity of the selection per head, spattn/threshold/model_tuner.py:118-226:
    dense softmax over all (visible) keys, masked with the selection (64-key blocks of the block
    tables in full width, selected columns), summed per row; sparsity = mean over rows of
    1 - |mask row| / visible keys.  ``round_probs`` rounds each probability to the input dtype
    before the sum, as the reference does."""
    b_, h_, s, d = q.shape
    sk = k.shape[2]
    rep = h_ // k.shape[1]
    if isinstance(threshold, torch.Tensor):
        gap = -torch.log(threshold.float())
    else:
        gap = -math.log(threshold)
    pq = block_size_q
    blk_count, blk_idx = block_tables(b_, h_, s, pq, causal)
    recalls = torch.zeros(b_, h_, s, dtype=torch.float64)
    sparsity = torch.zeros(h_, dtype=torch.float64)
    kk = k.double().repeat_interleave(rep, dim=1)
    for i in range(0, s, chunk_size):
        qc = q[:, :, i:i + chunk_size]
        n = qc.shape[2]
        cc, ci = select_columns(pool_q(qc, pq), k, i // pq, gap, causal, pq, block_size_k, wo_initial=causal,
                                group_k_block=group_size_k, bsq=bsq)
        scores = (qc.double() @ kk.transpose(-1, -2)) / math.sqrt(d)
        rows = i + torch.arange(n)
        see = torch.ones(n, sk, dtype=torch.bool)
        if causal:
            see = torch.arange(sk).view(1, -1) <= rows.view(-1, 1)
            scores = scores.masked_fill(~see, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        if round_probs:
            probs = probs.to(q.dtype).double()
        for bb in range(b_):
            for hh in range(h_):
                mask = torch.zeros(n, sk, dtype=torch.bool)
                for t in range(math.ceil(n / pq)):
                    g = i // pq + t
                    r0, r1 = t * pq, min((t + 1) * pq, n)
                    for o in blk_idx[bb, hh, g, : int(blk_count[bb, hh, g])].tolist():
                        mask[r0:r1, o:min(o + 64, sk)] = True
                    mask[r0:r1, ci[bb, hh, t, : int(cc[bb, hh, t])].long()] = True
                recalls[bb, hh, i:i + n] = (probs[bb, hh] * mask).sum(-1)
                sparsity[hh] += (1.0 - (mask.sum(-1).double() / see.sum(-1).double())).mean() * n
    return recalls.sum(dim=(0, 2)) / (b_ * s), sparsity / b_ / s


# --------------------------------------------------------------------------------------
# Q/K preparation of a video-DiT attention layer (RMSNorm over the hidden size, rotary embedding)
# --------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of the last dimension as the reference's Triton kernel computes it
    (eval/DiTEvalKit/kernels/triton/rmsnorm.py:30-47): fp32 throughout, ``x * rstd`` then ``* w``, rounded to
    the input dtype at the end.  (The association of the sum of squares is not specified there.)"""
    xf = x.float()
    rstd = 1.0 / torch.sqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return ((xf * rstd) * weight.float()).to(x.dtype)


def _round_from_double(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """float64 -> 16-bit type with ONE rounding to nearest, as the CUDA conversion the reference kernel uses
    does.  (torch converts by way of float32, i.e. rounds twice; here the float32 step rounds to odd, after
    which the final rounding to nearest is exact.)"""
    f = x.to(torch.float32)
    err = x - f.double()
    bits = f.view(torch.int32)
    inexact_even = (err != 0) & ((bits & 1) == 0) & torch.isfinite(f)
    toward_larger_magnitude = (err > 0) == (f > 0)
    bits = torch.where(inexact_even, torch.where(toward_larger_magnitude, bits + 1, bits - 1), bits)
    return bits.view(torch.float32).to(dtype)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, skip: int = 0) -> torch.Tensor:
    """Rotary embedding on interleaved (even, odd) element pairs of (B, H, S, D), in double precision, rounded
    to the input dtype: the in-place CUDA kernel of the reference (eval/DiTEvalKit/kernels/include/rope/
    rope_enc_complex.cuh:27-45, tokens before ``skip`` untouched, :82-100), equivalently its PyTorch fallback
    ``view_as_complex(x) * freqs`` (eval/DiTEvalKit/models/wan/attention.py:61-69).  ``cos`` / ``sin``: (S - skip, D/2)."""
    out = x.clone()
    xd = x[:, :, skip:].double()
    e, o = xd[..., 0::2], xd[..., 1::2]
    c, s = cos.double(), sin.double()
    rot = torch.stack((e * c - o * s, o * c + e * s), dim=-1).flatten(-2)
    out[:, :, skip:] = _round_from_double(rot, x.dtype)
    return out


def rope_interleaved_txtlast(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, txt_len: int = 0) -> torch.Tensor:
    """Rotary embedding of (B, H, L, D) on interleaved pairs with per-element float32 tables (L - txt_len, D),
    computed in float32 as the reference's text-last kernel does through flashinfer's helper
    (eval/DiTEvalKit/kernels/include/rope/rope_enc_txtlast.cuh:32-76; flashinfer/pos_enc.cuh
    ``vec_apply_llama_rope_cos_sin_interleave``): out[i] = x[i] cos[i] + (-x[i+1] if i even else x[i-1]) sin[i];
    the last ``txt_len`` tokens are not rotated.  (The product pair is evaluated here as
    ``other * sin + fl(x * cos)``; a fused or unfused choice there moves a result by one float32 unit at most.)"""
    out = x.clone()
    n = x.shape[2] - txt_len
    if n <= 0:
        return out
    xf = x[:, :, :n].float()
    other = torch.stack((-xf[..., 1::2], xf[..., 0::2]), dim=-1).flatten(-2)
    first = (xf * cos.float()).double()                       # fl(x cos), exact in double
    rot = (other.double() * sin.double() + first).float()     # one rounding of other * sin + fl(x cos): the fused form
    out[:, :, :n] = rot.to(x.dtype)
    return out

