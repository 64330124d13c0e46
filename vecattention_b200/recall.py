"""Recall and sparsity of a selection, the inner loop of the reference's threshold tuner
(``seg_pr_perHead``, spattn/threshold/model_tuner.py:118-226).

For every query row the reference materialises the dense softmax over all keys (fp32, rounded to
the input dtype), multiplies it with the selection mask (dense 64-key blocks and selected columns
of the row's tile) and sums: the attention mass the selection keeps.  Here that mass is
``exp(lse_selected - lse_all)``: the vector-sparse kernel returns the log-sum-exp of the scaled
scores over the keys it visits, once with the selection's tables and once with tables that list
every key, so no (rows x keys) matrix is ever formed.  (The reference rounds every probability to
16 bits before summing; this path does not, so the two agree to about 1e-3.)
"""
from __future__ import annotations

import math
from typing import Tuple, Union

import torch

from .api import _sparse_attn_bhsd, average_vector, block_tables, fuse_qk_softmax_minp_wo_causal
from .vision import dense_block_tables


def _all_block_tables(batch: int, heads: int, nq: int, sk: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    width = math.ceil(sk / 64)
    cnt = torch.full((batch, heads, nq), width, dtype=torch.int32, device=device)
    start = (torch.arange(width, device=device, dtype=torch.int32) * 64).expand(batch, heads, nq, width).contiguous()
    return cnt, start


def selection_recall_sparsity(q: torch.Tensor, k: torch.Tensor, block_size_q: int, block_size_k: int = 16,
                              group_size_k: int = 16, threshold: Union[float, torch.Tensor] = None,
                              chunk_size: int = 8 * 1024, causal: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Arguments as ``seg_pr_perHead``: q (B,H,S,D), k (B,Hkv,Sk,D), ``threshold`` a float or one value
    per head.  Returns (recall (H,), sparsity (H,)) in float32: the mean over batch and rows of the
    kept attention mass, and of ``1 - selected keys / visible keys`` with the reference's counting
    (a dense block counts all of its keys that exist, also those a causal row cannot see)."""
    b, h, s, d = q.shape
    sk = k.shape[2]
    dev = q.device
    pq = block_size_q
    if isinstance(threshold, torch.Tensor):
        gap = -torch.log(threshold.to(dev, torch.float32))  # the tuner adds 1e-50, which is zero in fp32
    else:
        gap = -math.log(threshold)
    blk_cnt, blk_idx = block_tables(b, h, s, pq, causal, dev)
    recall_rows = torch.empty(b, h, s, dtype=torch.float32, device=dev)
    kept = torch.empty(b, h, math.ceil(s / pq), dtype=torch.float32, device=dev)  # selected keys per tile
    scratch = torch.empty(b, h, min(chunk_size, s), d, dtype=q.dtype, device=dev)
    for i in range(0, s, chunk_size):
        qc = q[:, :, i:i + chunk_size]
        n = qc.shape[2]
        t0, t1 = i // pq, i // pq + math.ceil(n / pq)
        cc, ci = fuse_qk_softmax_minp_wo_causal(average_vector(qc, pq), k, t0, gap, causal, pq, block_size_k,
                                                wo_initial=causal, group_k_block=group_size_k, trim=False)
        bc, bi = blk_cnt[:, :, t0:t1].contiguous(), blk_idx[:, :, t0:t1].contiguous()
        lse_sel = torch.empty(b, h, n, dtype=torch.float32, device=dev)
        _sparse_attn_bhsd(qc, k, k, pq, bc, bi, cc, ci, causal, q_offset=i, out=scratch[:, :, :n], lse=lse_sel)
        # every key (causal: every 64-key block up to the diagonal, masked per element by the kernel)
        lse_all = torch.empty(b, h, n, dtype=torch.float32, device=dev)
        if causal:
            dc, di = dense_block_tables(b, h, i, n, dev)
        else:
            dc, di = _all_block_tables(b, h, math.ceil(n / 64), sk, dev)
        none = torch.zeros(b, h, dc.shape[2], dtype=torch.int32, device=dev)
        _sparse_attn_bhsd(qc, k, k, 64, dc, di, none, none.unsqueeze(-1).expand(-1, -1, -1, 4).contiguous(), causal,
                          q_offset=i, out=scratch[:, :, :n], lse=lse_all)
        recall_rows[:, :, i:i + n] = torch.exp(lse_sel - lse_all)
        # keys of the dense blocks that exist (the last block may run past the sequence)
        in_blocks = torch.zeros_like(cc, dtype=torch.float32)
        if causal:
            valid = torch.arange(bi.shape[3], device=dev).view(1, 1, 1, -1) < bc.unsqueeze(-1)
            in_blocks = (torch.clamp(sk - bi, min=0, max=64) * valid).sum(-1).float()
        kept[:, :, t0:t1] = cc.float() + in_blocks
    rows = torch.arange(s, device=dev)
    visible = (rows + 1).float() if causal else torch.full((s,), float(sk), device=dev)
    per_row = 1.0 - kept.repeat_interleave(pq, dim=2)[:, :, :s] / visible
    return recall_rows.mean(dim=(0, 2)), per_row.mean(dim=(0, 2))
