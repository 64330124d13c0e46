"""Vision-slice composition of the prefill operator, as the reference's dispatcher applies it to
vision-language models (spattn/src/models/utils.py:97-128, causal only): text tokens before the
vision span get full attention, positions up to the end of the vision span get VecAttention, text
tokens after it get full attention over all keys.

The reference makes three calls (two to its dense flash-attention wrapper) and concatenates.  Here
every part writes straight into one output tensor and the dense parts run on the same
vector-sparse kernel, so no second attention implementation is involved.  With q_pooling_size 64
all three parts are ONE attention launch: the sparse tiles of the vision span are cut at the span's
first row, and table-free dense tiles (every 64-key block up to the diagonal) cover the rows before
and after it.  Otherwise the parts run one after another, the dense ones with explicit block tables.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch

from .api import (VecAttention_prefill, VecAttentionArgumentError, _sparse_attn_bhsd, average_vector, block_tables,
                  fuse_qk_softmax_minp_wo_causal)

_DENSE_TILE = 64  # query rows per tile of the dense passes


def dense_block_tables(batch: int, heads: int, row0: int, rows: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block tables that make the sparse kernel compute full causal attention for query rows
    ``row0 .. row0+rows-1``: tile t (64 rows from ``row0 + 64 t``) gets every 64-key block that starts
    at or before its last row.  Returns (count (B,H,nq) int32, start (B,H,nq,width) int32)."""
    nq = math.ceil(rows / _DENSE_TILE)
    last_row = torch.clamp(row0 + (torch.arange(nq, device=device) + 1) * _DENSE_TILE, max=row0 + rows) - 1
    count = (last_row // 64 + 1).to(torch.int32)                      # blocks 0 .. last_row // 64
    width = (row0 + rows - 1) // 64 + 1 if nq else 1  # = count of the last tile, known without reading the device
    start = (torch.arange(width, device=device, dtype=torch.int32) * 64).expand(nq, width)
    return (count.view(1, 1, nq).expand(batch, heads, nq).contiguous(),
            start.reshape(1, 1, nq, width).expand(batch, heads, nq, width).contiguous())


def dense_causal_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row0: int, row1: int, out: torch.Tensor) -> None:
    """out[:, :, row0:row1] = causal softmax attention of query rows row0..row1-1 over keys 0..row."""
    rows = row1 - row0
    if rows <= 0:
        return
    b, h = q.shape[0], q.shape[1]
    dev = q.device
    cnt, start = dense_block_tables(b, h, row0, rows, dev)
    nq = cnt.shape[2]
    no_cols = torch.zeros(b, h, nq, dtype=torch.int32, device=dev)
    col_idx = torch.zeros(b, h, nq, 4, dtype=torch.int32, device=dev)
    _sparse_attn_bhsd(q[:, :, row0:row1], k[:, :, :row1], v[:, :, :row1], _DENSE_TILE, cnt, start, no_cols, col_idx,
                      True, q_offset=row0, out=out[:, :, row0:row1])


def VecAttention_prefill_vision(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    threshold: Union[float, torch.Tensor] = None,
    q_pooling_size: int = 128,
    k_local_size: int = 128,
    group_k_block: int = 1,
    causal: bool = True,
    chunk_size: int = 16 * 1024,
    vision_start_position: Optional[int] = None,
    vision_end_position: Optional[int] = None,
    *,
    compat_q1: bool = True,
    fused: Optional[bool] = None,
) -> torch.Tensor:
    """The ``vecattention`` branch of the reference's ``customize_prefill_attention``: with both
    positions ``None`` plain ``VecAttention_prefill``; otherwise (causal only) full attention for
    rows before ``vision_start_position``, VecAttention over ``[0, vision_end_position)`` and full
    attention over all keys for rows from ``vision_end_position`` on.  Returns (B,H,S,D).

    ``fused`` (default: whenever ``q_pooling_size`` is 64 and the index lists fit 4 GiB): one attention
    launch serves all three parts: sparse tiles for the vision span, cut at ``vision_start_position``,
    and table-free dense tiles before and after it; ``False`` runs the three parts one after another."""
    vs, ve = vision_start_position, vision_end_position
    if vs is None and ve is None:
        return VecAttention_prefill(query_states, key_states, value_states, threshold, q_pooling_size, k_local_size,
                                    group_k_block, causal, chunk_size, compat_q1=compat_q1)
    if not causal:
        raise VecAttentionArgumentError("Only causal attention is supported when vision positions are set")
    b, h, s, d = query_states.shape
    if key_states.shape[2] != s:
        raise VecAttentionArgumentError("vision slicing needs as many keys as queries")
    end = s if ve is None else max(0, min(int(ve), s))
    begin = 0 if vs is None else max(0, min(int(vs), end))
    out = torch.empty_like(query_states)
    if fused is None:
        fused = q_pooling_size == 64 and b * h * math.ceil(max(end, 1) / 64) * ((end + 3) // 4 * 4) * 4 <= (4 << 30)
    if fused and q_pooling_size != 64:
        raise VecAttentionArgumentError("the one-launch composition needs q_pooling_size 64")
    if fused and end > begin:
        # pooling and selection over rows [0, end) exactly as VecAttention_prefill runs them (its chunk loop only
        # shows in the rows the causal rule treats specially), then one attention launch over all rows
        if threshold is None:
            raise VecAttentionArgumentError("threshold is required")
        gap = -torch.log(threshold.to(query_states.device) + 1e-9) if isinstance(threshold, torch.Tensor) \
            else -math.log(threshold + 1e-9, math.e)
        if chunk_size % q_pooling_size != 0:
            raise VecAttentionArgumentError("chunk_size must be a multiple of q_pooling_size")
        avg = average_vector(query_states[:, :, :end], 64)
        cnt, idx = fuse_qk_softmax_minp_wo_causal(avg, key_states[:, :, :end], 0, gap, True, 64, k_local_size,
                                                  wo_initial=True, group_k_block=group_k_block, compat_q1=compat_q1,
                                                  trim=False, chunk_tiles=chunk_size // 64)
        bcnt, bidx = block_tables(b, h, end, 64, True, query_states.device)
        _sparse_attn_bhsd(query_states, key_states, value_states, 64, bcnt, bidx, cnt, idx, True, out=out,
                          vision=(begin, end))
        return out
    if end > 0:  # VecAttention on [0, end); the rows before `begin` are overwritten below
        VecAttention_prefill(query_states[:, :, :end], key_states[:, :, :end], value_states[:, :, :end], threshold,
                             q_pooling_size, k_local_size, group_k_block, True, chunk_size, compat_q1=compat_q1,
                             out=out[:, :, :end])
    dense_causal_rows(query_states, key_states, value_states, 0, begin, out)
    dense_causal_rows(query_states, key_states, value_states, end, s, out)
    return out
