"""Host side of the VecAttention prefill path: the reference's Python entry points, same names,
arguments and error conditions, each a thin call into ``libvecattn.so`` on the current CUDA
stream.  PyTorch is used for device memory and streams only.

Reference interfaces mirrored here (paths inside anminliu/VecAttention):
  * ``VecAttention_prefill``            spattn/src/VecAttention.py:10-123
  * ``average_vector``                  spattn/src/utils.py:340-360
  * ``fuse_qk_softmax_minp_wo_causal``  spattn/src/kernels/vecattention_kernels.py:59-181
  * ``sparse_attn_func``                vllm_flash_attn (call site spattn/src/VecAttention.py:110-121)
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple, Union

import torch

from . import _lib as L

import time

SPATTN_BLOCK_SIZE_K = 64
_FREE_MEMORY = {}  # device index -> (time of the query, free bytes): the query costs a fraction of a millisecond


def _free_bytes(dev: torch.device) -> int:
    """Free device memory, asked from the driver at most twice a second per device."""
    now = time.monotonic()
    hit = _FREE_MEMORY.get(dev.index)
    if hit is None or now - hit[0] > 0.5:
        hit = (now, torch.cuda.mem_get_info(dev)[0])
        _FREE_MEMORY[dev.index] = hit
    return hit[1]


DEFAULT_COMPAT_BSQ = 64  # Triton program height of every causal launch config the reference ships


class VecAttentionArgumentError(AssertionError, ValueError):
    """Raised where the reference fails a Python ``assert`` on its arguments."""


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return L.VA_BF16
    if t.dtype == torch.float16:
        return L.VA_FP16
    raise VecAttentionArgumentError(f"dtype {t.dtype} not supported: the CUDA path computes in bf16 or fp16")


def _require_cuda(*ts: torch.Tensor) -> torch.device:
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("VecAttention kernels need CUDA tensors (there is no CPU fallback)")
        if t.device != dev:
            raise VecAttentionArgumentError("all tensors must be on the same device")
    return dev


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """Return ``t`` if the kernels can address it in place (unit inner stride, 16-byte aligned
    rows), else a contiguous copy."""
    if t.stride(-1) == 1 and all(s % 8 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


def _t4(t: torch.Tensor) -> L.Tensor4:
    """(B,H,S,D) view -> pointer + element strides."""
    return L.Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int) -> None:
    if code != 0:
        msg = L.status_string(code)
        if code == -7:
            raise VecAttentionArgumentError(msg)
        raise RuntimeError(f"libvecattn: {msg} (status {code})")


def _gap_args(gap: Union[float, torch.Tensor], batch: int, heads: int, device) -> Tuple[float, Optional[torch.Tensor], int]:
    """float gap -> (gap, None, 0); tensor gap -> (0, fp32 device tensor, batch stride)."""
    if isinstance(gap, torch.Tensor):
        g = gap.to(device=device, dtype=torch.float32).contiguous().reshape(-1)
        if g.numel() == 1:  # one value for all heads, given as a tensor
            g = g.expand(heads).contiguous()
        if g.numel() == heads:
            return 0.0, g, 0
        if g.numel() == batch * heads:
            return 0.0, g, heads
        raise VecAttentionArgumentError(f"per-head threshold must have {heads} or {batch * heads} entries")
    return float(gap), None, 0


# ----------------------------------------------------------------------------------------------
def average_vector(q: torch.Tensor, block_size: int, use_triton: bool = True) -> torch.Tensor:
    """Mean-pool every ``block_size`` query rows: (B,H,S,D) -> (B,H,ceil(S/block_size),D), same
    dtype.  ``use_triton`` is accepted for signature compatibility and ignored."""
    _require_cuda(q)
    if block_size not in (64, 128):
        raise VecAttentionArgumentError("q_pooling_size must be 64 or 128")
    b, h, s, d = q.shape
    q = _rows_ok(q)
    out = torch.empty(b, h, math.ceil(s / block_size), d, dtype=q.dtype, device=q.device)
    args = L.PoolArgs(_dtype_code(q), b, h, s, d, block_size, _t4(q), out.data_ptr())
    with torch.cuda.device(q.device):
        _check(L.lib().va_pool_q(C.byref(args), _stream()))
    return out


def fuse_qk_softmax_minp_wo_causal(avg_q_chunk: torch.Tensor, k: torch.Tensor, avg_q_chunk_offset: int,
                                   gap: Union[float, torch.Tensor], causal: bool = True,
                                   q_pooling_size: int = 128, k_local_size: int = 128,
                                   wo_initial: bool = False, group_k_block: int = 1, *,
                                   compat_q1: bool = True, trim: bool = True,
                                   capacity: Optional[int] = None, status: Optional[torch.Tensor] = None,
                                   chunk_tiles: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Select key columns per pooled query row.  Returns ``(column_count (B,H,nq) int32,
    column_index (B,H,nq,n) int32)`` with each row's first ``count`` entries valid and ascending.

    ``trim=True`` slices ``column_index`` to the largest count like the reference does (this reads
    the maximum back to the host); ``trim=False`` returns the full ``capacity``-wide buffer with
    no synchronisation.  Entries past a row's count are uninitialised (the reference zero-fills).
    ``k`` may have fewer heads than ``avg_q_chunk`` (grouped-query attention).  ``chunk_tiles > 0``:
    the pooled rows span several prefill chunks of that many query tiles, and the causal rule's
    ``compat_q1`` rows restart at every chunk boundary, as in the reference's chunk loop.
    """
    dev = _require_cuda(avg_q_chunk, k)
    b, h, nq, d = avg_q_chunk.shape
    hkv, sk = k.shape[1], k.shape[2]
    if h % hkv != 0:
        raise VecAttentionArgumentError("query heads must be a multiple of key heads")
    if causal and q_pooling_size % k_local_size != 0:
        raise VecAttentionArgumentError("causal selection needs q_pooling_size % k_local_size == 0")
    avg_q_chunk = avg_q_chunk.contiguous()
    k = _rows_ok(k)
    cap = int(capacity) if capacity is not None else (sk + 3) // 4 * 4
    count = torch.empty(b, h, nq, dtype=torch.int32, device=dev)
    index = torch.empty(b, h, nq, cap, dtype=torch.int32, device=dev)
    gapf, gaps, gstride = _gap_args(gap, b, h, dev)
    args = L.SelectArgs(_dtype_code(k), b, h, hkv, nq, sk, d, q_pooling_size, k_local_size, group_k_block,
                        int(bool(causal)), int(bool(wo_initial)), DEFAULT_COMPAT_BSQ if compat_q1 else 0,
                        int(avg_q_chunk_offset), avg_q_chunk.data_ptr(), _t4(k), gapf,
                        gaps.data_ptr() if gaps is not None else None, gstride,
                        count.data_ptr(), index.data_ptr(), cap,
                        status.data_ptr() if status is not None else None, int(chunk_tiles), None, 0)
    if avg_q_chunk.dtype != k.dtype:
        raise VecAttentionArgumentError("pooled queries and keys must have the same dtype")
    nbytes = C.c_size_t(0)
    _check(L.lib().va_select_workspace_bytes(C.byref(args), C.byref(nbytes)))
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)  # keep bits, one per (pooled row, key)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes.value
    with torch.cuda.device(dev):
        _check(L.lib().va_select(C.byref(args), _stream()))
    if trim:
        n = max(min(sk, int(count.max())), 1)
        index = index[..., :n]
    return count, index


def sparse_attn_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pooling_size: int,
                     block_count: torch.Tensor, block_offset: torch.Tensor,
                     column_count: torch.Tensor, column_index: torch.Tensor,
                     return_softmax_lse: bool = False, causal: bool = False,
                     softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Vector-sparse attention in the reference's calling convention: ``q`` (B,Sq,H,D), ``k``/``v``
    (B,Sk,Hkv,D), tables per (B,H,ceil(Sq/q_pooling_size)); returns (B,Sq,H,D).  With ``causal``
    the queries are the last ``Sq`` positions of the ``Sk`` keys.  ``return_softmax_lse`` adds the
    (B,H,Sq) float32 log-sum-exp of the scaled scores over each row's keys."""
    lse = (torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
           if return_softmax_lse else None)
    out = _sparse_attn_bhsd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), q_pooling_size,
                            block_count, block_offset, column_count, column_index, causal,
                            q_offset=(k.shape[1] - q.shape[1]) if causal else 0, softmax_scale=softmax_scale,
                            out_layout="bshd", lse=lse)
    return (out, lse) if return_softmax_lse else out


def _sparse_attn_bhsd(q, k, v, pq, block_count, block_offset, column_count, column_index, causal,
                      q_offset=0, softmax_scale=None, out=None, out_layout="bhsd", status=None, lse=None,
                      vision: Optional[Tuple[int, int]] = None):
    """``vision = (begin, end)``: the vision-slice composition in one launch: the tables describe the query
    tiles of rows [0, end) only; rows before ``begin`` and from ``end`` on get full causal attention."""
    dev = _require_cuda(q, k, v, column_count, column_index)
    b, h, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    q, k, v = _rows_ok(q), _rows_ok(k), _rows_ok(v)
    if out is None:
        if out_layout == "bshd":
            out = torch.empty(b, sq, h, d, dtype=q.dtype, device=dev).transpose(1, 2)
        else:
            out = torch.empty(b, h, sq, d, dtype=q.dtype, device=dev)
    column_count = column_count.contiguous()
    nq = math.ceil((sq if vision is None else vision[1]) / pq)
    if tuple(column_count.shape) != (b, h, nq) or tuple(column_index.shape[:3]) != (b, h, nq):
        raise VecAttentionArgumentError("column tables must be shaped (B, H, ceil(Sq/q_pooling_size)[, n])")
    # the index table may be a trimmed view of a wider buffer: pass its row stride instead of copying
    col_stride = column_index.stride(2)
    if (column_index.stride(-1) != 1 or column_index.stride(1) != nq * col_stride
            or column_index.stride(0) != h * nq * col_stride):
        column_index = column_index.contiguous()
        col_stride = column_index.stride(2)
    if block_count is not None and block_offset is not None and block_offset.numel() > 0:
        block_count = block_count.contiguous()
        block_offset = block_offset.contiguous()
        bc, bo, bs = block_count.data_ptr(), block_offset.data_ptr(), block_offset.shape[-1]
    else:
        bc, bo, bs = None, None, 0
    args = L.AttnArgs(_dtype_code(q), b, h, hkv, sq, sk, d, pq, int(bool(causal)), int(q_offset),
                      _t4(q), _t4(k), _t4(v), _t4(out), bc, bo, bs,
                      column_count.data_ptr(), column_index.data_ptr(), col_stride,
                      float(softmax_scale) if softmax_scale else 0.0,
                      status.data_ptr() if status is not None else None,
                      lse.data_ptr() if lse is not None else None,
                      0 if vision is None else 1, 0 if vision is None else int(vision[0]), 0 if vision is None else int(vision[1]))
    if lse is not None and (lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (b, h, sq)):
        raise VecAttentionArgumentError("lse must be a contiguous float32 tensor shaped (B, H, Sq)")
    with torch.cuda.device(dev):
        _check(L.lib().va_sparse_attn(C.byref(args), _stream()))
    return out.transpose(1, 2) if out_layout == "bshd" else out


def block_tables(batch: int, heads: int, seq_len: int, q_pooling_size: int, causal: bool, device
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The dense-block tables ``VecAttention_prefill`` builds (spattn/src/VecAttention.py:62-92)."""
    nq = math.ceil(seq_len / q_pooling_size)
    width = 2 * (q_pooling_size // SPATTN_BLOCK_SIZE_K) if causal else 1
    cnt = torch.empty(batch, heads, nq, dtype=torch.int32, device=device)
    idx = torch.empty(batch, heads, nq, width, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _check(L.lib().va_block_tables(batch, heads, seq_len, q_pooling_size, int(bool(causal)),
                                       cnt.data_ptr(), idx.data_ptr(), _stream()))
    return cnt, idx


# ----------------------------------------------------------------------------------------------
def VecAttention_prefill(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    threshold: Union[float, torch.Tensor] = None,
    q_pooling_size: int = 128,
    k_local_size: int = 128,
    group_k_block: int = 1,
    causal: bool = True,
    chunk_size: int = 16 * 1024,
    *,
    compat_q1: bool = True,
    return_selection: bool = False,
    out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    single_pass_budget: Optional[int] = None,
):
    """Vectorized sparse attention prefill (VecAttention) on B200.

    Args (as in the reference):
        query_states: (batch, num_heads, seq_len, head_dim), bf16 or fp16, head_dim 128
        key_states, value_states: (batch, num_kv_heads, kv_len, head_dim); ``num_kv_heads`` may
            divide ``num_heads`` (treated like ``repeat_kv``-expanded keys, without the copy)
        threshold: MinP threshold, a float or a tensor with one value per head
        q_pooling_size: 64 or 128; k_local_size: 16/32/64/128; group_k_block: key blocks that share
            one running maximum; causal; chunk_size: multiple of q_pooling_size (bounds the index
            workspace; results do not depend on it except through the reference's causal quirk)
    Keyword-only extras:
        compat_q1: reproduce the reference's truncating-division quirk in the causal rule
        return_selection: also return the per-tile selected-column counts (B,H,nq) int32
        out: preallocated output
        status: int32 device tensor of one element that receives VA_STATUS_* bits (index capacity
            overflow, internal wait timeout); not cleared here, not read back here
        single_pass_budget: bytes of selected-column lists up to which the whole sequence is
            processed by one launch per stage instead of the reference's chunk loop (same
            results).  ``None`` picks it from the memory that is free right now (at most 40 % of
            it, at most 32 GiB); ``1`` forces the chunk loop, where ``chunk_size`` bounds the
            workspace as it does in the reference.  If the workspace cannot be allocated the
            call is retried with the chunk loop.

    Returns:
        attn_output: (batch, num_heads, seq_len, head_dim)
    """
    if chunk_size % q_pooling_size != 0:
        raise VecAttentionArgumentError("chunk_size must be a multiple of q_pooling_size")
    if q_pooling_size not in (64, 128):
        raise VecAttentionArgumentError("q_pooling_size must be 64 or 128")
    if threshold is None:
        raise TypeError("threshold must be a float or a tensor")
    dev = _require_cuda(query_states, key_states, value_states)
    if not (query_states.dtype == key_states.dtype == value_states.dtype):
        raise VecAttentionArgumentError("q, k and v must have the same dtype")
    b, h, sq, d = query_states.shape
    hkv, sk = key_states.shape[1], key_states.shape[2]
    if h % hkv != 0 or value_states.shape != key_states.shape:
        raise VecAttentionArgumentError("inconsistent head counts or k/v shapes")
    if causal and q_pooling_size % k_local_size != 0:
        raise VecAttentionArgumentError("causal selection needs q_pooling_size % k_local_size == 0")

    # gap = -log(threshold)  (spattn/src/VecAttention.py:48-52)
    if isinstance(threshold, torch.Tensor):
        gap = -torch.log(threshold.to(dev) + 1e-9)
    else:
        gap = -math.log(threshold + 1e-9, math.e)
    gapf, gaps, gstride = _gap_args(gap, b, h, dev)

    q, k, v = _rows_ok(query_states), _rows_ok(key_states), _rows_ok(value_states)
    if out is None:
        out = torch.empty(b, h, sq, d, dtype=q.dtype, device=dev)
    nq = math.ceil(sq / q_pooling_size)
    counts = torch.empty(b, h, nq, dtype=torch.int32, device=dev) if return_selection else None
    args = L.PrefillArgs(_dtype_code(q), b, h, hkv, sq, sk, d, q_pooling_size, k_local_size, group_k_block,
                         int(bool(causal)), chunk_size, DEFAULT_COMPAT_BSQ if compat_q1 else 0,
                         _t4(q), _t4(k), _t4(v), _t4(out), gapf,
                         gaps.data_ptr() if gaps is not None else None, gstride, None, 0,
                         counts.data_ptr() if counts is not None else None,
                         status.data_ptr() if status is not None else None, 0)
    if single_pass_budget is None:
        single_pass_budget = max(1, min(32 << 30, int(_free_bytes(dev) * 0.4)))
    args.single_pass_budget = int(single_pass_budget)
    nbytes = C.c_size_t(0)
    _check(L.lib().va_prefill_workspace_bytes(C.byref(args), C.byref(nbytes)))
    try:
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
    except torch.cuda.OutOfMemoryError:
        if args.single_pass_budget == 1:
            raise
        args.single_pass_budget = 1  # the reference's chunk loop: chunk_size bounds the workspace
        _check(L.lib().va_prefill_workspace_bytes(C.byref(args), C.byref(nbytes)))
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
    args.workspace = ws.data_ptr()
    args.workspace_bytes = nbytes.value
    with torch.cuda.device(dev):
        _check(L.lib().va_prefill(C.byref(args), _stream()))
    if return_selection:
        return out, counts
    return out
