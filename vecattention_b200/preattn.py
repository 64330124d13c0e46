"""Q/K preparation of a video-DiT attention layer in one pass: RMSNorm over the hidden dimension and the
rotary embedding on interleaved element pairs (eval/DiTEvalKit/models/wan/attention.py:108-136), with no
layout change: the results keep the projections' (B, S, H*D) storage and are handed to the operator as
(B, H, S, D) *views*, which it reads in place through strides.  The reference normalises (one kernel),
makes three transposed copies and rotates in place (another kernel).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib as L
from .api import VecAttentionArgumentError, _check, _dtype_code, _require_cuda, _rows_ok, _stream, _t4


def as_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    """(B, S, heads*D) storage viewed as (B, heads, S, D); no copy."""
    b, s, n = x.shape
    return x.view(b, s, heads, n // heads).transpose(1, 2)


def qk_norm_rope(query: torch.Tensor, key: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                 eps: float, freqs_real: Optional[torch.Tensor] = None, freqs_imag: Optional[torch.Tensor] = None,
                 len_text_prompt: int = 0, *, heads: int, kv_heads: Optional[int] = None, inplace: bool = False
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``query`` (B, S, heads*128), ``key`` (B, S, kv_heads*128): RMSNorm with the given weights (``None``: no
    norm), then the rotary embedding with ``freqs_real`` / ``freqs_imag`` (S - len_text_prompt, 64) float32
    (``None``: no rotation; the first ``len_text_prompt`` tokens are never rotated).  Returns the results as
    (B, heads, S, 128) and (B, kv_heads, S, 128) views, ready for ``VecAttention_prefill``."""
    dev = _require_cuda(query, key)
    kv_heads = heads if kv_heads is None else kv_heads
    b, s, n = query.shape
    if n != heads * 128 or tuple(key.shape) != (b, s, kv_heads * 128):
        raise VecAttentionArgumentError("query / key must be (B, S, heads*128) and (B, S, kv_heads*128)")
    if query.stride(2) != 1 or key.stride(2) != 1 or query.stride(0) != s * query.stride(1) or key.stride(0) != s * key.stride(1):
        query, key = query.contiguous(), key.contiguous()
    q_out = query if inplace else torch.empty_like(query, memory_format=torch.contiguous_format)
    k_out = key if inplace else torch.empty_like(key, memory_format=torch.contiguous_format)
    for w, size in ((q_weight, n), (k_weight, kv_heads * 128)):
        if w is not None and (w.dtype != query.dtype or w.numel() != size or not w.is_contiguous()):
            raise VecAttentionArgumentError("norm weights must be contiguous, of the hidden size and of the tensors' dtype")
    if (freqs_real is None) != (freqs_imag is None):
        raise VecAttentionArgumentError("give both rotary tables or neither")
    if freqs_real is not None:
        want = (s - len_text_prompt, 64)
        for f in (freqs_real, freqs_imag):
            if f.dtype != torch.float32 or tuple(f.shape) != want or not f.is_contiguous():
                raise VecAttentionArgumentError(f"rotary tables must be contiguous float32 of shape {want}")
    ptr = lambda t: t.data_ptr() if t is not None else None
    args = L.NormRopeArgs(_dtype_code(query), b, s, heads, kv_heads, int(len_text_prompt), query.data_ptr(), key.data_ptr(),
                          query.stride(1), key.stride(1), q_out.data_ptr(), k_out.data_ptr(), q_out.stride(1), k_out.stride(1),
                          ptr(q_weight), ptr(k_weight), float(eps), ptr(freqs_real), ptr(freqs_imag))
    with torch.cuda.device(dev):
        _check(L.lib().va_qk_norm_rope(C.byref(args), _stream()))
    return as_heads(q_out, heads), as_heads(k_out, kv_heads)


def qk_head_norm_rope(query: torch.Tensor, key: torch.Tensor, q_weight: Optional[torch.Tensor],
                      k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor] = None,
                      sin: Optional[torch.Tensor] = None, txt_len: int = 0, *, inplace: bool = False
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The per-head form of the preparation (HunyuanVideo, eval/DiTEvalKit/models/hyvideo/attention.py:187-213):
    ``query`` (B, H, L, 128) and ``key`` (B, Hkv, L, 128) get an RMSNorm over their 128 elements with weights of
    128 elements (``None``: no norm), then the rotary embedding on interleaved pairs with per-element float32
    tables ``cos`` / ``sin`` (L - txt_len, 128) on all but the last ``txt_len`` tokens (``None``: no rotation).
    One pass; ``inplace=True`` overwrites the inputs.  Returns (query, key) in the same (B, H, L, 128) layout."""
    dev = _require_cuda(query, key)
    b, h, l, d = query.shape
    hkv = key.shape[1]
    if d != 128 or key.shape[0] != b or key.shape[2] != l or key.shape[3] != 128 or query.dtype != key.dtype:
        raise VecAttentionArgumentError("query / key must be (B, H, L, 128) and (B, Hkv, L, 128) of one dtype")
    query, key = _rows_ok(query), _rows_ok(key)
    q_out = query if inplace else torch.empty_like(query, memory_format=torch.contiguous_format)
    k_out = key if inplace else torch.empty_like(key, memory_format=torch.contiguous_format)
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != query.dtype or w.numel() != 128 or not w.is_contiguous()):
            raise VecAttentionArgumentError("norm weights must be contiguous, of 128 elements and of the tensors' dtype")
    if (cos is None) != (sin is None):
        raise VecAttentionArgumentError("give both rotary tables or neither")
    rope_len = max(0, l - int(txt_len)) if cos is not None else 0
    if cos is not None:
        for f in (cos, sin):
            if f.dtype != torch.float32 or f.dim() != 2 or f.shape[0] < rope_len or f.shape[1] != 128 or not f.is_contiguous():
                raise VecAttentionArgumentError(f"rotary tables must be contiguous float32 of shape (>= {rope_len}, 128)")
    ptr = lambda t: t.data_ptr() if t is not None else None
    args = L.HeadNormRopeArgs(_dtype_code(query), b, l, h, hkv, rope_len, _t4(query), _t4(key), _t4(q_out), _t4(k_out),
                              ptr(q_weight), ptr(k_weight), float(eps), ptr(cos), ptr(sin))
    with torch.cuda.device(dev):
        _check(L.lib().va_qk_head_norm_rope(C.byref(args), _stream()))
    return q_out, k_out

