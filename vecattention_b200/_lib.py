"""ctypes binding of ``libvecattn.so`` (declarations mirror ``include/vecattn.h``).

There is no fallback: if the library is missing or fails to load, ``lib()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libvecattn.so")

VA_BF16, VA_FP16 = 0, 1
VA_STATUS_OVERFLOW = 1
VA_STATUS_TIMEOUT = 2

# every symbol include/vecattn.h declares
EXPORTS = ("va_pool_q", "va_select", "va_select_workspace_bytes", "va_sparse_attn", "va_sparse_attn_workspace_bytes",
           "va_block_tables", "va_prefill_workspace_bytes", "va_prefill", "va_prefill_static", "va_prefill_static_fits",
           "va_selftest_wait_timeout", "va_qk_norm_rope", "va_qk_head_norm_rope", "va_status_string", "va_version")
VA_SINGLE_PASS_INDEX_BYTES_DEFAULT = 4 << 30
VA_STATIC_SCRATCH_BYTES = 32 << 20


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class PoolArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32), ("seq_len", C.c_int32),
                ("head_dim", C.c_int32), ("pq", C.c_int32), ("q", Tensor4), ("out", C.c_void_p)]


class SelectArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("nq", C.c_int32), ("sk", C.c_int32), ("head_dim", C.c_int32),
                ("pq", C.c_int32), ("bk", C.c_int32), ("group_k_block", C.c_int32),
                ("causal", C.c_int32), ("wo_initial", C.c_int32), ("compat_bsq", C.c_int32),
                ("tile_offset", C.c_int32),
                ("avg_q", C.c_void_p), ("k", Tensor4), ("gap", C.c_float), ("gaps", C.c_void_p),
                ("gaps_stride_b", C.c_int64), ("col_count", C.c_void_p), ("col_idx", C.c_void_p),
                ("capacity", C.c_int64), ("status", C.c_void_p), ("chunk_tiles", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class AttnArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("sq", C.c_int32), ("sk", C.c_int32), ("head_dim", C.c_int32), ("pq", C.c_int32),
                ("causal", C.c_int32), ("q_offset", C.c_int32),
                ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("out", Tensor4),
                ("blk_count", C.c_void_p), ("blk_idx", C.c_void_p), ("blk_stride", C.c_int64),
                ("col_count", C.c_void_p), ("col_idx", C.c_void_p), ("col_stride", C.c_int64),
                ("softmax_scale", C.c_float), ("status", C.c_void_p), ("lse", C.c_void_p),
                ("vision_mode", C.c_int32), ("vision_begin", C.c_int32), ("vision_end", C.c_int32)]


class PrefillArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("sq", C.c_int32), ("sk", C.c_int32), ("head_dim", C.c_int32),
                ("pq", C.c_int32), ("bk", C.c_int32), ("group_k_block", C.c_int32), ("causal", C.c_int32),
                ("chunk_size", C.c_int32), ("compat_bsq", C.c_int32),
                ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("out", Tensor4),
                ("gap", C.c_float), ("gaps", C.c_void_p), ("gaps_stride_b", C.c_int64),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("col_count_out", C.c_void_p), ("status", C.c_void_p), ("single_pass_budget", C.c_size_t)]


class NormRopeArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("seq_len", C.c_int32), ("heads", C.c_int32),
                ("kv_heads", C.c_int32), ("rope_skip", C.c_int32),
                ("q", C.c_void_p), ("k", C.c_void_p), ("q_row_stride", C.c_int64), ("k_row_stride", C.c_int64),
                ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("q_out_row_stride", C.c_int64), ("k_out_row_stride", C.c_int64),
                ("q_weight", C.c_void_p), ("k_weight", C.c_void_p), ("eps", C.c_float),
                ("cos", C.c_void_p), ("sin", C.c_void_p)]


class HeadNormRopeArgs(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("seq_len", C.c_int32), ("heads", C.c_int32),
                ("kv_heads", C.c_int32), ("rope_len", C.c_int32),
                ("q", Tensor4), ("k", Tensor4), ("q_out", Tensor4), ("k_out", Tensor4),
                ("q_weight", C.c_void_p), ("k_weight", C.c_void_p), ("eps", C.c_float),
                ("cos", C.c_void_p), ("sin", C.c_void_p)]


_LIB = None


def lib() -> C.CDLL:
    """Load the library once.  Raises ``RuntimeError`` if it is absent or lacks a symbol."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m vecattention_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for this path)")
    handle = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(handle, name):
            raise RuntimeError(f"{LIB_PATH} does not export {name}")
    handle.va_pool_q.argtypes = [C.POINTER(PoolArgs), C.c_void_p]
    handle.va_select.argtypes = [C.POINTER(SelectArgs), C.c_void_p]
    handle.va_sparse_attn.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
    handle.va_select_workspace_bytes.argtypes = [C.POINTER(SelectArgs), C.POINTER(C.c_size_t)]
    handle.va_sparse_attn_workspace_bytes.argtypes = [C.POINTER(AttnArgs), C.POINTER(C.c_size_t)]
    handle.va_block_tables.argtypes = [C.c_int32] * 5 + [C.c_void_p, C.c_void_p, C.c_void_p]
    handle.va_prefill_workspace_bytes.argtypes = [C.POINTER(PrefillArgs), C.POINTER(C.c_size_t)]
    handle.va_prefill.argtypes = [C.POINTER(PrefillArgs), C.c_void_p]
    handle.va_prefill_static.argtypes = [C.POINTER(PrefillArgs), C.c_void_p]
    handle.va_prefill_static_fits.argtypes = [C.POINTER(PrefillArgs)]
    handle.va_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    handle.va_qk_norm_rope.argtypes = [C.POINTER(NormRopeArgs), C.c_void_p]
    handle.va_qk_head_norm_rope.argtypes = [C.POINTER(HeadNormRopeArgs), C.c_void_p]
    for name in EXPORTS:
        getattr(handle, name).restype = C.c_int
    handle.va_status_string.argtypes = [C.c_int]
    handle.va_status_string.restype = C.c_char_p
    handle.va_version.argtypes = []
    _LIB = handle
    return handle


def status_string(code: int) -> str:
    return lib().va_status_string(code).decode()
