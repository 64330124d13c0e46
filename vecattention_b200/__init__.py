"""B200-native VecAttention prefill: the reference's operator API over hand-written sm_100a
CUDA kernels reached through the C ABI of ``libvecattn.so`` (see ``include/vecattn.h``)."""
from .api import (VecAttention_prefill, VecAttentionArgumentError, average_vector, block_tables,
                  fuse_qk_softmax_minp_wo_causal, sparse_attn_func)
from .hostio import VecAttention_prefill_host
from .vision import VecAttention_prefill_vision

__all__ = ["VecAttention_prefill", "VecAttention_prefill_host", "VecAttention_prefill_vision", "VecAttentionArgumentError", "average_vector", "block_tables",
           "fuse_qk_softmax_minp_wo_causal", "sparse_attn_func"]
