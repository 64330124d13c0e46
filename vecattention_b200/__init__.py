"""B200-native VecAttention prefill: the reference's operator API over hand-written sm_100a
CUDA kernels reached through the C ABI of ``libvecattn.so`` (see ``include/vecattn.h``)."""
from .api import (VecAttention_prefill, VecAttentionArgumentError, average_vector, block_tables,
                  fuse_qk_softmax_minp_wo_causal, sparse_attn_func)
from .config import FastPrefillConfig, add_fastprefill_args, build_output_file_from_config, get_fastprefill_config
from .dispatch import Full_prefill, customize_prefill_attention
from .hostio import VecAttention_prefill_host
from .vision import VecAttention_prefill_vision

__all__ = ["FastPrefillConfig", "add_fastprefill_args", "get_fastprefill_config", "build_output_file_from_config",
           "customize_prefill_attention", "Full_prefill", "VecAttention_prefill", "VecAttention_prefill_host", "VecAttention_prefill_vision", "VecAttentionArgumentError", "average_vector", "block_tables",
           "fuse_qk_softmax_minp_wo_causal", "sparse_attn_func"]
