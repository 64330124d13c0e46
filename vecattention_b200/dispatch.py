"""The prefill dispatcher model adapters call, for the methods this package serves
(spattn/src/models/utils.py:46-171): ``customize_prefill_attention(self, q, k, v, ...,
config=FastPrefillConfig())`` picks the layer's threshold, applies the vision-slice composition
for ``metric="vecattention"`` or runs dense attention for ``metric="full"``, records the call's
device time as a pair of CUDA events on a thread-local list, and optionally dumps Q/K for the
threshold tuner.  The reference's other methods (xattn, flex, anchor) are separate baselines and
raise ``NotImplementedError`` here.

Dense attention ("full") runs on the vector-sparse kernel with block tables that list every
64-key block a tile may see; the reference calls flashinfer there (spattn/src/Fullprefill.py).
"""
from __future__ import annotations

import math
import os
import threading

import torch

from .api import VecAttentionArgumentError, _sparse_attn_bhsd
from .config import FastPrefillConfig
from .vision import VecAttention_prefill_vision

SPARSITY_RECORD = threading.local()  # .attention_latency_list: [(start event, end event), ...] of this thread's calls


def Full_prefill(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor, causal: bool = True
                 ) -> torch.Tensor:
    """Dense softmax attention, (B,H,S,D) in and out; causal rows see the keys up to their own position
    counted from the end of the keys (bottom-right aligned, as the reference's library call is)."""
    b, h, sq, _ = query_states.shape
    sk = key_states.shape[2]
    dev = query_states.device
    nq = math.ceil(sq / 64)
    q_off = sk - sq if causal else 0
    if causal and q_off < 0:
        raise VecAttentionArgumentError("causal dense attention needs at least as many keys as queries")
    if causal and q_off == 0:  # every tile is a table-free dense tile of the kernel's vision-slice mode
        none = torch.zeros(b, h, nq, dtype=torch.int32, device=dev)
        return _sparse_attn_bhsd(query_states, key_states, value_states, 64, None, None, none,
                                 torch.zeros(b, h, nq, 4, dtype=torch.int32, device=dev), True, vision=(sq, sq))
    last_key = (torch.clamp(q_off + (torch.arange(nq, device=dev) + 1) * 64, max=q_off + sq) - 1) if causal else \
        torch.full((nq,), sk - 1, device=dev)
    count = (last_key // 64 + 1).to(torch.int32)
    width = (sk - 1) // 64 + 1
    start = (torch.arange(width, device=dev, dtype=torch.int32) * 64).expand(b, h, nq, width).contiguous()
    none = torch.zeros(b, h, nq, dtype=torch.int32, device=dev)
    return _sparse_attn_bhsd(query_states, key_states, value_states, 64, count.view(1, 1, nq).expand(b, h, nq).contiguous(),
                             start, none, torch.zeros(b, h, nq, 4, dtype=torch.int32, device=dev), causal, q_offset=q_off)


def customize_prefill_attention(self, query_states, key_states, value_states, attention_mask=None, position_ids=None,
                                causal: bool = True, config: FastPrefillConfig = None) -> torch.Tensor:
    """Prefill attention of one layer.  ``self`` is the attention module (its ``layer_idx`` picks the
    row of a per-layer threshold tensor and names Q/K dumps); tensors are (B,H,S,D)."""
    config = config if config is not None else FastPrefillConfig()
    if not (causal or config.metric in ("full", "xattn", "vecattention")):
        raise VecAttentionArgumentError(
            f"Non-causal attention only supports full, xattn, or vecattention metrics. Got: {config.metric}.")
    events = None
    if config.output_time and query_states.is_cuda:
        events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        events[0].record(torch.cuda.current_stream(query_states.device))

    if config.metric == "vecattention":
        threshold = config.threshold[self.layer_idx] if isinstance(config.threshold, torch.Tensor) else config.threshold
        out = VecAttention_prefill_vision(query_states, key_states, value_states, threshold, config.block_size_q,
                                          config.block_size_k, config.group_k_block, causal, config.chunk_size,
                                          vision_start_position=config.vision_start_position,
                                          vision_end_position=config.vision_end_position)
    elif config.metric == "full":
        out = Full_prefill(query_states, key_states, value_states, causal=causal)
    elif config.metric in ("xattn", "flex", "anchor"):
        raise NotImplementedError(f"attention metric {config.metric!r} is one of the reference's comparison baselines; "
                                  "this package serves 'vecattention' and 'full'")
    else:
        raise NotImplementedError(f"Unknown attention metric: {config.metric}")

    if events is not None:
        events[1].record(torch.cuda.current_stream(query_states.device))
        if not hasattr(SPARSITY_RECORD, "attention_latency_list"):
            SPARSITY_RECORD.attention_latency_list = []
        SPARSITY_RECORD.attention_latency_list.append(events)
    if config.dump_qk_dir:
        folder = os.path.join(config.dump_qk_dir, config.input_id)
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, f"layer_{self.layer_idx}_qk.pt")
        if not os.path.exists(path):
            torch.save({"query_states": query_states, "key_states": key_states}, path)
    return out
