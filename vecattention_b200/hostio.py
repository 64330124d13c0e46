"""The prefill operator for callers whose q, k and v live in host memory.

The reference's callers hold their activations on the GPU already; a caller that does not (an
offloaded KV cache, a benchmark that starts from host buffers) pays the PCIe transfers, which for
this operator take several times longer than the kernels.  Every (batch, query head) is
independent, so the transfers are hidden the same way heads are sharded over GPUs: the heads are
cut into slices of whole KV groups and three streams work on them as a pipeline -- slice i + 1 is
copied in while slice i is computed and the output of slice i - 1 is copied out, with two sets of
device staging buffers.  The result equals one call of ``VecAttention_prefill`` on all heads.
"""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch

from .api import VecAttention_prefill, VecAttentionArgumentError
from .sharding import head_partition


def head_slices(heads: int, kv_heads: int, slices: int) -> List[Tuple[int, int]]:
    """Query-head ranges [h0, h1) of the pipeline's slices: whole KV groups, no empty slice."""
    slices = max(1, min(slices, kv_heads))
    return [r for r in head_partition(heads, kv_heads, slices) if r[1] > r[0]]


def VecAttention_prefill_host(
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
    out: Optional[torch.Tensor] = None,
    device: Union[str, torch.device, None] = None,
    slices: int = 24,
    compat_q1: bool = True,
    staging: Optional[dict] = None,
) -> torch.Tensor:
    """``VecAttention_prefill`` for host tensors (pinned memory gives asynchronous copies; pageable
    memory works but serialises).  ``out`` is a host tensor (allocated pinned if omitted) that is
    complete when the function returns.  ``slices`` is the number of pipeline stages the heads are
    cut into (at most one per KV group).  ``staging`` may carry the device buffers from call to
    call (a dict owned by the caller, filled on first use) so that repeated calls allocate nothing.
    """
    if query_states.is_cuda or key_states.is_cuda or value_states.is_cuda:
        raise VecAttentionArgumentError("VecAttention_prefill_host takes host tensors; use VecAttention_prefill")
    if not torch.cuda.is_available():
        raise RuntimeError("vecattention_b200 needs a CUDA device; there is no CPU path")
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    b, h, sq, d = query_states.shape
    hkv, sk = key_states.shape[1], key_states.shape[2]
    if h % hkv != 0 or value_states.shape != key_states.shape:
        raise VecAttentionArgumentError("inconsistent head counts or k/v shapes")
    rep = h // hkv
    if out is None:
        out = torch.empty((b, h, sq, d), dtype=query_states.dtype).pin_memory()
    parts = head_slices(h, hkv, slices)
    widest = max(h1 - h0 for h0, h1 in parts)
    per_head_thr = isinstance(threshold, torch.Tensor) and threshold.numel() == h
    if per_head_thr:
        threshold = threshold.reshape(-1).to(dev)

    st = staging if staging is not None else {}
    key = (str(dev), b, widest, rep, sq, sk, d, query_states.dtype)
    if st.get("key") != key:
        with torch.cuda.device(dev):
            st.clear()
            st["key"] = key
            st["q"] = [torch.empty((b, widest, sq, d), dtype=query_states.dtype, device=dev) for _ in range(2)]
            st["k"] = [torch.empty((b, widest // rep, sk, d), dtype=query_states.dtype, device=dev) for _ in range(2)]
            st["v"] = [torch.empty_like(st["k"][0]) for _ in range(2)]
            st["o"] = [torch.empty_like(st["q"][0]) for _ in range(2)]
            st["streams"] = [torch.cuda.Stream(device=dev) for _ in range(3)]
    s_in, s_run, s_out = st["streams"]
    with torch.cuda.device(dev):
        start = torch.cuda.Event()
        start.record()  # the side streams start after whatever the caller queued before
        for s in (s_in, s_run, s_out):
            s.wait_event(start)
        ran: List[Optional[torch.cuda.Event]] = [None, None]     # slot's inputs consumed
        copied: List[Optional[torch.cuda.Event]] = [None, None]  # slot's output copied to the host
        for i, (h0, h1) in enumerate(parts):
            slot, n = i & 1, h1 - h0
            qd, kd, vd, od = (st[name][slot][:, : (n if name in "qo" else n // rep)] for name in "qkvo")
            with torch.cuda.stream(s_in):
                if ran[slot] is not None:
                    s_in.wait_event(ran[slot])
                qd.copy_(query_states[:, h0:h1], non_blocking=True)
                kd.copy_(key_states[:, h0 // rep:h1 // rep], non_blocking=True)
                vd.copy_(value_states[:, h0 // rep:h1 // rep], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(arrived)
                if copied[slot] is not None:
                    s_run.wait_event(copied[slot])
                VecAttention_prefill(qd, kd, vd, threshold[h0:h1] if per_head_thr else threshold, q_pooling_size,
                                     k_local_size, group_k_block, causal, chunk_size, compat_q1=compat_q1, out=od)
                ran[slot] = torch.cuda.Event()
                ran[slot].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[slot])
                out[:, h0:h1].copy_(od, non_blocking=True)
                copied[slot] = torch.cuda.Event()
                copied[slot].record(s_out)
        # the caller's stream continues after the last copy; the host result needs a host wait
        cur = torch.cuda.current_stream(dev)
        for ev in copied:
            if ev is not None:
                cur.wait_event(ev)
        for ev in copied:
            if ev is not None:
                ev.synchronize()
    return out


def transfer_bytes(b: int, h: int, hkv: int, sq: int, sk: int, d: int, esz: int) -> Tuple[int, int]:
    """(host-to-device, device-to-host) bytes of one ``VecAttention_prefill_host`` call."""
    return (b * h * sq * d + 2 * b * hkv * sk * d) * esz, b * h * sq * d * esz
