"""Head sharding of the prefill operator across the GPUs of one node (one process per GPU).

Every (batch, query head) is independent in pooling, selection and attention, so the path has no
exchange step: a rank computes the heads it holds and nothing is communicated.  Heads are split
by KV group so that a query head and its KV head always live on the same rank.  The only
collective is the optional all-gather that reassembles the (B,H,S,D) output on every rank.

Failure handling.  A rank whose operator call raised must not leave the others waiting in the
all-gather: before the gather every rank contributes one "ok / failed" word to a small all-gather,
so all ranks learn of the failure on the host and raise ``ShardFailure`` together instead of
entering a collective with a missing participant.  A rank that died altogether surfaces on the
others as the process group's own error (connection closed, or its timeout).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def head_partition(heads: int, kv_heads: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous query-head ranges [h0, h1) per rank, whole KV groups only, sizes differing by
    at most one group.  Ranks beyond the number of groups get an empty range."""
    if heads % kv_heads != 0:
        raise ValueError("heads must be a multiple of kv_heads")
    rep = heads // kv_heads
    base, extra = divmod(kv_heads, world_size)
    out, g0 = [], 0
    for r in range(world_size):
        n = base + (1 if r < extra else 0)
        out.append((g0 * rep, (g0 + n) * rep))
        g0 += n
    return out


def local_slices(heads: int, kv_heads: int, rank: int, world_size: int) -> Tuple[slice, slice]:
    """(query-head slice, kv-head slice) of ``rank``."""
    h0, h1 = head_partition(heads, kv_heads, world_size)[rank]
    rep = heads // kv_heads
    return slice(h0, h1), slice(h0 // rep, h1 // rep)


def gather_heads(local: torch.Tensor, heads: int, kv_heads: int, group=None) -> torch.Tensor:
    """All-gather per-rank outputs (B,h_local,S,D) into (B,heads,S,D) on every rank."""
    world = dist.get_world_size(group)
    parts = head_partition(heads, kv_heads, world)
    widest = max(h1 - h0 for h0, h1 in parts)
    b, hl, s, d = local.shape
    send = local
    if hl != widest:
        send = local.new_zeros(b, widest, s, d)
        send[:, :hl] = local
    bufs = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(bufs, send.contiguous(), group=group)
    return torch.cat([buf[:, : h1 - h0] for buf, (h0, h1) in zip(bufs, parts)], dim=1)


class ShardFailure(RuntimeError):
    """Raised on every rank when the operator failed on some rank; ``ranks`` lists them."""

    def __init__(self, ranks: List[int], own: Optional[BaseException] = None):
        super().__init__(f"VecAttention prefill failed on rank(s) {ranks}; no output was gathered"
                         + (f" (this rank: {type(own).__name__}: {own})" if own is not None else ""))
        self.ranks = ranks


def agree_on_success(error: Optional[BaseException], group=None) -> None:
    """Every rank says whether its local work succeeded; if any did not, all raise ``ShardFailure``.
    The exchange is one small all-gather on the host side of the backend (CPU tensors for gloo, a
    device word for NCCL)."""
    world = dist.get_world_size(group)
    on_gpu = dist.get_backend(group) == "nccl"
    dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
    mine = torch.tensor([0 if error is None else 1], dtype=torch.int32, device=dev)
    words = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(words, mine, group=group)
    failed = [r for r, w in enumerate(words) if int(w.item()) != 0]
    if failed:
        raise ShardFailure(failed, error) from error


def prefill_head_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, threshold, *args,
                         total_heads: int, total_kv_heads: int, gather: bool = True, group=None,
                         prefill_fn: Optional[Callable] = None, **kwargs) -> torch.Tensor:
    """Run the operator on this rank's heads (``q``/``k``/``v`` hold only those) and optionally
    reassemble the full output.  A per-head ``threshold`` tensor is given for all heads and
    sliced here.  ``prefill_fn`` defaults to the CUDA operator.  With ``gather`` the ranks first
    agree that all of them succeeded (see the module text)."""
    if prefill_fn is None:
        from .api import VecAttention_prefill as prefill_fn
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    hs, _ = local_slices(total_heads, total_kv_heads, rank, world)
    if isinstance(threshold, torch.Tensor) and threshold.numel() == total_heads:
        threshold = threshold.reshape(-1)[hs]
    if q.shape[1] != hs.stop - hs.start:
        raise ValueError(f"rank {rank} holds {q.shape[1]} heads, partition says {hs.stop - hs.start}")
    if not gather:
        return prefill_fn(q, k, v, threshold, *args, **kwargs) if q.shape[1] else q.new_zeros(q.shape)
    out, error = None, None
    try:
        out = prefill_fn(q, k, v, threshold, *args, **kwargs) if q.shape[1] else q.new_zeros(q.shape)
    except Exception as e:  # noqa: BLE001 - reported to all ranks below
        error = e
    agree_on_success(error, group)
    return gather_heads(out, total_heads, total_kv_heads, group)
