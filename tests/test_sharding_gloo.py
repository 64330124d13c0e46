"""Head sharding on two CPU ranks (gloo): partitioning, per-head threshold slicing and the
output all-gather, with the CPU oracle standing in for the CUDA operator."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vecattention_b200.sharding import head_partition, local_slices


def test_head_partition():
    assert head_partition(24, 24, 8) == [(3 * r, 3 * r + 3) for r in range(8)]
    assert head_partition(28, 4, 2) == [(0, 14), (14, 28)]
    assert head_partition(28, 4, 4) == [(7 * r, 7 * r + 7) for r in range(4)]
    parts = head_partition(40, 40, 8)
    assert parts[0] == (0, 5) and parts[-1] == (35, 40) and sum(b - a for a, b in parts) == 40
    parts = head_partition(28, 4, 8)           # more ranks than KV groups: empty tails
    assert parts[3] == (21, 28) and parts[4] == (28, 28)
    assert local_slices(28, 4, 1, 2) == (slice(14, 28), slice(2, 4))
    with pytest.raises(ValueError):
        head_partition(10, 4, 2)


def _worker(rank, world, port, heads, kv_heads, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import vecattn_oracle as O
        from vecattention_b200.sharding import prefill_head_sharded
        g = torch.Generator().manual_seed(3)
        q = torch.randn(1, heads, 320, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(1, kv_heads, 320, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(1, kv_heads, 320, 128, generator=g).to(torch.bfloat16)
        th = torch.linspace(0.3, 0.8, heads)
        hs, ks = local_slices(heads, kv_heads, rank, world)
        out = prefill_head_sharded(q[:, hs], k[:, ks], v[:, ks], th, 64, 16, 4, True, 128,
                                   total_heads=heads, total_kv_heads=kv_heads,
                                   prefill_fn=O.vecattention_prefill)
        full = O.vecattention_prefill(q, k, v, th, 64, 16, 4, True, 128)
        results[rank] = bool(torch.equal(out, full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads,kv_heads", [(4, 4), (6, 3)])
def test_two_rank_head_sharding_equals_single_rank(heads, kv_heads):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, heads, kv_heads, results), nprocs=2, join=True)
    assert results[0] and results[1]
