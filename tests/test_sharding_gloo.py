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


# ---------------------------------------------------------------------------------------------
# A rank that fails before the gather: the others learn of it on the host and nobody hangs.
# ---------------------------------------------------------------------------------------------
def _failing_worker(rank, world, port, mode, results):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from oracle import vecattn_oracle as O
    from vecattention_b200.sharding import ShardFailure, prefill_head_sharded
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 2, 192, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 2, 192, 128, generator=g).to(torch.bfloat16)
    hs, ks = local_slices(2, 2, rank, world)

    def prefill(*a, **kw):
        if rank == 1 and mode == "raises":
            raise ValueError("injected failure on rank 1")
        return O.vecattention_prefill(*a, **kw)
    dist.barrier()
    if rank == 1 and mode == "exits":
        os._exit(3)   # the process is gone before the exchange: no goodbye to the group
    try:
        prefill_head_sharded(q[:, hs], k[:, ks], k[:, ks], 0.5, 64, 16, 4, True, 128, total_heads=2, total_kv_heads=2,
                             prefill_fn=prefill)
        results[rank] = "no error"
    except ShardFailure as e:
        results[rank] = f"ShardFailure {e.ranks}"
    except Exception as e:  # noqa: BLE001 - the process group's own error for a vanished peer
        results[rank] = f"group error {type(e).__name__}"
    os._exit(0)   # skip the group's teardown: the peer may be gone


@pytest.mark.parametrize("mode", ["raises", "exits"])
def test_failed_rank_is_reported_to_the_others_without_a_hang(mode):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    results = mgr.dict()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, mode, results)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=90)
    alive = [pr.is_alive() for pr in procs]
    for pr in procs:
        if pr.is_alive():
            pr.kill()
    assert not any(alive), "a rank hung after its peer failed"
    if mode == "raises":
        assert results[0] == "ShardFailure [1]" and results[1] == "ShardFailure [1]", dict(results)
    else:
        assert procs[1].exitcode == 3
        assert results[0].startswith("group error") or results[0].startswith("ShardFailure"), dict(results)
