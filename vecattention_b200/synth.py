"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (stand-ins for Qwen2.5-VL / Wan2.1 / HunyuanVideo activations, which need model
weights and datasets that are not available offline).

Every head is generated from its own seed, so a rank that holds only a slice of the heads
produces exactly the slice of the full tensor.  The reference has no keep-ratio knob: the
configurations' "keep ratio" is reached by calibrating the MinP threshold (bisection on the
selection counts, ``calibrate_threshold``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence

import torch


@dataclass
class Workload:
    name: str
    batch: int
    heads: int
    kv_heads: int
    seq_len: int
    causal: bool
    dtype: torch.dtype
    keep: float
    q_pooling_size: int = 64
    k_local_size: int = 16
    group_k_block: int = 16
    chunk_size: int = 32768
    seed: int = 0
    stripe_frac: float = 0.01
    sigma: float = 1.0
    frame: int = 0          # tokens per frame for the low-rank K structure (0 = none)
    sink: int = 0           # attention-sink prefix length
    q: Optional[torch.Tensor] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    extra: Dict = field(default_factory=dict)

    @property
    def nq(self) -> int:
        return math.ceil(self.seq_len / self.q_pooling_size)

    def eligible_pairs_per_head(self) -> int:
        """(query tile, key) pairs the selection may keep, per head."""
        pq, s = self.q_pooling_size, self.seq_len
        if not self.causal:
            return self.nq * s
        return sum(max(0, min(s, g * pq) - pq) for g in range(self.nq))


CONFIGS = {
    # BASELINE config 2: README quick-use shape
    "c2": dict(batch=1, heads=32, kv_heads=32, seq_len=32768, causal=False, keep=0.10, seed=1,
               stripe_frac=0.01, sigma=1.0, group_k_block=16, chunk_size=32768),
    # config 3: Wan-style video DiT, 21 frames x 3600 tokens
    "c3": dict(batch=1, heads=40, kv_heads=40, seq_len=75600, causal=False, keep=0.10, seed=2,
               stripe_frac=0.02, sigma=0.5, frame=3600, group_k_block=8192, chunk_size=32768),
    # config 4: HunyuanVideo-style, 33 frames x 3600 tokens
    "c4": dict(batch=1, heads=24, kv_heads=24, seq_len=118800, causal=False, keep=0.08, seed=3,
               stripe_frac=0.02, sigma=0.5, frame=3600, group_k_block=8192, chunk_size=32768),
    # config 5: Qwen2.5-VL-style GQA long-video prefill, causal
    "c5": dict(batch=1, heads=28, kv_heads=4, seq_len=65536, causal=True, keep=0.10, seed=4,
               stripe_frac=0.01, sigma=1.0, sink=4, group_k_block=16, chunk_size=65536),
    # the reference's default arguments (q_pooling_size 128, k_local_size 128, group_k_block 1, causal, chunks of
    # 16 K rows; spattn/src/VecAttention.py:14-18) on the quick-use shape
    "d128": dict(batch=1, heads=32, kv_heads=32, seq_len=32768, causal=True, keep=0.10, seed=1,
                 stripe_frac=0.01, sigma=1.0, q_pooling_size=128, k_local_size=128, group_k_block=1, chunk_size=16384),
    # 8 heads of config 2: inputs above the L2 size, small enough for a profiler capture
    "c2h8": dict(batch=1, heads=8, kv_heads=8, seq_len=32768, causal=False, keep=0.10, seed=1,
                 stripe_frac=0.01, sigma=1.0, group_k_block=16, chunk_size=32768),
    # small shape for smoke runs and profiler captures (same distribution as c2)
    "mini": dict(batch=1, heads=8, kv_heads=8, seq_len=8192, causal=False, keep=0.10, seed=1,
                 stripe_frac=0.01, sigma=1.0, group_k_block=16, chunk_size=32768),
}


def _head_kv(wl: Workload, kvh: int, device, gen_dev) -> Dict[str, torch.Tensor]:
    """K, V and the stripe direction of one KV head."""
    g = torch.Generator(device=gen_dev)
    g.manual_seed(wl.seed * 100003 + kvh)
    s, d = wl.seq_len, 128
    u = torch.randn(d, generator=g, device=gen_dev)
    u = u / u.norm()
    if wl.frame:
        nf = math.ceil(s / wl.frame)
        a = torch.randn(nf, wl.frame, 16, generator=g, device=gen_dev)
        bmat = torch.randn(nf, 16, d, generator=g, device=gen_dev)
        low = torch.bmm(a, bmat).reshape(nf * wl.frame, d)[:s] / 4.0
        k = wl.sigma * (0.8 * low + 0.6 * torch.randn(s, d, generator=g, device=gen_dev))
    else:
        k = wl.sigma * torch.randn(s, d, generator=g, device=gen_dev)
    v = wl.sigma * torch.randn(s, d, generator=g, device=gen_dev)
    n_stripe = max(1, int(round(wl.stripe_frac * s)))
    stripes = torch.randperm(s, generator=g, device=gen_dev)[:n_stripe]
    k[stripes] += 3.0 * wl.sigma * u
    if wl.sink:
        k[: wl.sink] += 3.0 * wl.sigma * u
    return dict(k=k, v=v, u=u)


def make_workload(name: str, device="cuda", heads: Optional[Sequence[int]] = None, keep: Optional[float] = None,
                  sample_seed: int = 0, **overrides) -> Workload:
    """Build configuration ``name`` on ``device``.  ``heads`` restricts the query heads generated
    (a contiguous range whose KV heads come along), ``sample_seed`` picks another draw of the
    same distribution."""
    cfg = dict(CONFIGS[name])
    cfg.update(overrides)
    if keep is not None:
        cfg["keep"] = keep
    wl = Workload(name=name, dtype=torch.bfloat16, **cfg)
    wl.seed = wl.seed + 7919 * sample_seed
    rep = wl.heads // wl.kv_heads
    hq = list(range(wl.heads)) if heads is None else list(heads)
    kvs = sorted({h // rep for h in hq})
    assert [h for kv in kvs for h in range(kv * rep, kv * rep + rep)] == hq, "head slice must cover whole KV groups"
    gen_dev = device
    s, d = wl.seq_len, 128
    q = torch.empty(wl.batch, len(hq), s, d, dtype=wl.dtype, device=device)
    k = torch.empty(wl.batch, len(kvs), s, d, dtype=wl.dtype, device=device)
    v = torch.empty_like(k)
    for b in range(wl.batch):
        for i, kvh in enumerate(kvs):
            kv = _head_kv(wl, kvh + 1000 * b, device, gen_dev)
            k[b, i] = kv["k"].to(wl.dtype)
            v[b, i] = kv["v"].to(wl.dtype)
            for j in range(rep):
                h = kvh * rep + j
                g = torch.Generator(device=gen_dev)
                g.manual_seed(wl.seed * 100003 + 50000 + h + 1000 * b)
                qq = wl.sigma * (torch.randn(s, d, generator=g, device=gen_dev) + kv["u"])
                q[b, i * rep + j] = qq.to(wl.dtype)
    wl.heads, wl.kv_heads = len(hq), len(kvs)
    wl.q, wl.k, wl.v = q, k, v
    return wl


def calibrate_threshold(wl: Workload, select_counts, iters: int = 14, max_heads: int = 4) -> float:
    """Bisect (geometrically) the MinP threshold so that the kept fraction of eligible
    (tile, key) pairs is ``wl.keep``.  ``select_counts(threshold, head_slice) -> int tensor`` runs
    the selection for the given query heads and returns the per-tile counts."""
    rep = wl.heads // wl.kv_heads
    nh = min(wl.heads, max(rep, max_heads // rep * rep))
    elig = wl.eligible_pairs_per_head() * nh * wl.batch
    lo, hi = 1e-9, 1.0
    for _ in range(iters):
        mid = math.sqrt(lo * hi)
        kept = float(select_counts(mid, slice(0, nh)).sum())
        if kept / elig > wl.keep:
            lo = mid
        else:
            hi = mid
    return math.sqrt(lo * hi)
