"""Randomised differential test: the whole operator on the GPU against the CPU oracle over seeded
random small configurations (batch, GQA ratio, ragged lengths, both tile heights, every
k_local_size, small and whole-sequence key groups, causal or not, chunk sizes that do and do not
cover the sequence, scalar and per-head thresholds, bf16 and fp16).  The fixed cases elsewhere pin
named situations; this one looks for combinations nobody thought of.  Needs a B200: ``-m gpu``.
"""
import random

import pytest
import torch

from oracle import vecattn_oracle as O
from parity_util import MAX_ABS, MEAN_ABS

pytestmark = pytest.mark.gpu


def _draw(seed: int) -> dict:
    r = random.Random(seed)
    pq = r.choice([64, 128])
    causal = r.random() < 0.5
    bk = r.choice([b for b in (16, 32, 64, 128) if not causal or pq % b == 0])
    hkv = r.choice([1, 2])
    rep = r.choice([1, 1, 2, 3])
    s = r.choice([r.randint(65, 400), r.randint(400, 1600), r.choice([256, 512, 1024, 1152])])
    chunk = pq * r.choice([1, 2, 4, 8, 64])
    per_head = r.random() < 0.3
    b = 1 if per_head else r.choice([1, 1, 2])  # a per-head tensor is indexed by head only
    th = [round(r.uniform(0.3, 0.9), 3) for _ in range(hkv * rep)] if per_head else round(r.uniform(0.3, 0.9), 3)
    return dict(b=b, h=hkv * rep, hkv=hkv, s=s, pq=pq, bk=bk, g=r.choice([1, 2, 16, 8192]), causal=causal, chunk=chunk,
                th=th, dtype=r.choice([torch.bfloat16, torch.float16]), stripe=r.choice([7, 31, 97]))


@pytest.mark.parametrize("seed", range(64))
def test_random_configuration_matches_oracle(built_library, seed):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import vecattention_b200 as va
    cfg = _draw(1000 + seed)
    g = torch.Generator().manual_seed(seed)
    mk = lambda heads: torch.randn(cfg["b"], heads, cfg["s"], 128, generator=g).to(cfg["dtype"])
    q, k, v = mk(cfg["h"]), mk(cfg["hkv"]), mk(cfg["hkv"])
    k[:, :, ::cfg["stripe"]] *= 3.0  # a few dominant keys, so that the running maximum matters
    th = torch.tensor(cfg["th"], dtype=torch.float32) if isinstance(cfg["th"], list) else cfg["th"]
    ref, sel = O.vecattention_prefill(q, k, v, th, cfg["pq"], cfg["bk"], cfg["g"], cfg["causal"], cfg["chunk"],
                                      return_selection=True)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, counts = va.VecAttention_prefill(q.cuda(), k.cuda(), v.cuda(), th.cuda() if isinstance(th, torch.Tensor) else th,
                                          cfg["pq"], cfg["bk"], cfg["g"], cfg["causal"], cfg["chunk"],
                                          return_selection=True, status=status)
    assert int(status.item()) == 0, f"{cfg}: a kernel reported overflow or an internal timeout"
    ref_counts = torch.cat([c for c, _ in sel], dim=2)
    # a key whose estimate sits on the keep/drop boundary may flip a count by one; anything else is a bug
    assert (counts.cpu() - ref_counts).abs().sum() <= 2, cfg
    assert torch.isfinite(out.float()).all(), cfg
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (cfg, err.max().item(), err.mean().item())
