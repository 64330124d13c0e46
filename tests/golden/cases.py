"""Seeded inputs of the golden cases, shared by ``make_golden.py`` (which runs the reference
on them) and by the tests (which run the oracle and the CUDA path on them).

Inputs come from ``numpy.random.RandomState`` (a frozen stream) and are rounded to bf16 (or
fp16) precision, so the same values can be fed to an fp32 run and to a 16-bit run.
"""
from __future__ import annotations

import hashlib
import math

import numpy as np
import torch

# name -> parameters.  ``dtype`` is the precision the reference was run in.
CASES = {
    # BASELINE config 1: B1 H4 S2048 D128 fp32 non-causal, 32 stripe key rows per head x4.
    "c1_g8192": dict(seed=0, b=1, h=4, hkv=4, sq=2048, sk=2048, pq=64, bk=16, g=8192, causal=False,
                     stripes=32, stripe_scale=4.0, keep=0.10, dtype="fp32"),
    "c1_g16": dict(seed=0, b=1, h=4, hkv=4, sq=2048, sk=2048, pq=64, bk=16, g=16, causal=False,
                   stripes=32, stripe_scale=4.0, keep=0.10, dtype="fp32"),
    # ragged last query tile (48 rows), Sk % 64 != 0, Sk % Bk == 0
    "ragged_nc": dict(seed=11, b=1, h=2, hkv=2, sq=1008, sk=1008, pq=64, bk=16, g=4, causal=False,
                      stripes=8, stripe_scale=4.0, keep=0.15, dtype="fp32"),
    "ragged_causal": dict(seed=12, b=1, h=2, hkv=2, sq=1008, sk=1008, pq=64, bk=16, g=16, causal=True,
                          stripes=8, stripe_scale=4.0, keep=0.2, dtype="fp32"),
    # Sq != Sk, q_pooling_size 128, k_local_size 32
    "sq_ne_sk_p128": dict(seed=13, b=2, h=2, hkv=2, sq=384, sk=1120, pq=128, bk=32, g=8192, causal=False,
                          stripes=8, stripe_scale=4.0, keep=0.1, dtype="fp32"),
    # per-head threshold tensor
    "per_head": dict(seed=14, b=1, h=3, hkv=3, sq=512, sk=512, pq=64, bk=16, g=2, causal=False,
                     stripes=8, stripe_scale=4.0, keep=(0.05, 0.15, 0.3), dtype="fp32"),
    # 16-bit inputs (the interpreter has fp16 but no bf16)
    "fp16_nc": dict(seed=15, b=1, h=2, hkv=2, sq=512, sk=768, pq=64, bk=16, g=8, causal=False,
                    stripes=8, stripe_scale=4.0, keep=0.12, dtype="fp16"),
    # causal, 66 tiles: tile 64 is the first row of the second 64-row Triton program
    "causal_q1": dict(seed=16, b=1, h=1, hkv=1, sq=4224, sk=4224, pq=64, bk=16, g=16, causal=True,
                      stripes=40, stripe_scale=4.0, keep=0.1, dtype="fp32"),
}

# whole-operator captures: VecAttention_prefill run with a recording stand-in for the
# absent sparse_attn_func; pins chunk loop, block tables and the arguments of every call.
OPERATOR_CASES = {
    "op_causal_chunked": dict(seed=21, b=1, h=2, hkv=2, sq=1200, sk=1200, pq=64, bk=16, g=16, causal=True,
                              stripes=8, stripe_scale=4.0, threshold=0.5, chunk=512, dtype="fp32"),
    "op_nc_chunked": dict(seed=22, b=1, h=2, hkv=2, sq=640, sk=640, pq=128, bk=16, g=8192, causal=False,
                          stripes=8, stripe_scale=4.0, threshold=0.6, chunk=256, dtype="fp32"),
}


def _round16(x: np.ndarray, dtype: str) -> torch.Tensor:
    t = torch.from_numpy(x.astype(np.float32))
    if dtype == "fp16":
        return t.to(torch.float16).float()
    return t.to(torch.bfloat16).float()


def make_inputs(p: dict):
    """q (B,H,Sq,D), k, v (B,Hkv,Sk,D) as fp32 tensors holding 16-bit-exact values."""
    rs = np.random.RandomState(p["seed"])
    d = 128
    q = rs.standard_normal((p["b"], p["h"], p["sq"], d))
    k = rs.standard_normal((p["b"], p["hkv"], p["sk"], d))
    v = rs.standard_normal((p["b"], p["hkv"], p["sk"], d))
    for b in range(p["b"]):
        for h in range(p["hkv"]):
            cols = rs.permutation(p["sk"])[: p["stripes"]]
            k[b, h, cols] *= p["stripe_scale"]
    kind = "fp16" if p["dtype"] == "fp16" else "bf16"
    return _round16(q, kind), _round16(k, kind), _round16(v, kind)


def input_digest(*tensors: torch.Tensor) -> str:
    hsh = hashlib.sha256()
    for t in tensors:
        hsh.update(t.contiguous().numpy().tobytes())
    return hsh.hexdigest()


def torch_dtype(name: str) -> torch.dtype:
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[name]


def calibrate_threshold(select_fn, avg_q, k, p: dict, keep: float, iters: int = 18) -> float:
    """Bisect the MinP threshold until the mean kept fraction of eligible keys is ``keep``
    (the reference has no keep-ratio knob; its knob is the threshold)."""
    nq = avg_q.shape[2]
    if p["causal"]:
        elig = sum(max(0, min(p["sk"], g * p["pq"]) - p["pq"]) for g in range(nq))
    else:
        elig = nq * p["sk"]
    elig = max(elig, 1) * avg_q.shape[0] * avg_q.shape[1]
    lo, hi = 1e-9, 1.0
    for _ in range(iters):
        mid = math.sqrt(lo * hi)
        cnt, _ = select_fn(avg_q, k, 0, -math.log(mid + 1e-9), p["causal"], p["pq"], p["bk"],
                           wo_initial=p["causal"], group_k_block=p["g"])
        if float(cnt.sum()) / elig > keep:
            lo = mid
        else:
            hi = mid
    return math.sqrt(lo * hi)
