"""Generate the golden fixtures in this directory by running the REFERENCE's own code.

Usage (only where the reference checkout is present; it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/VecAttention [case ...]

What runs: the reference's ``average_vector`` (Triton pooling kernel) and
``fuse_qk_softmax_minp_wo_causal`` (Triton selection kernels), executed on CPU tensors by
the Triton interpreter (``TRITON_INTERPRET=1``), and ``VecAttention_prefill`` itself with a
recording stand-in for ``vllm_flash_attn.sparse_attn_func`` (whose source is not part of the
reference tree).  Nothing from the oracle produces the stored outputs; the oracle is used
only to calibrate thresholds to a keep ratio before the reference is run.

The interpreter cannot run bf16 and (unlike compiled Triton) multiplies a 16-bit tensor by
a Python scalar in 16-bit, so: fp32 cases pin the selection rule exactly; the fp16 case
pins the 16-bit data flow with the scale applied in fp16 (``scale_in_dtype`` in the test).
"""
from __future__ import annotations

import os
import sys
import time
import types

os.environ["TRITON_INTERPRET"] = "1"

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import cases as C  # noqa: E402


def _load_reference(ref_root: str):
    sys.path.insert(0, ref_root)
    stub = types.ModuleType("vllm_flash_attn")
    stub.calls = []

    def sparse_attn_func(q, k, v, pq, blk_count, blk_idx, col_count, col_idx,
                         return_softmax_lse=False, causal=False):
        stub.calls.append(dict(q_shape=tuple(q.shape), k_shape=tuple(k.shape), pq=pq,
                               blk_count=blk_count.clone(), blk_idx=blk_idx.clone(),
                               col_count=col_count.clone(), col_idx=col_idx.clone(), causal=causal))
        return torch.zeros_like(q)

    stub.sparse_attn_func = sparse_attn_func
    sys.modules["vllm_flash_attn"] = stub
    from spattn.src.utils import average_vector
    from spattn.src.kernels.vecattention_kernels import fuse_qk_softmax_minp_wo_causal
    from spattn.src.VecAttention import VecAttention_prefill
    return stub, average_vector, fuse_qk_softmax_minp_wo_causal, VecAttention_prefill


def _sorted_rows(count: torch.Tensor, index: torch.Tensor) -> np.ndarray:
    """(B,H,nq,maxc) -> same shape, every row's first count entries sorted, rest -1."""
    cnt = count.numpy()
    idx = index.numpy()
    out = np.full(idx.shape, -1, dtype=np.int32)
    for pos in np.ndindex(cnt.shape):
        c = int(cnt[pos])
        out[pos][:c] = np.sort(idx[pos][:c])
    return out


def main():
    ref_root = sys.argv[1]
    want = sys.argv[2:]
    stub, average_vector, select_ref, prefill_ref = _load_reference(ref_root)
    from oracle import vecattn_oracle as O

    for name, p in C.CASES.items():
        if want and name not in want:
            continue
        t0 = time.time()
        dt = C.torch_dtype(p["dtype"])
        q, k, v = C.make_inputs(p)
        q, k = q.to(dt), k.to(dt)
        avg_triton = average_vector(q, p["pq"], use_triton=True)
        avg_torch = average_vector(q, p["pq"], use_triton=False)
        keep = p["keep"]
        if isinstance(keep, tuple):
            ths = [C.calibrate_threshold(O.select_columns, avg_triton[:, h:h + 1], k[:, h:h + 1], p, kp)
                   for h, kp in enumerate(keep)]
            threshold = torch.tensor(ths, dtype=torch.float32)
            gap = -torch.log(threshold + 1e-9)
        else:
            threshold = C.calibrate_threshold(O.select_columns, avg_triton, k, p, keep)
            gap = -np.log(threshold + 1e-9).item()
        cnt, idx = select_ref(avg_triton, k, 0, gap, p["causal"], p["pq"], p["bk"],
                              wo_initial=p["causal"], group_k_block=p["g"])
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            digest=C.input_digest(q.float(), k.float()),
            threshold=np.asarray(threshold, dtype=np.float64),
            gap=np.asarray(gap, dtype=np.float64),
            avg_triton=avg_triton.float().numpy(), avg_torch=avg_torch.float().numpy(),
            count=cnt.numpy(), index=_sorted_rows(cnt, idx))
        print(f"{name}: kept {float(cnt.sum()) / cnt.numel() / p['sk']:.4f} of keys, "
              f"{time.time() - t0:.0f}s", flush=True)

    for name, p in C.OPERATOR_CASES.items():
        if want and name not in want:
            continue
        t0 = time.time()
        q, k, v = C.make_inputs(p)
        stub.calls.clear()
        prefill_ref(q, k, v, p["threshold"], p["pq"], p["bk"], p["g"], p["causal"], p["chunk"])
        rec = dict(digest=C.input_digest(q, k), n_calls=len(stub.calls))
        for i, c in enumerate(stub.calls):
            rec[f"q_shape{i}"] = np.asarray(c["q_shape"])
            rec[f"k_shape{i}"] = np.asarray(c["k_shape"])
            rec[f"blk_count{i}"] = c["blk_count"].numpy()
            rec[f"blk_idx{i}"] = c["blk_idx"].numpy()
            rec[f"col_count{i}"] = c["col_count"].numpy()
            rec[f"col_idx{i}"] = _sorted_rows(c["col_count"], c["col_idx"])
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **rec)
        print(f"{name}: {len(stub.calls)} chunks, {time.time() - t0:.0f}s", flush=True)


if __name__ == "__main__":
    main()
