"""The CPU oracle against fixtures produced by the reference's own code (tests/golden/*.npz,
made by tests/golden/make_golden.py).  No GPU needed."""
import math
import os

import numpy as np
import pytest
import torch

import cases as C
from oracle import vecattn_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    path = os.path.join(GOLDEN, f"{name}.npz")
    if not os.path.exists(path):
        pytest.fail(f"missing fixture {path}")
    return np.load(path)


def _rows_as_sets(count, index):
    cnt = np.asarray(count)
    idx = np.asarray(index)
    return {pos: set(idx[pos][: int(cnt[pos])].tolist()) for pos in np.ndindex(cnt.shape)}


@pytest.mark.parametrize("name", list(C.CASES))
def test_selection_matches_reference(name):
    p = C.CASES[name]
    g = _load(name)
    dt = C.torch_dtype(p["dtype"])
    q, k, _ = C.make_inputs(p)
    assert C.input_digest(q.to(dt).float(), k.to(dt).float()) == str(g["digest"]), "seeded inputs differ from the fixture's"
    q, k = q.to(dt), k.to(dt)

    # pooling: the reference's Triton kernel and its PyTorch fallback differ from each other only
    # in the association of the fp32 sum; the oracle's balanced tree must agree to fp32 rounding,
    # and in a 16-bit dtype to one unit in the last place on a vanishing fraction of elements.
    mine = O.pool_q(q, p["pq"]).float().numpy()
    for key in ("avg_triton", "avg_torch"):
        ref = g[key]
        if p["dtype"] == "fp32":
            np.testing.assert_allclose(mine, ref, rtol=0, atol=4e-7)
        else:
            diff = mine != ref
            assert diff.mean() < 2e-3
            np.testing.assert_allclose(mine, ref, rtol=2e-3, atol=1e-6)

    # selection: fed with the reference's own pooled queries the kept sets must be identical
    avg = torch.from_numpy(g["avg_triton"]).to(dt)
    gap = g["gap"]
    gap = torch.from_numpy(gap).float() if gap.ndim else float(gap)
    cnt, idx, amb = O.select_columns(avg, k, 0, gap, p["causal"], p["pq"], p["bk"], wo_initial=p["causal"],
                                     group_k_block=p["g"], return_ambiguous=True,
                                     scale_in_dtype=(p["dtype"] == "fp16"))
    ref_sets = _rows_as_sets(g["count"], g["index"])
    my_sets = _rows_as_sets(cnt.numpy(), idx.numpy())
    n_amb = 0
    for (b, h, r), ref in ref_sets.items():
        diff = ref ^ my_sets[(b, h, r)]
        allowed = set(amb[b * p["h"] + h][r].tolist())
        assert diff <= allowed, f"{name} row {(b, h, r)}: {sorted(diff - allowed)[:8]} differ away from the boundary"
        n_amb += len(diff)
    # fp32 accumulation order (numpy in the interpreter, MKL here) may flip boundary keys only
    assert n_amb <= 2, f"{n_amb} boundary keys differ"
    kept = float(np.asarray(g["count"]).sum())
    assert kept > 0


def test_causal_quirk_is_present_in_fixture():
    """Tile 64 is the first row of the second 64-row Triton program: the reference drops the
    last 48 keys before its diagonal tile (truncating division)."""
    p = C.CASES["causal_q1"]
    g = _load("causal_q1")
    _, hi = O.row_key_limits(66, 0, p["sk"], p["pq"], p["bk"], True, True)
    assert hi[64] == 63 * 64 + 16 and hi[63] == 63 * 64 and hi[65] == 65 * 64
    row = g["index"][0, 0, 64][: int(g["count"][0, 0, 64])]
    assert row.max() < 63 * 64 + 16


@pytest.mark.parametrize("name", list(C.OPERATOR_CASES))
def test_operator_arguments_match_reference(name):
    """VecAttention_prefill of the reference, run with a recording stand-in for the absent
    sparse_attn_func: chunk loop, block tables and selected columns of every call."""
    p = C.OPERATOR_CASES[name]
    g = _load(name)
    q, k, v = C.make_inputs(p)
    assert C.input_digest(q, k) == str(g["digest"])
    out, sel = O.vecattention_prefill(q, k, v, p["threshold"], p["pq"], p["bk"], p["g"], p["causal"], p["chunk"],
                                      return_selection=True)
    assert int(g["n_calls"]) == len(sel) == math.ceil(p["sq"] / p["chunk"])
    bc, bi = O.block_tables(p["b"], p["h"], p["sq"], p["pq"], p["causal"])
    for i, (cc, ci) in enumerate(sel):
        t0, t1 = i * p["chunk"] // p["pq"], (i + 1) * p["chunk"] // p["pq"]
        np.testing.assert_array_equal(bc[:, :, t0:t1].numpy(), g[f"blk_count{i}"])
        np.testing.assert_array_equal(bi[:, :, t0:t1].numpy(), g[f"blk_idx{i}"])
        # the reference pools with its Triton kernel (fp32 here), the oracle with its own tree: a
        # key whose estimate sits on the boundary may flip, nothing else
        ref_sets = _rows_as_sets(g[f"col_count{i}"], g[f"col_idx{i}"])
        my_sets = _rows_as_sets(cc.numpy(), ci.numpy())
        ndiff = sum(len(ref_sets[pos] ^ my_sets[pos]) for pos in ref_sets)
        total = sum(len(s) for s in ref_sets.values())
        assert ndiff <= max(2, 1e-4 * total), f"chunk {i}: {ndiff} of {total} selected keys differ"
        exp_q = (p["b"], min(p["chunk"], p["sq"] - i * p["chunk"]), p["h"], 128)
        assert tuple(g[f"q_shape{i}"]) == exp_q
        exp_k = min(p["sk"], (i + 1) * p["chunk"]) if p["causal"] else p["sk"]
        assert tuple(g[f"k_shape{i}"])[1] == exp_k
    assert torch.isfinite(out).all()
