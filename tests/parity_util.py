"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

MAX_ABS, MEAN_ABS = 2e-2, 2e-3   # bf16/fp16 output tolerance against the fp32 oracle


def check_selection(cnt_gpu, idx_gpu, cnt_ref, idx_ref, amb, heads, sk, max_flips=None):
    """Per row: the CUDA list is strictly ascending and in range, and differs from the reference
    set only in keys of the row's ambiguity set (estimate within 1e-6 of the keep/drop boundary).
    ``amb[b * heads + h][row]`` is that set.  Returns (differing keys, reference keys)."""
    cnt_gpu, idx_gpu = cnt_gpu.cpu().numpy(), idx_gpu.cpu().numpy()
    cnt_ref, idx_ref = cnt_ref.cpu().numpy(), idx_ref.cpu().numpy()
    flips = 0
    total = 0
    for (b, h, r) in np.ndindex(cnt_ref.shape):
        mine = idx_gpu[b, h, r, : cnt_gpu[b, h, r]]
        assert np.all(np.diff(mine) > 0), "indices must be strictly ascending"
        assert mine.size == 0 or (mine[0] >= 0 and mine[-1] < sk)
        ref = set(idx_ref[b, h, r, : cnt_ref[b, h, r]].tolist())
        diff = set(mine.tolist()) ^ ref
        allowed = set(np.asarray(amb[b * heads + h][r]).tolist())
        assert diff <= allowed, f"row {(b, h, r)}: keys {sorted(diff - allowed)[:8]} differ away from the boundary"
        flips += len(diff)
        total += len(ref)
    if max_flips is None:
        max_flips = max(3, int(2e-5 * total))
    assert flips <= max_flips, f"{flips} boundary keys differ (of {total})"
    return flips, total


def membership(cnt: torch.Tensor, idx: torch.Tensor, sk: int) -> torch.Tensor:
    """(rows, n) index lists with per-row counts -> boolean (rows, sk) membership matrix, on the
    lists' device.  Entries past a row's count are ignored."""
    rows, n = idx.shape
    valid = torch.arange(n, device=idx.device).view(1, -1) < cnt.view(-1, 1)
    m = torch.zeros(rows, sk + 1, dtype=torch.bool, device=idx.device)
    safe = torch.where(valid, idx.long(), torch.full_like(idx, sk, dtype=torch.long))
    m.scatter_(1, safe, True)
    return m[:, :sk]


def boundary_band(qt_rows: torch.Tensor, k: torch.Tensor, gap: float, bk: int, group_k_block: int, lo: int,
                  rel_tol: float = 1e-6) -> torch.Tensor:
    """Which (row, key) pairs lie within ``rel_tol`` (relative to the magnitudes compared) of the
    keep/drop boundary ``s + gap == running maximum``, in fp64, on the tensors' device.
    ``qt_rows`` (n, D): scaled, re-rounded pooled queries; ``k`` (Sk, D); keys before ``lo`` are not
    walked.  Returns bool (n, Sk)."""
    n, sk = qt_rows.shape[0], k.shape[0]
    nblk = -(-sk // bk)
    ngrp = -(-nblk // group_k_block)
    s = torch.full((n, ngrp * group_k_block * bk), float("-inf"), dtype=torch.float64, device=k.device)
    s[:, :sk] = qt_rows.double() @ k.double().t()
    bmax = s.view(n, ngrp * group_k_block, bk).amax(-1)
    bmax[:, : lo // bk] = float("-inf")
    pm = torch.cummax(bmax.view(n, ngrp, group_k_block), dim=-1).values.reshape(n, -1)
    m = pm.repeat_interleave(bk, dim=1)[:, :sk]
    s = s[:, :sk]
    scale = torch.maximum(m.abs(), s.abs() + abs(gap))
    return (s + gap - m).abs() <= rel_tol * scale
