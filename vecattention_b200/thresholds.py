"""Per-head MinP thresholds for the prefill operator: the reference's file format and the switch
between the two threshold sets of classifier-free guidance.

* File format (eval/DiTEvalKit/utils/misc.py:44-62 in the reference): a JSON list with one list per
  layer, each holding one threshold per head.  ``load_threshold_matrix`` returns it as a contiguous
  fp32 tensor (layers, heads); row ``layer_idx`` is what ``VecAttention_prefill`` takes as its
  per-head ``threshold``.  The operator indexes the thresholds per (batch, head), so one row serves
  any batch size (the reference's per-head kernel reads ``gaps[b * H + h]`` from an ``(H,)`` array
  and is only valid for batch 1, spattn/src/kernels/vecattention_kernels.py:301-302).
* Classifier-free guidance (eval/DiTEvalKit/models/wan/attention.py:647-666): a diffusion step runs
  the model twice with the same timestep; the first pass uses the positive-prompt thresholds, the
  second the negative-prompt ones.  ``GuidanceThresholds.select`` reproduces that rule.
"""
from __future__ import annotations

import json
from typing import Optional, Union

import torch


def load_threshold_matrix(path: str, num_layers: int, num_heads: int,
                          device: Union[str, torch.device] = "cpu") -> torch.Tensor:
    """Read a (layers, heads) threshold file; any problem is a RuntimeError naming the file, as in
    the reference."""
    try:
        with open(path, "r") as f:
            rows = json.load(f)
        if not isinstance(rows, list):
            raise ValueError(f"Threshold matrix must be a list, got {type(rows)}")
        if len(rows) != num_layers:
            raise ValueError(f"Threshold matrix length must be {num_layers}, got {len(rows)}")
        if any(not isinstance(r, list) or len(r) != num_heads for r in rows):
            raise ValueError(f"Threshold matrix heads per layer must be {num_heads}")
        return torch.tensor(rows, dtype=torch.float32, device=device).contiguous()
    except Exception as e:  # noqa: BLE001 - the reference wraps every failure the same way
        raise RuntimeError(f"Cannot load threshold file {path}: {e}")


def save_threshold_matrix(path: str, thresholds: Union[torch.Tensor, float], num_layers: int, num_heads: int) -> None:
    """Write thresholds in the same format; a scalar is broadcast to every layer and head."""
    if isinstance(thresholds, torch.Tensor):
        mat = thresholds.detach().to("cpu", torch.float32)
        if tuple(mat.shape) != (num_layers, num_heads):
            raise ValueError(f"expected a ({num_layers}, {num_heads}) tensor, got {tuple(mat.shape)}")
        rows = mat.tolist()
    else:
        rows = [[float(thresholds)] * num_heads for _ in range(num_layers)]
    with open(path, "w") as f:
        json.dump(rows, f)


class GuidanceThresholds:
    """Which threshold set a forward pass uses under classifier-free guidance: the first pass of a
    diffusion step (a timestep not seen in the previous call) takes ``positive``, the repeat of
    the same timestep takes ``negative``.  Without guidance ``positive`` is always used.  Call
    ``select(timestep)`` once per forward pass (the reference does so in layer 0)."""

    def __init__(self, positive, negative=None, guidance: bool = True):
        self.positive = positive
        self.negative = negative if negative is not None else positive
        self.guidance = guidance
        self.previous_timestep: Optional[float] = None
        self.step = 0  # diffusion steps seen so far
        self.current = positive

    def select(self, timestep: float):
        changed = self.previous_timestep is None or self.previous_timestep != timestep
        if changed:
            self.step += 1
        if self.guidance:
            self.current = self.positive if changed else self.negative
        self.previous_timestep = timestep
        return self.current

    def for_layer(self, layer_idx: int):
        """The operator's ``threshold`` argument for one layer under the current selection."""
        cur = self.current
        return cur[layer_idx] if isinstance(cur, torch.Tensor) and cur.dim() == 2 else cur
