"""Caller-side configuration of the prefill attention, with the reference's names: the
``FastPrefillConfig`` object model adapters hand to the dispatcher and the ``--fastprefill-*``
command-line flags that fill it (spattn/src/models/config_args.py:6-129).

Only the fields the VecAttention path reads change anything here; the fields of the reference's
other attention methods (``stride``, ``gamma``, ``tau``, ``theta``, ``step``) are carried so that a
configuration written for the reference loads unchanged.
"""
from __future__ import annotations

import argparse
import os
from typing import Any, Dict, Optional

# field -> default of the constructor (config_args.py:24-52); ``threshold`` is only set when given
_FIELDS: Dict[str, Any] = {
    "metric": "xattn",
    "block_size_q": 64, "block_size_k": 16, "group_k_block": 1, "chunk_size": 8 * 1024,
    "vision_start_position": None, "vision_end_position": None,
    "stride": 16, "gamma": 0.9, "tau": 0.1, "theta": 12, "step": 16,
    "output_time": True, "dump_qk_dir": None, "input_id": "input",
}
# flag (without the --fastprefill- prefix) -> (type, default) of the command line (config_args.py:77-97);
# the command line's defaults differ from the constructor's, as in the reference
_FLAGS = {
    "metric": (str, "full"), "threshold": (float, 0.9), "block-size-q": (int, 64), "block-size-k": (int, 16),
    "group-k-block": (int, 1), "chunk-size": (int, 64 * 1024), "stride": (int, 16), "gamma": (float, 0.9),
    "tau": (float, 0.1), "theta": (float, 12), "step": (int, 16), "dump-qk-dir": (str, None), "input-id": (str, None),
}


class FastPrefillConfig(dict):
    """Attribute-style settings of the prefill dispatcher.  ``metric`` picks the attention method
    ("vecattention" and "full" are served by this package); ``threshold`` is the MinP threshold, a
    float or a tensor indexed by layer (then optionally by head); ``block_size_q`` / ``block_size_k``
    / ``group_k_block`` / ``chunk_size`` are the operator's q_pooling_size / k_local_size /
    group_k_block / chunk_size; the two vision positions bound the span that gets VecAttention."""

    def __init__(self, metric: str = _FIELDS["metric"], threshold=None, **kwargs):
        super().__init__()
        unknown = set(kwargs) - set(_FIELDS)
        if unknown:
            raise TypeError(f"unknown FastPrefillConfig field(s): {sorted(unknown)}")
        self.metric = metric
        for name, default in _FIELDS.items():
            if name != "metric":
                setattr(self, name, kwargs.get(name, default))
        if threshold is not None:  # optional: not every method needs one
            self.threshold = threshold

    # a dict whose entries read and write as attributes
    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        self[name] = value


def add_fastprefill_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """Add the ``--fastprefill-*`` flags to ``parser``."""
    for flag, (typ, default) in _FLAGS.items():
        parser.add_argument(f"--fastprefill-{flag}", type=typ, default=default)
    return parser


def get_fastprefill_config(args: argparse.Namespace) -> FastPrefillConfig:
    """The configuration the parsed ``--fastprefill-*`` flags describe (flags left at ``None`` keep the
    constructor's default)."""
    picked = {k[len("fastprefill_"):]: v for k, v in vars(args).items() if k.startswith("fastprefill_") and v is not None}
    return FastPrefillConfig(**picked)


def build_output_file_from_config(base_path: str, config: FastPrefillConfig) -> str:
    """``base_path`` with the method and its main settings inserted before the extension."""
    tags = {"vecattention": [("th", "threshold"), ("qps", "block_size_q"), ("kls", "block_size_k"), ("gkb", "group_k_block")],
            "xattn": [("th", "threshold"), ("stride", "stride")],
            "flex": [("th", "gamma"), ("tau", "tau")],
            "anchor": [("bsq", "block_size_q"), ("step", "step"), ("th", "theta")]}
    parts = [f"metric={config.metric}"] + [f"{tag}={getattr(config, field)}" for tag, field in tags.get(config.metric, [])]
    stem, ext = os.path.splitext(base_path)
    return f"{stem}_{'_'.join(parts)}{ext}"
