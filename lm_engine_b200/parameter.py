"""Parameter markers: no-weight-decay, muP learning rate, initialised, and tensor-parallel shard metadata.

Markers are plain attributes on ``nn.Parameter`` (reference: lm_engine/parameter.py:8-83).  ``tp_shard_dim`` records
along which dimension a parameter is split across the tensor-parallel group (None = replicated) so checkpointing
can present it as a standard sharded DTensor.
"""

from __future__ import annotations

import torch
import torch.nn as nn

_MARKERS = ("_no_weight_decay", "_has_mup_learning_rate", "_is_initialized", "tp_shard_dim", "tp_global_shape",
            "ep_shard_dim")


def mark_parameter_as_no_weight_decay(p: nn.Parameter | None) -> nn.Parameter | None:
    if p is not None:
        p._no_weight_decay = True
    return p


def mark_parameter_as_mup_learning_rate(p: nn.Parameter | None) -> nn.Parameter | None:
    if p is not None:
        p._has_mup_learning_rate = True
    return p


def mark_parameter_as_initialized(p: torch.Tensor | None) -> torch.Tensor | None:
    if p is not None:
        p._is_initialized = True
    return p


def is_parameter_with_no_weight_decay(p: nn.Parameter | None) -> bool:
    return getattr(p, "_no_weight_decay", False)


def is_parameter_with_mup_learning_rate(p: nn.Parameter | None) -> bool:
    return getattr(p, "_has_mup_learning_rate", False)


def is_parameter_initialized(p: nn.Parameter | None) -> bool:
    return getattr(p, "_is_initialized", False)


def mark_tp_shard(p: nn.Parameter, dim: int | None, global_shape: tuple[int, ...] | None = None) -> nn.Parameter:
    p.tp_shard_dim = dim
    p.tp_global_shape = tuple(global_shape) if global_shape is not None else None
    return p


def get_parameter_marker_maps(modules: list[nn.Module]) -> list[dict[str, dict]]:
    """Snapshot of all markers by parameter name, taken before parameters are re-created (flat-buffer views)."""
    out = []
    for m in modules:
        out.append({n: {k: getattr(p, k) for k in _MARKERS if hasattr(p, k)} for n, p in m.named_parameters()})
    return out


def set_parameter_marker_maps(modules: list[nn.Module], maps: list[dict[str, dict]]) -> None:
    for m, mp in zip(modules, maps):
        for n, p in m.named_parameters():
            for k, v in mp.get(n, {}).items():
                setattr(p, k, v)
