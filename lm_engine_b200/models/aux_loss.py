"""Accumulator of auxiliary (router) losses over the layers of one forward pass (lm_engine/loss.py:104-118)."""

from __future__ import annotations

import torch

_AUX: torch.Tensor | float = 0


def clear_aux_loss() -> None:
    global _AUX
    _AUX = 0


def add_aux_loss(value: torch.Tensor | float) -> None:
    global _AUX
    _AUX = _AUX + value


def get_aux_loss() -> torch.Tensor | float:
    return _AUX


def swap_aux_loss(value: torch.Tensor | float) -> torch.Tensor | float:
    """Replaces the accumulator and returns the previous one (a sharded unit collects its own share, which then
    leaves the unit as an explicit output so that autograd sees it on the outer graph)."""
    global _AUX
    old, _AUX = _AUX, value
    return old
