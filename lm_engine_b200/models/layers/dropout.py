"""Dropout that is a no-op module for p = 0 (lm_engine/modeling_utils/dropout.py:15-36)."""

from __future__ import annotations

import torch
import torch.nn as nn


class Dropout(nn.Dropout):
    def __init__(self, p: float = 0.0, **_unused) -> None:
        super().__init__(p)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.p == 0 or not self.training:
            return x
        return super().forward(x)
