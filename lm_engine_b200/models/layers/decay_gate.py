"""Softplus decay gate: ``dt = softplus(x + dt_bias)``, decay ``= -exp(A_log) * dt`` (optionally exponentiated).
``A_log`` / ``dt_bias`` are fp32, excluded from weight decay, initialised from ``log U(A_min, A_max)`` and the
inverse softplus of a log-uniform time step (lm_engine/modeling_utils/softplus_decay_gate/module.py:24-131)."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
)
from .linear import ParameterizedLinear


class SoftplusDecayGate(nn.Module):
    def __init__(self, hidden_size: int | None, output_size: int, std: float | None, has_projection: bool = False,
                 A_init_min: float = 0, A_init_max: float = 16, dt_init_min: float = 1e-3, dt_init_max: float = 0.1,
                 dt_init_floor: float = 1e-4) -> None:
        super().__init__()
        self.output_size, self.has_projection = output_size, has_projection
        if has_projection:
            self.proj = ParameterizedLinear(hidden_size, output_size, std=std)
            mark_parameter_as_mup_learning_rate(self.proj.weight)
        else:
            assert hidden_size is None
        assert 0 <= A_init_min <= A_init_max and 0 < dt_init_min <= dt_init_max
        self.A_init = (A_init_min, A_init_max)
        self.dt_init = (dt_init_min, dt_init_max, dt_init_floor)
        self.A_log = nn.Parameter(torch.empty(output_size, dtype=torch.float32))
        self.dt_bias = nn.Parameter(torch.empty(output_size, dtype=torch.float32))
        mark_parameter_as_no_weight_decay(self.A_log)
        mark_parameter_as_no_weight_decay(self.dt_bias)
        self.A_log.keep_fp32 = True
        self.dt_bias.keep_fp32 = True
        self.reset_parameters()

    def get_dt(self, x: torch.Tensor, dt_min: float = 0, dt_max: float = float("inf")) -> torch.Tensor:
        if self.has_projection:
            x = self.proj(x)
        dt = F.softplus(x.float() + self.dt_bias.float())
        if (dt_min, dt_max) != (0, float("inf")):
            dt = dt.clamp(min=dt_min, max=dt_max)
        return dt

    def forward(self, x: torch.Tensor, final_exponential: bool, dt_min: float = 0, dt_max: float = float("inf"),
                output_dtype: torch.dtype = torch.float32) -> tuple[torch.Tensor, torch.Tensor]:
        dt = self.get_dt(x, dt_min, dt_max)
        y = -self.A_log.float().exp() * dt
        if final_exponential:
            y = torch.exp(y)
        return y.to(output_dtype), dt

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.A_log.is_meta:
            return
        A = torch.empty(self.output_size, dtype=torch.float32).uniform_(*self.A_init)
        self.A_log.copy_(torch.log(A))
        lo, hi, floor = self.dt_init
        dt = torch.exp(torch.rand(self.output_size) * (math.log(hi) - math.log(lo)) + math.log(lo)).clamp(min=floor)
        self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        mark_parameter_as_initialized(self.A_log)
        mark_parameter_as_initialized(self.dt_bias)
