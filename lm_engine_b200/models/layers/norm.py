"""Normalisation layers: RMSNorm (CUDA kernel with optional fused residual add), LayerNorm, PNorm.

All norm parameters are excluded from weight decay (lm_engine/modeling_utils/normalization.py:30-205).  Under
sequence parallelism a norm sees only its sequence shard, which needs no communication in forward; the weight
gradient is then a partial sum that the gradient reduction over the TP group completes (parameters carry
``sequence_parallel_grad = True``).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...parameter import mark_parameter_as_initialized, mark_parameter_as_no_weight_decay


class RMSNorm(nn.Module):
    def __init__(self, normalized_shape: int, eps: float | None = None, elementwise_affine: bool = True) -> None:
        super().__init__()
        self.normalized_shape = normalized_shape
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(normalized_shape)) if elementwise_affine else None
        mark_parameter_as_initialized(self.weight)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.weight is not None and not self.weight.is_meta:
            self.weight.fill_(1)
            mark_parameter_as_initialized(self.weight)

    def _eps(self, x: torch.Tensor) -> float:
        return torch.finfo(x.dtype).eps if self.eps is None else self.eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self._eps(x))[0]

    def forward_with_residual(self, x: torch.Tensor, residual: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(norm(x + residual), x + residual)`` in one pass."""
        return ops.rmsnorm(x, self.weight, self._eps(x), residual=residual)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}"


class LayerNorm(nn.LayerNorm):
    def __init__(self, normalized_shape: int, eps: float = 1e-5) -> None:
        super().__init__(normalized_shape, eps=eps)
        mark_parameter_as_initialized(self.weight)
        mark_parameter_as_initialized(self.bias)

    def reset_parameters(self) -> None:
        if not self.weight.is_meta:
            super().reset_parameters()
            mark_parameter_as_initialized(self.weight)
            mark_parameter_as_initialized(self.bias)


class PNorm(RMSNorm):
    """``weight * x / ||x||_p`` computed in fp32."""

    def __init__(self, normalized_shape: int, p: int, eps: float | None = None) -> None:
        super().__init__(normalized_shape, eps=eps)
        self.p = p

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.normalize(x.float(), p=self.p, eps=self._eps(x), dim=-1).to(x.dtype)
        return y if self.weight is None else self.weight * y

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, p={self.p}"


def get_normalization_function(name: str | None, normalized_shape: int, eps: float = 1e-5, p: int | None = None,
                               sequence_parallel: bool = False, **_unused) -> nn.Module:
    if name is None:
        return nn.Identity()
    if name == "rmsnorm":
        assert p is None
        norm = RMSNorm(normalized_shape, eps=eps)
    elif name == "layernorm":
        assert p is None
        norm = LayerNorm(normalized_shape, eps=eps)
    elif name == "p_norm":
        assert p is not None
        norm = PNorm(normalized_shape, p=p, eps=eps)
    else:
        raise ValueError(f"unexpected `normalization_function` {name}")
    for prm in norm.parameters():
        mark_parameter_as_no_weight_decay(prm)
        prm.sequence_parallel_grad = sequence_parallel
    return norm
