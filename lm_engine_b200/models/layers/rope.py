"""Rotary position embeddings: fp32 cos/sin tables (NeoX half-rotation, optional YaRN scaling).

Table construction follows lm_engine/modeling_utils/position_embedding/rope.py:15-171: ``inv_freq = base^(-2i/d)``,
angles duplicated for both halves, magnitude scale ``mscale`` folded into the tables.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...ops.rope import apply_rope_reference


class RoPE(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int = 2048, base: int = 10000) -> None:
        super().__init__()
        self.head_dim, self.max_position_embeddings, self.base = head_dim, max_position_embeddings, base
        self.mscale = 1.0
        self.reset_parameters()

    def inv_freq(self) -> torch.Tensor:
        return 1.0 / (self.base ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) * (1 / self.head_dim)))

    @torch.no_grad()
    def _build(self, seq_len: int) -> None:
        self.max_seq_len_cached = seq_len
        device = self.cos_cached.device if hasattr(self, "cos_cached") else None
        if device is not None and device.type == "meta":
            device = None
        ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), self.inv_freq())
        ang = torch.cat((ang, ang), dim=-1)
        self.register_buffer("cos_cached", (ang.cos() * self.mscale).to(device), persistent=False)
        self.register_buffer("sin_cached", (ang.sin() * self.mscale).to(device), persistent=False)

    def reset_parameters(self) -> None:
        self._build(self.max_position_embeddings)

    def tables(self, seq_len: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Full fp32 ``[>= seq_len, head_dim]`` tables (grown on demand)."""
        # a module-wide ``.to(dtype)`` also casts these buffers; the angles are needed (and read by the kernels) in fp32
        if seq_len > self.max_seq_len_cached or self.cos_cached.dtype != torch.float32:
            self._build(max(seq_len, self.max_seq_len_cached))
        return self.cos_cached, self.sin_cached

    def forward(self, seq_len: int) -> tuple[torch.Tensor, torch.Tensor]:
        cos, sin = self.tables(seq_len)
        return cos[:seq_len], sin[:seq_len]


class YaRNScaledRoPE(RoPE):
    def __init__(self, head_dim: int, max_position_embeddings: int = 2048, base: int = 10000, scale: float = 1,
                 original_max_position_embeddings: int = 2048, extrapolation_factor: float = 1,
                 attn_factor: float = 1, beta_fast: int = 32, beta_slow: int = 1) -> None:
        nn.Module.__init__(self)
        self.head_dim, self.max_position_embeddings, self.base = head_dim, max_position_embeddings, base
        self.scale = scale
        self.original_max_position_embeddings = original_max_position_embeddings
        self.extrapolation_factor, self.attn_factor = extrapolation_factor, attn_factor
        self.beta_fast, self.beta_slow = beta_fast, beta_slow
        self.mscale = (1.0 if scale <= 1 else 0.1 * math.log(scale) + 1.0) * attn_factor
        self.reset_parameters()

    def _correction_dim(self, rotations: float) -> float:
        return (self.head_dim * math.log(self.original_max_position_embeddings / (rotations * 2 * math.pi))) / (
            2 * math.log(self.base))

    def inv_freq(self) -> torch.Tensor:
        pos = self.base ** (torch.arange(0, self.head_dim, 2).float() * (1 / self.head_dim))
        extrapolation, interpolation = 1.0 / pos, 1.0 / (self.scale * pos)
        low = max(math.floor(self._correction_dim(self.beta_fast)), 0)
        high = min(math.ceil(self._correction_dim(self.beta_slow)), self.head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(self.head_dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        mask = (1 - ramp) * self.extrapolation_factor
        return interpolation * (1 - mask) + extrapolation * mask


def apply_rotary_pos_emb(x: torch.Tensor, cos_sin: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """x ``[..., heads, D]``; cos/sin ``[..., rope_dim]`` already gathered by position."""
    cos, sin = cos_sin
    return apply_rope_reference(x, cos[..., None, :], sin[..., None, :])
