"""Mamba-2 mixer: ``in_proj -> (gate | x B C | dt)``, causal depthwise conv + activation on ``x B C``, SSD scan,
``y * silu(gate)`` -> norm -> ``out_proj``; caches the conv window and the SSM state for generation; context
parallel through a zero-initialised first pass and a prefix over the ranks' final states
(lm_engine/modeling_utils/sequence_mixer_blocks/mamba2/module.py:31-207)."""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.ssd import ssd_chunk_scan, ssd_context_parallel_initial_state, ssd_recurrent_step
from ...parallel.manager import ProcessGroupManager
from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
)
from ...utils import divide_if_divisible
from ..config import Mamba2Args
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import silu
from .conv import DepthwiseCausalConvolution, apply_mask_to_padding_states
from .decay_gate import SoftplusDecayGate
from .init_utils import std_for_linear
from .linear import ParameterizedLinear
from .norm import get_normalization_function
from .packed import PackedBatch


class Mamba2(nn.Module):
    def __init__(self, hidden_size: int, config: Mamba2Args, layer_norm_epsilon: float, initializer_range: float,
                 m_width: float | None, init_method: str, num_layers: int, layer_idx: int,
                 use_depth_scaled_init: bool = False, use_padding_free_transformer: bool = False) -> None:
        super().__init__()
        self.use_padding_free_transformer = use_padding_free_transformer
        self.num_heads, self.hidden_size = config.num_heads, hidden_size
        self.ssm_state_size, self.num_groups = config.state_size, config.num_groups
        self.intermediate_size, self.layer_idx = config.intermediate_size, layer_idx
        self.head_dim = divide_if_divisible(config.intermediate_size, config.num_heads)
        self.chunk_size, self.time_step_limit = config.chunk_size, tuple(config.time_step_limit)
        I, G, Sd = self.intermediate_size, self.num_groups, self.ssm_state_size
        self.conv_dim = I + 2 * G * Sd
        std = lambda fan, depth=False: std_for_linear(initializer_range, init_method, m_width, fan, num_layers, depth)  # noqa: E731
        self.conv1d = DepthwiseCausalConvolution(self.conv_dim, config.conv_kernel_size, config.activation_function,
                                                 config.use_conv_bias, std(config.conv_kernel_size))
        self.in_proj = ParameterizedLinear(hidden_size, I + self.conv_dim + self.num_heads, bias=config.add_bias,
                                           std=std(hidden_size))
        self.decay_gate = SoftplusDecayGate(None, self.num_heads, None, False, config.A_init_min, config.A_init_max,
                                            config.dt_init_min, config.dt_init_max, config.dt_init_floor)
        self.norm = get_normalization_function(config.normalization_function, I, eps=layer_norm_epsilon)
        self.out_proj = ParameterizedLinear(I, hidden_size, bias=config.add_bias, std=std(I, use_depth_scaled_init))
        self.D = nn.Parameter(torch.empty(self.num_heads))
        mark_parameter_as_no_weight_decay(self.D)
        for p in (self.decay_gate.A_log, self.D, self.conv1d.weight, self.in_proj.weight, self.out_proj.weight):
            mark_parameter_as_mup_learning_rate(p)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if not self.D.is_meta:
            self.D.fill_(1)
            mark_parameter_as_initialized(self.D)

    def forward(self, x: torch.Tensor, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None,
                position_info: PositionInfo | None = None) -> torch.Tensor:
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, x, cache_params)
        if layout is not None:
            mask, b, S = layout.mask, layout.num_sequences, layout.max_seqlen
        else:
            assert info.cu_seqlens is None
            mask = info.recurrent_mask(cache_params)
            x = apply_mask_to_padding_states(x, mask)
            b, S, _ = x.shape
        I, G, Sd, N, P = self.intermediate_size, self.num_groups, self.ssm_state_size, self.num_heads, self.head_dim
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "ssm")
        gate, xBC, dt = self.in_proj(x).split((I, self.conv_dim, N), dim=-1)
        if layout is not None:
            xBC, dt = layout.unpack(xBC), layout.unpack(dt)
        xBC, c = self.conv1d(xBC, c, mask, output_state=cache_params is not None)
        A = -torch.exp(self.decay_gate.A_log.float())
        dt = self.decay_gate.get_dt(dt, *self.time_step_limit)
        xs, B, C = xBC.split((I, G * Sd, G * Sd), dim=-1)
        xs = xs.reshape(b, S, N, P)
        B, C = B.reshape(b, S, G, Sd), C.reshape(b, S, G, Sd)
        if S == 1 and h is not None:
            y, h = ssd_recurrent_step(xs[:, 0], dt[:, 0], A, B[:, 0], C[:, 0], self.D, h)
            y = y[:, None]
        else:
            cp = ProcessGroupManager.get_context_parallel_group()
            if cp is not None:
                # Context parallel: ONE scan per rank.  The recurrence is linear in the state, so the shard is
                # scanned from a zero state (all ranks at once), the boundary states are exchanged and combined
                # (ssd_context_parallel_initial_state), and what the entering state h0 adds to every position is a
                # closed form: y_t += exp(sum_{tau <= t} A dt_tau) C_t . h0, and the state leaving the shard is
                # exp(sum A dt) h0 + (final state from zero).
                assert h is None
                y, f0 = ssd_chunk_scan(xs, dt, A, B, C, self.D, self.chunk_size)
                log_decay = (A[None, None, :] * dt.float()).cumsum(1)                       # [b, S, N]
                total = torch.exp(log_decay[:, -1])                                         # [b, N]
                h0 = ssd_context_parallel_initial_state(f0, total, cp)                      # [b, N, P, Sd]
                hg = h0.float().reshape(b, G, N // G, P, Sd)
                add = torch.einsum("bsgd,bgjpd->bsgjp", C.float(), hg).reshape(b, S, N, P)
                y = (y.float() + torch.exp(log_decay)[..., None] * add).to(y.dtype)
                h = total[..., None, None] * h0 + f0
            else:
                y, h = ssd_chunk_scan(xs, dt, A, B, C, self.D, self.chunk_size, initial_state=h)
        if cache_params is not None:
            cache_params.update(self.layer_idx, "conv", c, GenerationCache.REPLACE, num_tokens_added=S)
            cache_params.update(self.layer_idx, "ssm", h, GenerationCache.REPLACE)
        y = y.reshape(b, S, I)
        if layout is not None:
            y = layout.pack(y)
        y = y * silu(gate)
        return self.out_proj(self.norm(y))
