"""M2RNN mixer: matrix-valued state per head, ``h = f h + (1 - f) tanh(h W + k (x) v)``, ``y = q . h``, forget gate
from a softplus decay gate, identity-initialised ``state_weight``, optional residual ``D``, context parallel as a
pipeline along the sequence (lm_engine/modeling_utils/sequence_mixer_blocks/m2rnn/module.py:42-331)."""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.recurrence import m2rnn
from ...parallel.manager import ProcessGroupManager
from ...parallel.sequence_pipeline import sequence_pipeline
from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
)
from ...utils import divide_if_divisible
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import is_glu, silu
from .conv import DepthwiseCausalConvolution
from .decay_gate import SoftplusDecayGate
from .init_utils import std_for_linear
from .linear import ParameterizedLinear
from .norm import get_normalization_function
from .packed import PackedBatch
from .recurrent import run_per_sample


class M2RNN(nn.Module):
    def __init__(self, hidden_size: int, config, initializer_range: float, m_width, init_method: str,
                 num_layers: int, layer_idx: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        self.use_padding_free_transformer = use_padding_free_transformer
        self.k_head_dim, self.v_head_dim, self.layer_idx = config.k_head_dim, config.v_head_dim, layer_idx
        self.kernel_size, self.activation_string = config.kernel_size, config.activation_function
        self.gradient_clipping, self.use_residual = config.gradient_clipping, config.use_residual
        self.num_q_heads, self.num_k_heads, self.num_v_heads = config.num_q_heads, config.num_k_heads, config.num_v_heads
        self.num_f_heads, self.num_g_heads, self.num_weight_heads = (config.num_f_heads, config.num_g_heads,
                                                                     config.num_weight_heads)
        self.num_heads = max(self.num_q_heads, self.num_k_heads, self.num_v_heads, self.num_f_heads,
                             self.num_weight_heads)
        for n in (self.num_q_heads, self.num_k_heads, self.num_v_heads, self.num_f_heads, self.num_weight_heads,
                  self.num_g_heads):
            divide_if_divisible(self.num_heads, n)
        self.q_shape, self.k_shape = self.num_q_heads * self.k_head_dim, self.num_k_heads * self.k_head_dim
        self.v_shape, self.g_shape = self.num_v_heads * self.v_head_dim, self.num_g_heads * self.v_head_dim
        self.conv_dim = self.q_shape + self.k_shape + self.v_shape
        std = lambda fan, depth=False: std_for_linear(initializer_range, init_method, m_width, fan, num_layers, depth)  # noqa: E731
        self.input_projection = ParameterizedLinear(hidden_size, self.conv_dim + self.num_f_heads + self.g_shape,
                                                    bias=config.add_bias, std=std(hidden_size))
        self.decay_gate = SoftplusDecayGate(None, self.num_heads, None, False, config.A_init_min, config.A_init_max,
                                            config.dt_init_min, config.dt_init_max, config.dt_init_floor)
        if self.kernel_size is None:
            assert self.activation_string is None
        else:
            assert self.activation_string is None or not is_glu(self.activation_string)
            self.conv1d = DepthwiseCausalConvolution(self.conv_dim, self.kernel_size, self.activation_string,
                                                     config.add_bias, std(self.kernel_size))
            mark_parameter_as_mup_learning_rate(self.conv1d.weight)
        if self.use_residual:
            self.D = nn.Parameter(torch.empty(self.num_heads, self.v_head_dim))
            mark_parameter_as_no_weight_decay(self.D)
        self.state_weight = nn.Parameter(torch.empty(self.num_weight_heads, self.v_head_dim, self.v_head_dim))
        self.output_projection = ParameterizedLinear(self.g_shape, hidden_size, bias=False,
                                                     std=std(self.g_shape, use_depth_scaled_init))
        self.g_norm = get_normalization_function(config.normalization_function, self.num_heads * self.v_head_dim)
        for p in (self.input_projection.weight, self.state_weight, self.output_projection.weight):
            mark_parameter_as_mup_learning_rate(p)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.state_weight.is_meta:
            return
        self.state_weight.copy_(torch.eye(self.v_head_dim)[None].expand(self.num_weight_heads, -1, -1))
        mark_parameter_as_initialized(self.state_weight)
        if self.use_residual:
            self.D.fill_(1)
            mark_parameter_as_initialized(self.D)

    def forward(self, x, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None):
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, x, cache_params)
        mask = layout.mask if layout is not None else info.recurrent_mask(cache_params)
        B, S = (layout.num_sequences, layout.max_seqlen) if layout is not None else x.shape[:2]
        cp = ProcessGroupManager.is_context_parallel_enabled()
        if cp:
            assert cache_params is None and mask is None
            assert ProcessGroupManager.get_context_parallel_load_balancing_method() is None
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "state")
        xc, f, g = self.input_projection(x).split((self.conv_dim, self.num_f_heads, self.g_shape), dim=-1)
        f, _ = self.decay_gate(f, final_exponential=True, output_dtype=f.dtype)
        if layout is not None:
            xc, f = layout.unpack(xc), layout.unpack(f)
        if self.kernel_size is not None:
            xc, c = self.conv1d(xc, c, mask, output_state=cache_params is not None)
        q, k, v = xc.split((self.q_shape, self.k_shape, self.v_shape), dim=-1)
        q = q.view(B, S, self.num_q_heads, self.k_head_dim)
        k = k.view(B, S, self.num_k_heads, self.k_head_dim)
        v = v.view(B, S, self.num_v_heads, self.v_head_dim)

        def scan(t, st):
            return m2rnn(t[0], t[1], t[2], t[3], self.state_weight, st, self.gradient_clipping)

        if cp:
            y, h = sequence_pipeline(lambda q_, k_, v_, f_, W_, h0: m2rnn(q_, k_, v_, f_, W_, h0,
                                                                                 self.gradient_clipping),
                                     (q, k, v, f, self.state_weight),
                                     (B, self.num_heads, self.k_head_dim, self.v_head_dim))
        else:
            y, h = run_per_sample(scan, mask, [q, k, v, f], h)
        if self.use_residual:
            y = y + v.repeat_interleave(self.num_heads // self.num_v_heads, dim=2) * self.D
        if layout is not None:
            y = layout.pack(y)
        if cache_params is not None:
            cache_params.update(self.layer_idx, "conv", c, GenerationCache.REPLACE, num_tokens_added=S)
            cache_params.update(self.layer_idx, "state", h, GenerationCache.REPLACE)
        g = g.repeat_interleave(self.num_heads // self.num_g_heads, dim=-1)
        y = y.flatten(-2, -1) * silu(g)
        return self.output_projection(self.g_norm(y))
