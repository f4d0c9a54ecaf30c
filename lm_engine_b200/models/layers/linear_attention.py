"""Linear attention mixer: ``y_t = q_t . h_{t-1}``, ``h_t = h_{t-1} + k_t (x) v_t`` with head broadcasting, optional
causal conv on ``q k v``, gate and norm (lm_engine/modeling_utils/sequence_mixer_blocks/linear_attention/
module.py:29-206)."""

from __future__ import annotations

import torch.nn as nn

from ...ops.recurrence import linear_attention
from ...parallel.manager import ProcessGroupManager
from ...parameter import mark_parameter_as_mup_learning_rate
from ...utils import divide_if_divisible
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import is_glu, silu
from .conv import DepthwiseCausalConvolution
from .init_utils import std_for_linear
from .linear import ParameterizedLinear
from .norm import get_normalization_function
from .packed import PackedBatch
from .recurrent import run_per_sample


class LinearAttention(nn.Module):
    def __init__(self, hidden_size: int, config, initializer_range: float, m_width, init_method: str,
                 num_layers: int, layer_idx: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        self.use_padding_free_transformer = use_padding_free_transformer
        ProcessGroupManager.reject_context_parallel("linear attention")
        self.k_head_dim, self.v_head_dim, self.layer_idx = config.k_head_dim, config.v_head_dim, layer_idx
        self.kernel_size, self.activation_string = config.kernel_size, config.activation_function
        self.num_q_heads, self.num_k_heads = config.num_q_heads, config.num_k_heads
        self.num_v_heads, self.num_g_heads = config.num_v_heads, config.num_g_heads
        self.num_heads = max(self.num_q_heads, self.num_k_heads, self.num_v_heads)
        self.attention_multiplier = config.attention_multiplier if config.attention_multiplier is not None else 1.0
        for n in (self.num_q_heads, self.num_k_heads, self.num_v_heads, self.num_g_heads):
            divide_if_divisible(self.num_heads, n)
        self.q_shape, self.k_shape = self.num_q_heads * self.k_head_dim, self.num_k_heads * self.k_head_dim
        self.v_shape, self.g_shape = self.num_v_heads * self.v_head_dim, self.num_g_heads * self.v_head_dim
        self.conv_dim = self.q_shape + self.k_shape + self.v_shape
        std = lambda fan, depth=False: std_for_linear(initializer_range, init_method, m_width, fan, num_layers, depth)  # noqa: E731
        self.input_projection = ParameterizedLinear(hidden_size, self.conv_dim + self.g_shape, bias=config.add_bias,
                                                    std=std(hidden_size))
        if self.kernel_size is None:
            assert self.activation_string is None
        else:
            assert self.activation_string is None or not is_glu(self.activation_string)
            self.conv1d = DepthwiseCausalConvolution(self.conv_dim, self.kernel_size, self.activation_string,
                                                     config.add_bias, std(self.kernel_size))
            mark_parameter_as_mup_learning_rate(self.conv1d.weight)
        self.output_projection = ParameterizedLinear(self.g_shape, hidden_size, bias=False,
                                                     std=std(self.g_shape, use_depth_scaled_init))
        self.g_norm = get_normalization_function(config.normalization_function, self.num_heads * self.v_head_dim)
        mark_parameter_as_mup_learning_rate(self.input_projection.weight)
        mark_parameter_as_mup_learning_rate(self.output_projection.weight)

    def forward(self, x, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None):
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, x, cache_params)
        mask = layout.mask if layout is not None else info.recurrent_mask(cache_params)
        B, S = (layout.num_sequences, layout.max_seqlen) if layout is not None else x.shape[:2]
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "state")
        xc, g = self.input_projection(x).split((self.conv_dim, self.g_shape), dim=-1)
        if layout is not None:
            xc = layout.unpack(xc)
        if self.kernel_size is not None:
            xc, c = self.conv1d(xc, c, mask, output_state=cache_params is not None)
        q, k, v = xc.split((self.q_shape, self.k_shape, self.v_shape), dim=-1)
        q = q.view(B, S, self.num_q_heads, self.k_head_dim)
        k = k.view(B, S, self.num_k_heads, self.k_head_dim)
        v = v.view(B, S, self.num_v_heads, self.v_head_dim)
        y, h = run_per_sample(lambda t, st: linear_attention(t[0], t[1], t[2], st, self.attention_multiplier),
                              mask, [q, k, v], h)
        if layout is not None:
            y = layout.pack(y)
        if cache_params is not None:
            cache_params.update(self.layer_idx, "conv", c, GenerationCache.REPLACE, num_tokens_added=S)
            cache_params.update(self.layer_idx, "state", h, GenerationCache.REPLACE)
        g = g.repeat_interleave(self.num_heads // self.num_g_heads, dim=-1)
        y = y.flatten(-2, -1) * silu(g)
        return self.output_projection(self.g_norm(y))
