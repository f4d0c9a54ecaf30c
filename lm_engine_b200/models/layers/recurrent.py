"""RNN and GRU mixers: multi-head recurrences with per-head ``state_weight`` blocks, optional causal conv on the
input branch, ``y * silu(gate)`` -> norm -> output projection
(lm_engine/modeling_utils/sequence_mixer_blocks/rnn/module.py:35-229, gru/module.py:34-365)."""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.recurrence import gru, rnn
from ...parallel.manager import ProcessGroupManager
from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
)
from ...utils import divide_if_divisible
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import get_activation_function, is_glu, silu
from .conv import DepthwiseCausalConvolution
from .init_utils import std_for_linear
from .linear import ParameterizedLinear
from .norm import get_normalization_function
from .packed import PackedBatch


def run_per_sample(fn, mask: torch.Tensor | None, tensors: list[torch.Tensor], state):
    """``fn(tensors, state) -> (y, state)`` on a left-padded batch so that every sample sees only its own tokens
    (what pack -> kernel -> unpack does in the reference); identity wrapper when there is no padding.  Only a padded
    batch that also carries a state is run sample by sample."""
    if mask is None:
        return fn(tensors, state)
    if state is None:
        # zero inputs and a zero state keep every recurrence here at zero through the padding in front of a sample,
        # so the whole batch runs as one scan
        keep = [mask.view(*mask.shape, *([1] * (t.dim() - 2))).to(t.dtype) for t in tensors]
        return fn([t * m for t, m in zip(tensors, keep)], None)
    B, S = mask.shape
    ys, hs = [], []
    for b in range(B):
        n = int(mask[b].sum())
        y, h = fn([t[b:b + 1, S - n:] for t in tensors], None if state is None else state[b:b + 1])
        pad = y.new_zeros((1, S - n, *y.shape[2:]))
        ys.append(torch.cat((pad, y), dim=1))
        hs.append(h)
    return torch.cat(ys, 0), torch.cat(hs, 0)


class _RecurrentBase(nn.Module):
    def _common(self, hidden_size, config, init_method, initializer_range, m_width, num_layers, layer_idx,
                use_depth_scaled_init, use_padding_free_transformer, in_width: int) -> None:
        self.use_padding_free_transformer = use_padding_free_transformer
        self.layer_idx = layer_idx
        ProcessGroupManager.reject_context_parallel("RNN / GRU")
        self.gradient_clipping = config.gradient_clipping
        self.state_head_dim = config.state_head_dim
        self.state_size = self.num_heads * self.state_head_dim
        self.kernel_size, self.activation_string = config.kernel_size, config.activation_function
        std = lambda fan, depth=False: std_for_linear(initializer_range, init_method, m_width, fan, num_layers, depth)  # noqa: E731
        self.state_weight_std = std(self.state_head_dim)
        self.input_projection = ParameterizedLinear(hidden_size, in_width, bias=config.add_bias, std=std(hidden_size))
        if self.kernel_size is not None:
            assert not is_glu(self.activation_string)
            self.conv1d = DepthwiseCausalConvolution(self.state_size, self.kernel_size, self.activation_string,
                                                     config.add_bias, std(self.kernel_size))
            mark_parameter_as_mup_learning_rate(self.conv1d.weight)
        self.activation_function = (nn.Identity() if self.activation_string is None
                                    else get_activation_function(self.activation_string))
        self.output_projection = ParameterizedLinear(self.state_size, hidden_size, bias=False,
                                                     std=std(self.state_size, use_depth_scaled_init))
        self.norm = get_normalization_function(config.normalization_function, self.state_size)

    def _finish_init(self) -> None:
        mark_parameter_as_mup_learning_rate(self.input_projection.weight)
        mark_parameter_as_mup_learning_rate(self.state_weight)
        mark_parameter_as_mup_learning_rate(self.output_projection.weight)
        mark_parameter_as_no_weight_decay(self.state_weight)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if not self.state_weight.is_meta:
            nn.init.normal_(self.state_weight, std=self.state_weight_std)
            mark_parameter_as_initialized(self.state_weight)

    def _input_branch(self, x, c, mask, use_cache):
        if self.kernel_size is None:
            return self.activation_function(x), c
        return self.conv1d(x, c, mask, output_state=use_cache)

    def _finish(self, y, g, c, h, S, cache_params):
        if cache_params is not None:
            cache_params.update(self.layer_idx, "conv", c, GenerationCache.REPLACE, num_tokens_added=S)
            cache_params.update(self.layer_idx, "state", h, GenerationCache.REPLACE)
        y = y.flatten(-2, -1) * silu(g)
        return self.output_projection(self.norm(y))

    def extra_repr(self) -> str:
        return f"gradient_clipping = {self.gradient_clipping}\nweight_shape: {tuple(self.state_weight.shape)}"


class RNN(_RecurrentBase):
    def __init__(self, hidden_size: int, config, initializer_range: float, m_width, init_method: str,
                 num_layers: int, layer_idx: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        self.num_input_heads, self.num_weight_heads = config.num_input_heads, config.num_weight_heads
        self.num_heads = max(self.num_input_heads, self.num_weight_heads)
        divide_if_divisible(self.num_heads, self.num_input_heads)
        divide_if_divisible(self.num_heads, self.num_weight_heads)
        d = config.state_head_dim
        self.x_shape, self.g_shape = self.num_input_heads * d, self.num_heads * d
        self._common(hidden_size, config, init_method, initializer_range, m_width, num_layers, layer_idx,
                     use_depth_scaled_init, use_padding_free_transformer, self.x_shape + self.g_shape)
        self.state_weight = nn.Parameter(torch.empty(self.num_heads, d, d))
        self._finish_init()

    def forward(self, x, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None):
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, x, cache_params)
        mask = layout.mask if layout is not None else info.recurrent_mask(cache_params)
        S = x.size(-2)
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "state")
        xi, g = self.input_projection(x).split((self.x_shape, self.g_shape), dim=-1)
        if layout is not None:
            xi = layout.unpack(xi)
        xi, c = self._input_branch(xi, c, mask, cache_params is not None)
        xi = xi.view(*xi.shape[:-1], -1, self.state_head_dim)
        y, h = run_per_sample(lambda t, st: rnn(t[0], self.state_weight, st, self.gradient_clipping), mask,
                              [xi], h)
        if layout is not None:
            y = layout.pack(y)
        return self._finish(y, g, c, h, S, cache_params)


class GRU(_RecurrentBase):
    def __init__(self, hidden_size: int, config, initializer_range: float, m_width, init_method: str,
                 num_layers: int, layer_idx: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        self.heads = (config.num_input_heads, config.num_forget_input_heads, config.num_reset_input_heads)
        self.weight_heads = (config.num_weight_heads, config.num_forget_weight_heads, config.num_reset_weight_heads)
        self.num_heads = max(*self.heads, *self.weight_heads)
        for n in (*self.heads, *self.weight_heads):
            divide_if_divisible(self.num_heads, n)
        d = config.state_head_dim
        self.splits = tuple(n * d for n in self.heads) + (self.num_heads * d,)
        self._common(hidden_size, config, init_method, initializer_range, m_width, num_layers, layer_idx,
                     use_depth_scaled_init, use_padding_free_transformer, sum(self.splits))
        self.state_weight = nn.Parameter(torch.empty(sum(self.weight_heads), d, d))
        self._finish_init()

    def forward(self, x, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None):
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, x, cache_params)
        mask = layout.mask if layout is not None else info.recurrent_mask(cache_params)
        S = x.size(-2)
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "state")
        xi, xf, xr, g = self.input_projection(x).split(self.splits, dim=-1)
        if layout is not None:
            xi, xf, xr = layout.unpack(xi), layout.unpack(xf), layout.unpack(xr)
        xi, c = self._input_branch(xi, c, mask, cache_params is not None)
        d = self.state_head_dim
        xi, xf, xr = (t.view(*t.shape[:-1], -1, d) for t in (xi, xf, xr))
        W, Wf, Wr = self.state_weight.split(self.weight_heads, dim=0)
        y, h = run_per_sample(lambda t, st: gru(t[0], t[1], t[2], W, Wf, Wr, st, self.gradient_clipping), mask,
                              [xi, xf, xr], h)
        if layout is not None:
            y = layout.pack(y)
        return self._finish(y, g, c, h, S, cache_params)
