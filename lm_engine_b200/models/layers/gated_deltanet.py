"""Gated DeltaNet mixer: ``qkv_proj`` / ``ab_proj``, short causal conv (silu) on q k v, ``beta = sigmoid(b)`` (x 2
when negative eigenvalues are allowed), log-decay ``g = -exp(A_log) softplus(a + dt_bias)``, GQA-style repetition of
q / k heads up to the v heads, gated delta rule with l2-normalised q / k, optional output gate, per-head RMSNorm,
``o_proj`` (lm_engine/modeling_utils/sequence_mixer_blocks/gated_deltanet/module.py:28-246).  The reference has no
PyTorch path for the recurrence (it calls fla's Triton kernels); ``ops.recurrence.gated_delta_rule`` is this engine's
statement of it: the token recurrence for decode, the chunk-parallel (triangular-solve) form otherwise."""

from __future__ import annotations

import torch.nn as nn

from ...ops.recurrence import gated_delta_rule
from ...parallel.manager import ProcessGroupManager
from ...utils import divide_if_divisible
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import silu
from .conv import DepthwiseCausalConvolution
from .decay_gate import SoftplusDecayGate
from .init_utils import std_for_linear
from .linear import ParameterizedLinear
from .norm import get_normalization_function
from .packed import PackedBatch
from .recurrent import run_per_sample


class GatedDeltaNet(nn.Module):
    def __init__(self, hidden_size: int, config, layer_idx: int, init_method: str, initializer_range: float,
                 m_width, num_layers: int, use_depth_scaled_init: bool, use_padding_free_transformer: bool = False,
                 layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        ProcessGroupManager.reject_context_parallel("gated delta net")
        self.use_padding_free_transformer = use_padding_free_transformer
        self.allow_neg_eigval, self.use_gate, self.layer_idx = config.allow_neg_eigval, config.use_gate, layer_idx
        self.num_k_heads, self.num_v_heads = config.num_k_heads, config.num_v_heads
        self.k_head_dim, self.v_head_dim = config.k_head_dim, config.v_head_dim
        self.key_dim, self.value_dim = self.num_k_heads * self.k_head_dim, self.num_v_heads * self.v_head_dim
        self.attention_multiplier = config.attention_multiplier
        divide_if_divisible(self.num_v_heads, self.num_k_heads)
        std = lambda fan, depth=False: std_for_linear(initializer_range, init_method, m_width, fan, num_layers, depth)  # noqa: E731
        self.qkv_proj = ParameterizedLinear(hidden_size, 2 * self.key_dim + self.value_dim, bias=False,
                                            std=std(hidden_size))
        self.ab_proj = ParameterizedLinear(hidden_size, 2 * self.num_v_heads + (self.value_dim if self.use_gate else 0),
                                           bias=False, std=std(hidden_size))
        self.decay_gate = SoftplusDecayGate(None, self.num_v_heads, None, False, config.A_init_min, config.A_init_max,
                                            config.dt_init_min, config.dt_init_max, config.dt_init_floor)
        self.qkv_conv1d = DepthwiseCausalConvolution(2 * self.key_dim + self.value_dim, config.kernel_size, "silu",
                                                     False, std(config.kernel_size))
        self.o_norm = get_normalization_function("rmsnorm", self.v_head_dim, eps=layer_norm_epsilon)
        self.o_proj = ParameterizedLinear(self.value_dim, hidden_size, bias=False,
                                          std=std(self.value_dim, use_depth_scaled_init))

    def forward(self, hidden_states, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None):
        info, _ = resolve_attention_and_position_info(attention_mask_info, position_info)
        layout = PackedBatch.of(self.use_padding_free_transformer, info, hidden_states, cache_params)
        mask = layout.mask if layout is not None else info.recurrent_mask(cache_params)
        B, S = (layout.num_sequences, layout.max_seqlen) if layout is not None else hidden_states.shape[:2]
        c = h = None
        if cache_params is not None:
            c, h = cache_params.get(self.layer_idx, "conv"), cache_params.get(self.layer_idx, "state")
        qkv = self.qkv_proj(hidden_states)
        ab = self.ab_proj(hidden_states)
        if self.use_gate:
            a, b, gate = ab.split((self.num_v_heads, self.num_v_heads, self.value_dim), dim=-1)
        else:
            a, b = ab.chunk(2, dim=-1)
        if layout is not None:
            qkv, a, b = layout.unpack(qkv), layout.unpack(a), layout.unpack(b)
        qkv, c = self.qkv_conv1d(qkv, c, mask, output_state=cache_params is not None)
        q, k, v = qkv.split((self.key_dim, self.key_dim, self.value_dim), dim=-1)
        q = q.view(B, S, -1, self.k_head_dim)
        k = k.view(B, S, -1, self.k_head_dim)
        v = v.view(B, S, -1, self.v_head_dim)
        if self.num_v_heads > self.num_k_heads:
            rep = self.num_v_heads // self.num_k_heads
            q, k = q.repeat_interleave(rep, dim=-2), k.repeat_interleave(rep, dim=-2)
        beta = b.sigmoid()
        if self.allow_neg_eigval:
            beta = beta * 2
        g, _ = self.decay_gate(a, final_exponential=False)
        o, h = run_per_sample(
            lambda t, st: gated_delta_rule(t[0], t[1], t[2], t[3], t[4], self.attention_multiplier, st, True),
            mask, [q, k, v, g, beta], h)
        if layout is not None:
            o = layout.pack(o)
        if cache_params is not None:
            cache_params.update(self.layer_idx, "conv", c, GenerationCache.REPLACE, num_tokens_added=S)
            cache_params.update(self.layer_idx, "state", h, GenerationCache.REPLACE)
        if self.use_gate:
            o = o * silu(gate.view(*o.shape[:-2], -1, self.v_head_dim))
        o = self.o_norm(o)
        return self.o_proj(o.flatten(-2, -1))
