"""``gpt_crosslayer``: layers share key/value projections.  ``sharing_pattern[i]`` names the layer whose K/V layer
``i`` attends over; a layer that names itself owns a ``kv_proj`` (its own norm + a fused K|V projection per KV
head), the others reuse the K/V computed by their parent
(lm_engine/models/gpt_crosslayer/{config,layer,base}.py, sequence_mixers/base.py)."""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..utils import divide_if_divisible
from .base import CausalLM, TransformerModel
from .blocks import get_mlp_block
from .config import CommonConfig
from .layers.dropout import Dropout
from .layers.linear import ParameterizedLinear
from .layers.norm import get_normalization_function
from .layers.rope import apply_rotary_pos_emb


def resolve_sharing_pattern(config: CommonConfig) -> list[int]:
    sp = config.sharing_pattern
    if sp is None:
        return list(range(config.num_layers))
    assert all(sp[i] == i for i in set(sp)), "a filled sharing pattern doesn't have a parent layer"
    assert all(sp[i] <= sp[i + 1] for i in range(len(sp) - 1))
    assert all(0 <= i < config.num_layers for i in sp)
    assert config.init_method == "normal"
    return list(sp)


class KeyValueProjection(nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int, add_bias: bool,
                 initializer_range: float, normalization_function: str, layer_norm_epsilon: float) -> None:
        super().__init__()
        self.num_key_value_heads = num_key_value_heads
        self.head_dim = divide_if_divisible(hidden_size, num_attention_heads)
        self.ln = get_normalization_function(normalization_function, hidden_size, eps=layer_norm_epsilon)
        self.kv_attn = ParameterizedLinear(hidden_size, 2 * num_key_value_heads * self.head_dim, bias=add_bias,
                                           std=initializer_range)

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        kv = self.kv_attn(self.ln(x))
        kv = kv.view(*kv.shape[:-1], self.num_key_value_heads, 2 * self.head_dim)
        k, v = kv.chunk(2, dim=-1)
        return k, v                                     # [..., Hkv, D]


class CrossLayerAttention(nn.Module):
    def __init__(self, config: CommonConfig, layer_idx: int, use_padding_free_transformer: bool) -> None:
        super().__init__()
        blk = config.sequence_mixer_blocks[layer_idx]
        assert blk.sequence_mixer_type == "softmax_attention"
        H = config.hidden_size
        self.num_heads, self.num_key_value_heads = blk.num_attention_heads, blk.num_key_value_heads
        self.head_dim = divide_if_divisible(H, self.num_heads)
        self.position_embedding_type = config.position_embedding_type
        self.use_padding_free_transformer = use_padding_free_transformer
        self.attention_multiplier = (blk.attention_multiplier if blk.attention_multiplier is not None
                                     else 1 / math.sqrt(self.head_dim))
        self.softmax_dropout_p = blk.softmax_dropout
        self.q_attn = ParameterizedLinear(H, H, bias=blk.add_bias, std=config.initializer_range)
        self.c_proj = ParameterizedLinear(H, H, bias=blk.add_bias,
                                          std=config.initializer_range / math.sqrt(2 * config.num_layers))
        self.dropout = Dropout(blk.dropout)

    def forward(self, x, key, value, attention_mask_info, position_info):
        q = self.q_attn(x)
        q = q.view(*q.shape[:-1], self.num_heads, self.head_dim)
        if self.position_embedding_type == "rope":
            q = apply_rotary_pos_emb(q, position_info.rope_cos_sin)
        drop = self.softmax_dropout_p if self.training else 0.0
        if self.use_padding_free_transformer:
            o = ops.attention(q, key, value, causal=True, softmax_scale=self.attention_multiplier,
                              cu_seqlens=attention_mask_info.cu_seqlens, max_seqlen=attention_mask_info.max_seqlen,
                              dropout_p=drop)
        else:
            o = ops.attention(q, key, value, causal=True, softmax_scale=self.attention_multiplier,
                              attention_mask=attention_mask_info.attention_mask, dropout_p=drop)
        return self.dropout(self.c_proj(o.flatten(-2, -1)))


class GPTCrossLayerBlock(nn.Module):
    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int,
                 sequence_parallel: bool = False) -> None:
        super().__init__()
        H = config.hidden_size
        self.m_residual, self.layer_idx = config.m_residual, layer_idx
        self.position_embedding_type = config.position_embedding_type
        blk = config.sequence_mixer_blocks[layer_idx]
        self.kv_proj = None
        if resolve_sharing_pattern(config)[layer_idx] == layer_idx:
            self.kv_proj = KeyValueProjection(H, blk.num_attention_heads, blk.num_key_value_heads, blk.add_bias,
                                              config.initializer_range, config.normalization_function,
                                              config.layer_norm_epsilon)
        self.ln_1 = get_normalization_function(config.normalization_function, H, eps=config.layer_norm_epsilon)
        self.sequence_mixer = CrossLayerAttention(config, layer_idx, use_padding_free_transformer)
        self.ln_2 = get_normalization_function(config.normalization_function, H, eps=config.layer_norm_epsilon)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer, False, layer_idx)

    def forward(self, state, cache_params=None, attention_mask_info=None, position_info=None):
        x, key, value = state
        if self.kv_proj is not None:
            key, value = self.kv_proj(x)
            if self.position_embedding_type == "rope":
                key = apply_rotary_pos_emb(key, position_info.rope_cos_sin)
            if cache_params is not None:
                key = cache_params.update(self.layer_idx, "key", key)
                value = cache_params.update(self.layer_idx, "value", value)
        y = self.sequence_mixer(self.ln_1(x), key, value, attention_mask_info, position_info)
        x = x + (y if self.m_residual is None else y * self.m_residual)
        y = self.mlp_block(self.ln_2(x))
        x = x + (y if self.m_residual is None else y * self.m_residual)
        return x, key, value


class GPTCrossLayerModel(TransformerModel):
    layer_class = GPTCrossLayerBlock

    def run_blocks(self, x, cache_params, attention_mask_info, position_info):
        state = (x, None, None)
        for i in range(self.layer_start_id, self.layer_end_id):
            state = self.h[str(i)](state, cache_params=cache_params, attention_mask_info=attention_mask_info,
                                   position_info=position_info)
        return state[0]


class GPTCrossLayerForCausalLM(CausalLM):
    base_model_class = GPTCrossLayerModel
    model_type = "gpt_crosslayer"
