"""Softmax attention mixer with a fused, per-KV-group interleaved QKV projection.

``c_attn`` rows are grouped per KV head as ``[q_0 .. q_{G-1} | k | v]`` (``+ gate`` of ``G*D`` rows when
``attention_gate``) - the checkpoint-visible layout of the reference
(lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/module.py:33-282, utils.py:10-48).  RoPE is applied
to q and k, K/V may come from / go to the generation cache, the output can be gated (sigmoid) or made "exclusive"
(projection on the token's own V removed) before ``c_proj``.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ... import ops
from ...parallel.manager import ProcessGroupManager
from ...parameter import mark_parameter_as_mup_learning_rate
from ...utils import divide_if_divisible
from ..config import INVERSE, INVERSE_SQRT, SoftmaxAttentionArgs
from ..context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .activations import sigmoid
from .dropout import Dropout
from .init_utils import std_for_linear
from .linear import ColumnParallelLinear, RowParallelLinear
from .rope import apply_rotary_pos_emb


def interleave_query_key_value_tensor_for_attention(q, k, v, num_heads: int, num_key_value_heads: int,
                                                    head_dim: int) -> torch.Tensor:
    """Separate q ``[Hq*D, ...]``, k, v ``[Hkv*D, ...]`` projection weights -> fused ``c_attn`` layout."""
    G = num_heads // num_key_value_heads
    tail = q.shape[1:]
    qg = q.reshape(num_key_value_heads, G * head_dim, *tail)
    kg = k.reshape(num_key_value_heads, head_dim, *tail)
    vg = v.reshape(num_key_value_heads, head_dim, *tail)
    return torch.cat((qg, kg, vg), dim=1).reshape(-1, *tail)


def split_query_key_value_tensor_for_attention(qkv, num_heads: int, num_key_value_heads: int, head_dim: int):
    G = num_heads // num_key_value_heads
    tail = qkv.shape[1:]
    x = qkv.reshape(num_key_value_heads, (G + 2) * head_dim, *tail)
    q, k, v = x.split((G * head_dim, head_dim, head_dim), dim=1)
    return q.reshape(-1, *tail), k.reshape(-1, *tail), v.reshape(-1, *tail)


class SoftmaxAttention(nn.Module):
    def __init__(self, hidden_size: int, config: SoftmaxAttentionArgs, position_embedding_type: str,
                 init_method: str, initializer_range: float, m_width: float | None, num_layers: int, causal: bool,
                 layer_idx: int, use_depth_scaled_init: bool, use_padding_free_transformer: bool = False,
                 sequence_parallel: bool = False) -> None:
        super().__init__()
        tp = ProcessGroupManager.get_tensor_parallel_world_size()
        self.tp_world_size = tp
        self.causal, self.layer_idx = causal, layer_idx
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.global_num_heads = config.num_attention_heads
        self.global_num_key_value_heads = config.num_key_value_heads
        self.num_heads = divide_if_divisible(config.num_attention_heads, tp, "num_heads must be divisible by TP world size")
        self.num_key_value_heads = divide_if_divisible(
            config.num_key_value_heads, tp,
            f"`num_key_value_heads` ({config.num_key_value_heads}) must be divisible by `tensor_parallel_world_size` ({tp})")
        self.num_groups = divide_if_divisible(
            config.num_attention_heads, config.num_key_value_heads,
            f"`num_heads` ({config.num_attention_heads}) should be a multiple of `num_key_value_heads` "
            f"({config.num_key_value_heads})")
        self.head_dim = (divide_if_divisible(hidden_size, config.num_attention_heads)
                         if config.head_dim is None else config.head_dim)
        self.position_embedding_type = position_embedding_type
        self.attention_gate = config.attention_gate
        self.exclusive_self_attention = config.exclusive_self_attention
        self.sliding_window = config.sliding_window
        # The reference hands (sliding_window, sliding_window) to flash-attn as the window, i.e. a causal query
        # attends to itself and the `sliding_window` keys before it: sliding_window + 1 keys
        # (softmax_attention/flash_attention.py:128-130).  The ops of this repository count the attended keys, so
        # the layer passes one more: a checkpoint trained by either engine gives the same logits in the other.
        self._attended_keys = None if config.sliding_window is None else config.sliding_window + 1
        if config.attention_multiplier_method == INVERSE_SQRT:
            self.attention_multiplier = 1 / math.sqrt(self.head_dim)
        elif config.attention_multiplier_method == INVERSE:
            self.attention_multiplier = 1 / self.head_dim
        else:
            self.attention_multiplier = config.attention_multiplier
        D = self.head_dim
        qkv_out = (config.num_attention_heads + 2 * config.num_key_value_heads) * D
        if self.attention_gate:
            qkv_out += config.num_attention_heads * D
        self.c_attn = ColumnParallelLinear(
            hidden_size, qkv_out, bias=config.add_bias,
            std=std_for_linear(initializer_range, init_method, m_width, hidden_size, num_layers, False),
            use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel)
        fan_in = config.num_attention_heads * D
        self.c_proj = RowParallelLinear(
            fan_in, hidden_size, bias=config.add_bias,
            std=std_for_linear(initializer_range, init_method, m_width, fan_in, num_layers, use_depth_scaled_init),
            use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel)
        self.softmax_dropout_p = config.softmax_dropout
        self.dropout = Dropout(config.dropout)
        mark_parameter_as_mup_learning_rate(self.c_attn.weight)
        mark_parameter_as_mup_learning_rate(self.c_proj.weight)

    def forward(self, x: torch.Tensor, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        attention_mask_info, position_info = resolve_attention_and_position_info(attention_mask_info, position_info)
        Hkv, G, D = self.num_key_value_heads, self.num_groups, self.head_dim
        qkv = self.c_attn(x)
        lead = qkv.shape[:-1]
        use_rope = self.position_embedding_type == "rope"
        g = v_self = None
        if not self.attention_gate and qkv.is_cuda and qkv.dtype == torch.bfloat16:
            cos_t, sin_t = position_info.rope_tables if use_rope else (None, None)
            seq = position_info.sequence_length or (lead[-1] if len(lead) > 1 else 1)
            q, k, v = ops.qkv_split_rope(qkv, Hkv, G, D, cos_t, sin_t,
                                         position_info.position_ids if use_rope else None, seq)
        else:
            parts = (G * D, D, D) + ((G * D,) if self.attention_gate else ())
            sp = qkv.view(*lead, Hkv, sum(parts)).split(parts, dim=-1)
            q, k, v = sp[0].reshape(*lead, Hkv * G, D), sp[1], sp[2]
            if self.attention_gate:
                g = sp[3].reshape(*lead, Hkv * G, D)
            if use_rope:
                q = apply_rotary_pos_emb(q, position_info.rope_cos_sin)
                k = apply_rotary_pos_emb(k, position_info.rope_cos_sin)
        if self.exclusive_self_attention:
            v_self = v
        if cache_params is not None:
            k = cache_params.update(self.layer_idx, "key", k)
            v = cache_params.update(self.layer_idx, "value", v)
        packed = self.use_padding_free_transformer
        out = self._attend(q, k, v, attention_mask_info, packed)
        if self.exclusive_self_attention:
            out = self._remove_self_projection(out, v_self)
        if g is not None:
            out = out * sigmoid(g)
        out = out.flatten(-2, -1)
        fuse_res = residual is not None and self.dropout.p == 0
        out = self.c_proj(out, residual if fuse_res else None)
        out = self.dropout(out)
        if residual is not None and not fuse_res:
            out = out + residual
        return out

    def _attend(self, q, k, v, info: AttentionMaskInfo, packed: bool) -> torch.Tensor:
        from ...parallel.ring_attention import ring_attention

        dropout = self.softmax_dropout_p if self.training else 0.0
        if ProcessGroupManager.is_context_parallel_enabled():
            from ...parallel.ulysses import ulysses_attention, ulysses_eligible

            how = ProcessGroupManager.get_context_parallel_attention()
            cp = ProcessGroupManager.get_context_parallel_world_size()
            if how == "ulysses" or (how == "auto" and ulysses_eligible(q.size(-2), k.size(-2), cp)):
                return ulysses_attention(q, k, v, causal=self.causal, softmax_scale=self.attention_multiplier,
                                         sliding_window=self._attended_keys, dropout_p=dropout)
            from ...parallel import gathered_attention as gathered

            method = ProcessGroupManager.get_context_parallel_load_balancing_method()
            if how == "gathered" and dropout == 0 and gathered.eligible(q, k, self.causal, self._attended_keys,
                                                                        method):
                # the K / V exchange runs inside the attention kernel (copy engines + readiness words).  Opt-in:
                # it matches one GPU on 2 GPUs, but on 4 GPUs (2.7B hybrid, 32768 tokens) readiness words of some
                # launches never arrived and the bounded waits ran out; until that is understood `auto` takes the ring
                return gathered.gathered_kv_attention(q, k, v, softmax_scale=self.attention_multiplier)
            return ring_attention(q, k, v, causal=self.causal, softmax_scale=self.attention_multiplier,
                                  sliding_window=self._attended_keys)
        if packed:
            return ops.attention(q, k, v, causal=self.causal, softmax_scale=self.attention_multiplier,
                                 sliding_window=self._attended_keys, cu_seqlens=info.cu_seqlens,
                                 max_seqlen=info.max_seqlen, dropout_p=dropout)
        return ops.attention(q, k, v, causal=self.causal, softmax_scale=self.attention_multiplier,
                             sliding_window=self._attended_keys, attention_mask=info.attention_mask,
                             dropout_p=dropout)

    @staticmethod
    def _remove_self_projection(x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if v.size(-2) != x.size(-2):
            v = v.repeat_interleave(x.size(-2) // v.size(-2), dim=-2)
        v = v.float()
        coef = (x * v).sum(-1, keepdim=True) / (v * v).sum(-1, keepdim=True)
        return (x - coef * v).type_as(x)
