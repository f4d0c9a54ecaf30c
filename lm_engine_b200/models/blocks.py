"""Decoder blocks of the model families and the factories that pick a sequence mixer / MLP per layer.

* ``Block``            pre-norm residual block (gpt_base; lm_engine/mixins/dense/layer.py:22-92)
* ``PaLMBlock``        attention and MLP in parallel from one norm (lm_engine/models/palm/layer.py:22-75)
* ``LadderBlock``      each sub-layer's output joins the residual stream one sub-layer late
                       (lm_engine/models/ladder_residual/layer.py)
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .config import CommonConfig
from .context import AttentionMaskInfo, GenerationCache, PositionInfo
from .layers.mlp import MLP
from .layers.norm import get_normalization_function


def get_sequence_mixer(config: CommonConfig, causal: bool, use_padding_free_transformer: bool, layer_idx: int,
                       sequence_parallel: bool = False) -> nn.Module:
    block = config.sequence_mixer_blocks[layer_idx]
    kind = block.sequence_mixer_type
    common = dict(init_method=config.init_method, initializer_range=config.initializer_range,
                  m_width=config.m_width, num_layers=config.num_layers, layer_idx=layer_idx,
                  use_padding_free_transformer=use_padding_free_transformer)
    if kind == "softmax_attention":
        from .layers.attention import SoftmaxAttention

        return SoftmaxAttention(config.hidden_size, block, config.position_embedding_type, causal=causal,
                                use_depth_scaled_init=config.use_depth_scaled_init,
                                sequence_parallel=sequence_parallel, **common)
    from ..parallel.manager import ProcessGroupManager

    if kind != "m2rnn":
        assert not ProcessGroupManager.is_tensor_parallel_enabled(), f"{kind} does not support tensor parallel"
    if kind == "mamba2":
        from .layers.mamba2 import Mamba2

        return Mamba2(config.hidden_size, block, layer_norm_epsilon=config.layer_norm_epsilon, **common)
    if kind == "gated_deltanet":
        from .layers.gated_deltanet import GatedDeltaNet

        return GatedDeltaNet(config.hidden_size, block, layer_norm_epsilon=config.layer_norm_epsilon,
                             use_depth_scaled_init=config.use_depth_scaled_init, **common)
    if kind in ("gru", "rnn"):
        from .layers.recurrent import GRU, RNN

        cls = GRU if kind == "gru" else RNN
        return cls(config.hidden_size, block, layer_norm_epsilon=config.layer_norm_epsilon,
                   use_depth_scaled_init=config.use_depth_scaled_init, **common)
    if kind == "m2rnn":
        from .layers.m2rnn import M2RNN

        return M2RNN(config.hidden_size, block, layer_norm_epsilon=config.layer_norm_epsilon,
                     use_depth_scaled_init=config.use_depth_scaled_init, **common)
    if kind == "linear_attention":
        from .layers.linear_attention import LinearAttention

        return LinearAttention(config.hidden_size, block, layer_norm_epsilon=config.layer_norm_epsilon,
                               use_depth_scaled_init=config.use_depth_scaled_init, **common)
    raise ValueError(f"unexpected sequence_mixer_type ({kind})")


def get_mlp_block(config: CommonConfig, use_padding_free_transformer: bool, sequence_parallel: bool,
                  layer_idx: int) -> nn.Module:
    block = config.mlp_blocks[layer_idx]
    common = dict(hidden_size=config.hidden_size, config=block, init_method=config.init_method,
                  initializer_range=config.initializer_range, m_width=config.m_width, num_layers=config.num_layers,
                  use_depth_scaled_init=config.use_depth_scaled_init,
                  use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel)
    if block.mlp_type == "MLP":
        return MLP(**common)
    if block.mlp_type == "MoE":
        from .layers.moe import MoE

        return MoE(**common)
    raise ValueError(f"invalid mlp_type ({block.mlp_type}) for layer ({layer_idx})")


def _supports_residual(module: nn.Module) -> bool:
    return getattr(module, "accepts_residual", False) or type(module).__name__ in ("MLP", "SoftmaxAttention")


class Block(nn.Module):
    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int,
                 sequence_parallel: bool = False) -> None:
        super().__init__()
        H = config.hidden_size
        self.layer_idx = layer_idx
        self.m_residual = config.m_residual
        self.ln_1 = get_normalization_function(config.normalization_function, H, eps=config.layer_norm_epsilon,
                                               sequence_parallel=sequence_parallel)
        self.sequence_mixer = get_sequence_mixer(config, True, use_padding_free_transformer, layer_idx,
                                                 sequence_parallel)
        self.ln_2 = get_normalization_function(config.normalization_function, H, eps=config.layer_norm_epsilon,
                                               sequence_parallel=sequence_parallel)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer, sequence_parallel, layer_idx)
        self._fuse_mixer = self.m_residual is None and _supports_residual(self.sequence_mixer)
        self._fuse_mlp = self.m_residual is None and _supports_residual(self.mlp_block)

    def forward(self, x: torch.Tensor, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None,
                position_info: PositionInfo | None = None) -> torch.Tensor:
        kw = dict(cache_params=cache_params, attention_mask_info=attention_mask_info, position_info=position_info)
        # the residual add is folded into the epilogue of each branch's output projection when possible
        if self._fuse_mixer:
            x = self.sequence_mixer(self.ln_1(x), residual=x, **kw)
        else:
            y = self.sequence_mixer(self.ln_1(x), **kw)
            x = x + (y if self.m_residual is None else y * self.m_residual)
        if self._fuse_mlp:
            x = self.mlp_block(self.ln_2(x), residual=x)
        else:
            y = self.mlp_block(self.ln_2(x))
            x = x + (y if self.m_residual is None else y * self.m_residual)
        return x


class PaLMBlock(nn.Module):
    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int,
                 sequence_parallel: bool = False) -> None:
        super().__init__()
        self.m_residual = config.m_residual
        self.ln = get_normalization_function(config.normalization_function, config.hidden_size,
                                             eps=config.layer_norm_epsilon, sequence_parallel=sequence_parallel)
        self.sequence_mixer = get_sequence_mixer(config, True, use_padding_free_transformer, layer_idx,
                                                 sequence_parallel)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer, sequence_parallel, layer_idx)

    def forward(self, x, cache_params=None, attention_mask_info=None, position_info=None):
        h = self.ln(x)
        a = self.sequence_mixer(h, cache_params=cache_params, attention_mask_info=attention_mask_info,
                                position_info=position_info)
        m = self.mlp_block(h)
        y = a + m
        if self.m_residual is not None:
            y = y * self.m_residual
        return x + y


class LadderBlock(Block):
    """Ladder residual: the block consumes the previous sub-layers' pending outputs.  State flows through the
    triple ``(residual, pending_attention_out, pending_mlp_out)``."""

    def forward(self, state, cache_params=None, attention_mask_info=None, position_info=None):
        residual, pending_attn, pending_mlp = state
        if pending_attn is not None:
            residual = residual + pending_attn
        h = self.ln_1(residual)
        cur_attn = self.sequence_mixer(h, cache_params=cache_params, attention_mask_info=attention_mask_info,
                                       position_info=position_info)
        if self.m_residual is not None:
            cur_attn = cur_attn * self.m_residual
        if pending_mlp is not None:
            residual = residual + pending_mlp
        h = self.ln_2(residual)
        cur_mlp = self.mlp_block(h)
        if self.m_residual is not None:
            cur_mlp = cur_mlp * self.m_residual
        return residual, cur_attn, cur_mlp
