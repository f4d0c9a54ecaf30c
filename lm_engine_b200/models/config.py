"""Model configuration: ``CommonConfig`` with per-layer lists of sequence-mixer and MLP block arguments.

The field set and JSON form are the reference's (lm_engine/model_config.py:34-186 and the ``*Args`` classes under
lm_engine/modeling_utils/**/config.py), so ``config.json`` files and inline ``pretrained_config`` dicts are
interchangeable.  Model families differ only in ``model_type``.
"""

from __future__ import annotations

import json
import os
from typing import Annotated, Any, Literal

from pydantic import Field

from ..arguments.base import BaseArgs
from ..utils import divide_if_divisible

INVERSE_SQRT = "1 / sqrt(head_dim)"
INVERSE = "1 / head_dim"


class SoftmaxAttentionArgs(BaseArgs):
    sequence_mixer_type: Literal["softmax_attention"] = "softmax_attention"
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int | None = None
    softmax_dropout: float = 0
    dropout: float = 0
    add_bias: bool = False
    attention_multiplier: float | None = None
    attention_multiplier_method: str | None = INVERSE_SQRT
    attention_gate: bool = False
    exclusive_self_attention: bool = False
    sliding_window: int | None = None

    def model_post_init(self, _ctx: Any) -> None:
        assert self.attention_multiplier_method in (INVERSE_SQRT, INVERSE, None)
        if self.attention_multiplier_method is None:
            assert self.attention_multiplier is not None
        else:
            assert self.attention_multiplier is None


class SoftPlusDecayGateArgs(BaseArgs):
    A_init_min: float = 0
    A_init_max: float = 16
    dt_init_min: float = 0.001
    dt_init_max: float = 0.1
    dt_init_floor: float = 1e-4

    def model_post_init(self, _ctx: Any) -> None:
        assert 0 <= self.A_init_min <= self.A_init_max
        assert self.dt_init_min <= self.dt_init_max


class Mamba2Args(SoftPlusDecayGateArgs):
    sequence_mixer_type: Literal["mamba2"] = "mamba2"
    state_size: int
    intermediate_size: int
    num_heads: int
    conv_kernel_size: int
    time_step_limit: tuple[float, float] = (0, float("inf"))
    add_bias: bool = False
    use_conv_bias: bool = True
    activation_function: str
    num_groups: int
    chunk_size: int = 256
    normalization_function: str | None


class GatedDeltaNetArgs(SoftPlusDecayGateArgs):
    sequence_mixer_type: Literal["gated_deltanet"] = "gated_deltanet"
    k_head_dim: int
    v_head_dim: int
    num_k_heads: int
    num_v_heads: int
    use_gate: bool
    attention_multiplier: float | None
    allow_neg_eigval: bool
    kernel_size: int


class GRUArgs(BaseArgs):
    sequence_mixer_type: Literal["gru"] = "gru"
    state_head_dim: int
    num_input_heads: int
    num_forget_input_heads: int
    num_reset_input_heads: int
    num_weight_heads: int
    num_forget_weight_heads: int
    num_reset_weight_heads: int
    add_bias: bool
    normalization_function: str | None
    gradient_clipping: float | None
    kernel_size: int | None
    activation_function: str | None


class RNNArgs(BaseArgs):
    sequence_mixer_type: Literal["rnn"] = "rnn"
    state_head_dim: int
    num_input_heads: int
    num_weight_heads: int
    add_bias: bool
    normalization_function: str | None
    gradient_clipping: float | None
    kernel_size: int | None
    activation_function: str | None


class M2RNNArgs(SoftPlusDecayGateArgs):
    sequence_mixer_type: Literal["m2rnn"] = "m2rnn"
    k_head_dim: int
    v_head_dim: int
    num_q_heads: int
    num_k_heads: int
    num_v_heads: int
    num_f_heads: int
    num_g_heads: int
    num_weight_heads: int
    use_residual: bool
    kernel_size: int | None
    activation_function: str | None
    add_bias: bool
    gradient_clipping: float | None
    normalization_function: str | None


class LinearAttentionArgs(SoftPlusDecayGateArgs):
    sequence_mixer_type: Literal["linear_attention"] = "linear_attention"
    k_head_dim: int
    v_head_dim: int
    num_q_heads: int
    num_k_heads: int
    num_v_heads: int
    num_g_heads: int
    kernel_size: int | None
    activation_function: str | None
    add_bias: bool
    normalization_function: str | None
    attention_multiplier: float | None


class MLPArgs(BaseArgs):
    mlp_type: Literal["MLP"] = "MLP"
    intermediate_size: int
    activation_function: str
    dropout: float = 0
    add_bias: bool = False


class MoEArgs(MLPArgs):
    mlp_type: Literal["MoE"] = "MoE"
    shared_intermediate_size: int | None
    num_experts: int
    num_experts_per_tok: int
    shared_expert_gating: bool = False
    normalized_topk: bool = True


SequenceMixerArgs = Annotated[
    SoftmaxAttentionArgs | Mamba2Args | GRUArgs | RNNArgs | M2RNNArgs | GatedDeltaNetArgs | LinearAttentionArgs,
    Field(discriminator="sequence_mixer_type"),
]
MLPBlockArgs = Annotated[MLPArgs | MoEArgs, Field(discriminator="mlp_type")]

_HF_KEYS = {"name_or_path", "_name_or_path", "architectures", "_from_auto", "_commit_hash", "transformers_version",
            "auto_map", "torch_dtype", "dtype"}


class CommonConfig(BaseArgs):
    model_type: str = None
    vocab_size: int
    max_position_embeddings: int
    hidden_size: int
    num_layers: int
    embedding_dropout: float = 0
    normalization_function: str
    layer_norm_epsilon: float = 1e-5
    initializer_range: float
    bos_token_id: int
    eos_token_id: int
    pad_token_id: int
    position_embedding_type: Literal["rope", "learned_absolute", "nope"]
    rope_theta: int
    rope_scaling: dict | None
    m_emb: float | None
    m_width: float | None
    m_residual: float | None
    init_method: Literal["normal", "mup", "fan_in"]
    embedding_init_method: Literal["normal", "mup", "fan_in"]
    use_depth_scaled_init: bool
    sequence_mixer_blocks: list[SequenceMixerArgs]
    mlp_blocks: list[MLPBlockArgs]
    tie_word_embeddings: bool
    router_aux_loss_coef: float | None = None
    rope_dim: int | None = None
    # gpt_crosslayer only: layer i reuses the KV projection of layer sharing_pattern[i]
    sharing_pattern: list[int] | None = None

    def model_post_init(self, _ctx: Any) -> None:
        assert len(self.sequence_mixer_blocks) == self.num_layers, (
            f"sequence_mixer_blocks has {len(self.sequence_mixer_blocks)} entries but num_layers={self.num_layers}")
        assert len(self.mlp_blocks) == self.num_layers, (
            f"mlp_blocks has {len(self.mlp_blocks)} entries but num_layers={self.num_layers}")
        if self.position_embedding_type == "rope":
            assert self.rope_theta is not None
            if self.rope_dim is None:
                kinds = {b.sequence_mixer_type for b in self.sequence_mixer_blocks}
                assert kinds == {"softmax_attention"}, "specify rope_dim"
                self.rope_dim = self.uniform_value("sequence_mixer_blocks", "head_dim")
                if self.rope_dim is None:
                    self.rope_dim = divide_if_divisible(
                        self.hidden_size, self.uniform_value("sequence_mixer_blocks", "num_attention_heads"))

    # ------------------------------------------------------------------ helpers
    def uniform_value(self, list_name: str, key: str, *, sequence_mixer_type: str | None = None,
                      mlp_type: str | None = None, expected: Any = None) -> Any:
        """Value of ``key`` shared by all (optionally filtered) blocks of ``list_name``; asserts that it is shared."""
        blocks = list(getattr(self, list_name))
        if sequence_mixer_type is not None:
            blocks = [b for b in blocks if b.sequence_mixer_type == sequence_mixer_type]
        if mlp_type is not None:
            blocks = [b for b in blocks if b.mlp_type == mlp_type]
        value = getattr(blocks[0], key)
        assert all(getattr(b, key) == value for b in blocks), f"{key} differs between layers"
        if expected is not None:
            assert value == expected, f"{value} {expected}"
        return value

    # kept under the reference's name for callers that use it
    def check_equal_for_all_and_get_value(self, key: str, key_block: str, expected_value: Any = None,
                                          sequence_mixer_type: str | None = None, mlp_type: str | None = None) -> Any:
        return self.uniform_value(key, key_block, sequence_mixer_type=sequence_mixer_type, mlp_type=mlp_type,
                                  expected=expected_value)

    # ------------------------------------------------------------------ (de)serialisation, HF-compatible
    def to_dict(self) -> dict:
        d = super().to_dict()
        if d.get("sharing_pattern") is None:
            d.pop("sharing_pattern", None)
        for blk in d["sequence_mixer_blocks"]:
            if "time_step_limit" in blk:
                blk["time_step_limit"] = list(blk["time_step_limit"])
        return d

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=4)

    def save_pretrained(self, save_directory: str, **_: Any) -> None:
        os.makedirs(save_directory, exist_ok=True)
        d = self.to_dict()
        d["architectures"] = [architecture_name(self.model_type)]
        with open(os.path.join(save_directory, "config.json"), "w") as f:
            json.dump(d, f, indent=4)

    @classmethod
    def from_dict(cls, config_dict: dict, **kwargs: Any):
        unused = kwargs.pop("return_unused_kwargs", False)
        cfg = cls(**{k: v for k, v in config_dict.items() if k not in _HF_KEYS})
        return (cfg, kwargs) if unused else cfg

    @classmethod
    def from_pretrained(cls, path: str, **kwargs: Any):
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f), **kwargs)


MODEL_TYPES = ("gpt_base", "palm", "ladder_residual", "gpt_crosslayer")


def architecture_name(model_type: str) -> str:
    return {"gpt_base": "GPTBaseForCausalLM", "palm": "PaLMForCausalLM",
            "ladder_residual": "LadderResidualForCausalLM",
            "gpt_crosslayer": "GPTCrossLayerForCausalLM"}[model_type]


def config_from_dict(d: dict) -> CommonConfig:
    d = dict(d)
    d.setdefault("model_type", "gpt_base")
    if d["model_type"] not in MODEL_TYPES:
        raise ValueError(f"unknown model_type {d['model_type']}")
    return CommonConfig.from_dict(d)


def dense_config(*, vocab_size: int, hidden_size: int, num_layers: int, num_attention_heads: int,
                 num_key_value_heads: int, intermediate_size: int, max_position_embeddings: int = 4096,
                 rope_theta: int = 10000, head_dim: int | None = None, activation_function: str = "swiglu",
                 normalization_function: str = "rmsnorm", layer_norm_epsilon: float = 1e-5,
                 initializer_range: float = 0.02, tie_word_embeddings: bool = False,
                 model_type: str = "gpt_base", **extra: Any) -> CommonConfig:
    """Convenience constructor for a homogeneous Llama-style decoder."""
    return CommonConfig(
        model_type=model_type, vocab_size=vocab_size, max_position_embeddings=max_position_embeddings,
        hidden_size=hidden_size, num_layers=num_layers, normalization_function=normalization_function,
        layer_norm_epsilon=layer_norm_epsilon, initializer_range=initializer_range,
        bos_token_id=extra.pop("bos_token_id", 0), eos_token_id=extra.pop("eos_token_id", 1),
        pad_token_id=extra.pop("pad_token_id", 2), position_embedding_type=extra.pop("position_embedding_type", "rope"),
        rope_theta=rope_theta, rope_scaling=extra.pop("rope_scaling", None), m_emb=extra.pop("m_emb", None),
        m_width=extra.pop("m_width", None), m_residual=extra.pop("m_residual", None),
        init_method=extra.pop("init_method", "normal"), embedding_init_method=extra.pop("embedding_init_method", "normal"),
        use_depth_scaled_init=extra.pop("use_depth_scaled_init", False),
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=num_attention_heads,
                                    num_key_value_heads=num_key_value_heads, head_dim=head_dim)
                               for _ in range(num_layers)],
        mlp_blocks=[dict(mlp_type="MLP", intermediate_size=intermediate_size, activation_function=activation_function)
                    for _ in range(num_layers)],
        tie_word_embeddings=tie_word_embeddings, **extra)
