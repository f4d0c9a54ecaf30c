"""Model families: gpt_base, palm, ladder_residual, gpt_crosslayer (lm_engine/models/*)."""

from __future__ import annotations

from .base import (
    BaseModelOutputWithPast,
    CausalLM,
    CausalLMOutputWithPast,
    LadderResidualForCausalLM,
    PaLMForCausalLM,
    PipelineParallelInput,
    PipelineParallelOutput,
    TransformerModel,
)
from .config import CommonConfig, config_from_dict, dense_config
from .context import AttentionMaskInfo, GenerationCache, PositionInfo

GPTBaseForCausalLM = CausalLM
GPTBaseModel = TransformerModel


def get_causal_lm_class(model_type: str) -> type[CausalLM]:
    if model_type == "gpt_base":
        return CausalLM
    if model_type == "palm":
        return PaLMForCausalLM
    if model_type == "ladder_residual":
        return LadderResidualForCausalLM
    if model_type == "gpt_crosslayer":
        from .crosslayer import GPTCrossLayerForCausalLM

        return GPTCrossLayerForCausalLM
    raise ValueError(f"unknown model_type {model_type}")


def build_model(config: CommonConfig | dict, **kwargs) -> CausalLM:
    if isinstance(config, dict):
        config = config_from_dict(config)
    return get_causal_lm_class(config.model_type or "gpt_base")(config, **kwargs)
