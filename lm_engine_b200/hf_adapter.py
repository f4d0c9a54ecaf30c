"""Inference adapter around a raw ``CausalLM``: checkpoint I/O for every architecture of this package and a
``generate`` loop with the package's own ``GenerationCache`` (role of lm_engine/hf_adapter.py:58-343).

``LLMAdapter_HF.from_pretrained(path, config=...)`` loads either a safetensors directory or, when ``path`` holds
``latest_checkpointed_iteration.json``, a sharded training checkpoint that is unsharded on the fly.
``generate`` is Hugging Face's (the adapter is a ``PreTrainedModel`` + ``GenerationMixin``); ``generate_simple``
decodes greedily or samples (temperature / top-k / top-p) for left-padded batches and stops rows at
``eos_token_id`` without that machinery; ``forward`` returns ``loss`` (mean, shifted) / ``logits`` / ``past_key_values`` under the field
names Hugging Face evaluation code expects.  The adapter is for single-stage, padded (not packed) inference.
"""

from __future__ import annotations

import os
from contextlib import nullcontext
from dataclasses import dataclass

import torch
import torch.nn as nn

from .loss import get_autoregressive_language_modeling_loss
from .models import AttentionMaskInfo, CommonConfig, PositionInfo, get_causal_lm_class as _get_class
from .models.context import GenerationCache
from .utils import SafeTensorsWeightsManager, disable_generation_cache

_CUSTOM_MODEL_TYPES = ("gpt_base", "gpt_crosslayer", "ladder_residual", "palm")
_IGNORED_HF_KWARGS = ("revision", "subfolder", "gguf_file", "quantization_config", "max_memory", "name_or_path",
                      "trust_remote_code", "adapter_kwargs", "low_cpu_mem_usage")
_MODEL_CONSTRUCTOR_KWARGS = ("use_padding_free_transformer", "sequence_parallel", "num_pipeline_stages",
                             "pipeline_stage_id")


def is_custom_model(model_type: str) -> bool:
    return model_type in _CUSTOM_MODEL_TYPES


def get_causal_lm_class(model_type: str):
    return _get_class(model_type)


try:    # the adapter is a transformers model when that package is importable, else a plain module
    from transformers import GenerationMixin, PretrainedConfig, PreTrainedModel
    from transformers.utils import ModelOutput

    _HAVE_TRANSFORMERS = True
except Exception:  # noqa: BLE001
    _HAVE_TRANSFORMERS = False
    GenerationMixin = object
    PreTrainedModel = nn.Module
    PretrainedConfig = object
    ModelOutput = object


if _HAVE_TRANSFORMERS:

    @dataclass
    class AdapterOutput(ModelOutput):
        """``loss`` / ``logits`` / ``past_key_values`` under the names ``GenerationMixin`` looks for."""

        loss: torch.Tensor | None = None
        logits: torch.Tensor | None = None
        past_key_values: GenerationCache | None = None

    class LLMAdapterConfig(PretrainedConfig):
        """What ``PreTrainedModel`` / ``GenerationMixin`` read from a config (token ids, sizes), filled from the
        package's own :class:`CommonConfig`; the full model description travels along as ``common``."""

        model_type = "lm_engine_b200_adapter"

        def __init__(self, common: dict | None = None, **kwargs) -> None:
            common = dict(common or {})
            self.common = common
            for k in ("bos_token_id", "eos_token_id", "pad_token_id"):
                kwargs.setdefault(k, common.get(k))
            self.vocab_size = common.get("vocab_size")
            self.hidden_size = common.get("hidden_size")
            self.num_hidden_layers = common.get("num_layers")
            self.max_position_embeddings = common.get("max_position_embeddings")
            kwargs.setdefault("tie_word_embeddings", bool(common.get("tie_word_embeddings", False)))
            super().__init__(**kwargs)

        @classmethod
        def from_common_config(cls, config: CommonConfig) -> "LLMAdapterConfig":
            return cls(common=config.to_dict())

else:

    @dataclass
    class AdapterOutput:
        loss: torch.Tensor | None = None
        logits: torch.Tensor | None = None
        past_key_values: GenerationCache | None = None


class LLMAdapter_HF(PreTrainedModel, GenerationMixin):
    """``transformers.PreTrainedModel`` + ``GenerationMixin`` around an already built ``CausalLM`` of this package, so
    that ``model.generate(...)`` with the Hugging Face arguments (beam search, logits processors, stopping criteria,
    streamers), ``transformers.pipeline`` and evaluation harnesses work unchanged (lm_engine/hf_adapter.py:107-272).
    The cache is the package's own :class:`GenerationCache`; :meth:`generate_simple` is a dependency-free greedy /
    sampling loop over the same ``forward``."""

    if _HAVE_TRANSFORMERS:
        config_class = LLMAdapterConfig
        base_model_prefix = "model"
        main_input_name = "input_ids"
        _supports_cache_class = False

    def __init__(self, model: nn.Module) -> None:
        if _HAVE_TRANSFORMERS:
            super().__init__(LLMAdapterConfig.from_common_config(model.config))
        else:
            super().__init__()
            self.config = model.config
        self.model = model
        self.common_config = model.config

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        # the models create their own cache on the first forward call; generate() must not build a DynamicCache
        return False

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs) -> dict:
        """One decoding step's inputs: the whole prompt on the first call, the newest token afterwards; positions
        count the real tokens of a left-padded row."""
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        pos = (attention_mask.long().cumsum(-1) - 1).clamp_min(0)
        use_cache = kwargs.get("use_cache", True)
        if past_key_values is not None and use_cache:
            input_ids, pos = input_ids[:, -1:], pos[:, -1:]
        return {"input_ids": input_ids, "attention_mask": attention_mask, "position_ids": pos,
                "past_key_values": past_key_values if use_cache else None, "use_cache": use_cache}

    # ------------------------------------------------------------------ construction / IO
    @classmethod
    def _from_config(cls, config: CommonConfig, dtype: torch.dtype | None = None, **kwargs) -> "LLMAdapter_HF":
        model = _get_class(config.model_type)(config, **kwargs)
        return cls(model.to(dtype) if dtype is not None else model)

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, *model_args, config: CommonConfig | None = None,
                        dtype: torch.dtype = torch.float32, iteration: int | None = None,
                        **kwargs) -> "LLMAdapter_HF":
        assert not model_args
        for k in _IGNORED_HF_KWARGS:
            kwargs.pop(k, None)
        dtype = kwargs.pop("torch_dtype", None) or dtype
        model_kwargs = {k: kwargs.pop(k) for k in _MODEL_CONSTRUCTOR_KWARGS if k in kwargs}
        device_map = kwargs.pop("device_map", {"": None})
        assert isinstance(device_map, dict) and set(device_map) == {""}, (
            f"only device_map={{'': <device>}} is supported, got {device_map!r}")
        assert not kwargs, f"unexpected arguments {sorted(kwargs)}"
        path = pretrained_model_name_or_path
        if os.path.isfile(os.path.join(path, "latest_checkpointed_iteration.json")):
            from .arguments import LoadArgs, MixedPrecisionArgs, UnshardingArgs
            from .checkpointing import load_checkpoint_and_unshard
            from .utils import torch_dtype_to_string

            args = UnshardingArgs(load_args=LoadArgs(load_path=path, iteration=iteration),
                                  mixed_precision_args=MixedPrecisionArgs(dtype=torch_dtype_to_string(dtype)),
                                  unsharded_path="")
            wrapper, _, _ = load_checkpoint_and_unshard(args)
            model = wrapper.model
        else:
            assert iteration is None, "iteration only applies to sharded training checkpoints"
            if config is None:
                config = CommonConfig.from_pretrained(path)
            model = _get_class(config.model_type)(config, **model_kwargs).to(dtype)
            model.load_from_safetensors_weights_manager(SafeTensorsWeightsManager(path))
        if device_map[""] is not None:
            model = model.to(device_map[""])
        return cls(model)

    def save_pretrained(self, save_directory: str, **_unused) -> None:
        self.model.config.save_pretrained(save_directory)
        SafeTensorsWeightsManager.save_state_dict(self.model.state_dict(), save_directory)

    # ------------------------------------------------------------------ HF-style accessors
    def can_generate(self) -> bool:
        return True

    def get_input_embeddings(self):
        return self.model.transformer.wte if self.model.is_first_stage else None

    def set_input_embeddings(self, value) -> None:
        self.model.transformer.wte = value

    def get_output_embeddings(self):
        return self.model.get_output_embeddings() if self.model.is_last_stage else None

    def set_output_embeddings(self, value) -> None:
        if not self.model._tied_word_embeddings:
            self.model.lm_head = value

    @property
    def device(self) -> torch.device:
        return next(self.model.parameters()).device

    # ------------------------------------------------------------------ forward / generate
    def forward(self, input_ids: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None,
                position_ids: torch.Tensor | None = None, past_key_values: GenerationCache | None = None,
                inputs_embeds: torch.Tensor | None = None, labels: torch.Tensor | None = None,
                use_cache: bool | None = None, **_ignored) -> AdapterOutput:
        assert inputs_embeds is None, "inputs_embeds is not supported"
        with nullcontext() if use_cache else disable_generation_cache():
            out = self.model(input_ids=input_ids, cache_params=past_key_values,
                             attention_mask_info=AttentionMaskInfo(attention_mask=attention_mask),
                             position_info=PositionInfo(position_ids=position_ids))
        loss = None
        if labels is not None:
            loss = get_autoregressive_language_modeling_loss(
                lm_logits=out.logits, labels=labels, reduction="mean", shift_logits_and_labels=True,
                tensor_parallel_enabled=False, use_padding_free_transformer=False)
        return AdapterOutput(loss=loss, logits=out.logits, past_key_values=out.cache_params)

    @torch.no_grad()
    def generate_simple(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                        max_new_tokens: int = 20, do_sample: bool = False, temperature: float = 1.0,
                 top_k: int | None = None, top_p: float | None = None, eos_token_id: int | None = None,
                 pad_token_id: int | None = None, generator: torch.Generator | None = None,
                 use_cache: bool = True, **_ignored) -> torch.Tensor:
        """Returns ``[batch, prompt + new]`` token ids.  Prompts are left-padded (``attention_mask`` 0 on padding);
        finished rows keep emitting ``pad_token_id``."""
        was_training = self.model.training
        self.model.eval()
        cfg = self.common_config
        eos = cfg.eos_token_id if eos_token_id is None else eos_token_id
        pad = pad_token_id if pad_token_id is not None else (cfg.pad_token_id if cfg.pad_token_id is not None
                                                             else eos)
        B = input_ids.size(0)
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        tokens, mask = input_ids, attention_mask
        done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
        cache = None
        for _ in range(max_new_tokens):
            pos = (mask.long().cumsum(-1) - 1).clamp_min(0)
            if use_cache and cache is not None:
                step = self.forward(tokens[:, -1:], attention_mask=mask, position_ids=pos[:, -1:],
                                    past_key_values=cache, use_cache=True)
            else:
                step = self.forward(tokens, attention_mask=mask, position_ids=pos, use_cache=use_cache)
            cache = step.past_key_values if use_cache else None
            logits = step.logits[:, -1].float()
            if do_sample:
                nxt = _sample(logits, temperature, top_k, top_p, generator)
            else:
                nxt = logits.argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            tokens = torch.cat((tokens, nxt[:, None]), dim=1)
            mask = torch.cat((mask, torch.ones_like(mask[:, :1])), dim=1)
            if eos is not None:
                done = done | (nxt == eos)
                if bool(done.all()):
                    break
        self.model.train(was_training)
        return tokens


def _sample(logits: torch.Tensor, temperature: float, top_k: int | None, top_p: float | None,
            generator: torch.Generator | None) -> torch.Tensor:
    if temperature != 1.0:
        logits = logits / max(temperature, 1e-6)
    if top_k is not None and 0 < top_k < logits.size(-1):
        kth = logits.topk(top_k, dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0 < top_p < 1:
        srt, idx = logits.sort(dim=-1, descending=True)
        probs = srt.softmax(-1)
        drop = probs.cumsum(-1) - probs > top_p    # keep the smallest prefix whose mass reaches top_p
        srt = srt.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return torch.multinomial(logits.softmax(-1), 1, generator=generator).squeeze(-1)


def register_model_classes() -> None:
    """Registers the architectures with ``transformers``' Auto classes when that package is importable:
    ``AutoConfig`` resolves the ``model_type`` of exported checkpoints, and ``AutoModelForCausalLM`` maps the
    adapter's config to :class:`LLMAdapter_HF`."""
    if not _HAVE_TRANSFORMERS:
        return
    from transformers import AutoConfig, AutoModelForCausalLM

    for mt in _CUSTOM_MODEL_TYPES:
        shim = type(f"{mt}_Config", (PretrainedConfig,), {"model_type": mt})
        try:
            AutoConfig.register(mt, shim)
        except ValueError:
            pass
    try:
        AutoConfig.register(LLMAdapterConfig.model_type, LLMAdapterConfig)
        AutoModelForCausalLM.register(LLMAdapterConfig, LLMAdapter_HF)
    except ValueError:
        pass
