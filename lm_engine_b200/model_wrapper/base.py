"""Task-independent model wrapper: owns the config, the optional tokenizer and the raw model of one pipeline stage;
computes the training loss (lm_engine/model_wrapper/base.py:27-347).

``keep_in_fp32`` has no effect on the layout of this engine: master weights are always the fp32 shards of the
sharding runtime and the module parameters are compute-dtype views.
"""

from __future__ import annotations

import logging
import os

import torch
import torch.nn as nn

from ..kernels import is_fused_linear_cross_entropy_enabled
from ..logging_utils import log_rank_0
from ..loss import get_autoregressive_language_modeling_loss, is_aux_loss_zero
from ..models import CommonConfig, build_model, config_from_dict
from ..parallel.manager import ProcessGroupManager
from ..utils import string_to_torch_dtype


class ModelWrapper(nn.Module):
    def __init__(self, model_name: str | None = None, pretrained_config: dict | None = None,
                 dtype: torch.dtype | str = torch.float32, efficient_initialization: bool = False,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False,
                 num_pipeline_stages: int = 1, pipeline_stage_id: int = 0, trust_remote_code: bool = False,
                 tokenizer_name: str | None = None, additional_special_tokens: list[str] | None = None,
                 keep_in_fp32: bool = True) -> None:
        super().__init__()
        self.model_name = model_name
        self.dtype = string_to_torch_dtype(dtype) if isinstance(dtype, str) and dtype != "fp8" else dtype
        self.use_fp8 = dtype == "fp8"
        if self.use_fp8:
            self.dtype = torch.bfloat16
        self.efficient_initialization = efficient_initialization
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.num_pipeline_stages, self.pipeline_stage_id = num_pipeline_stages, pipeline_stage_id
        self.is_first_stage = pipeline_stage_id == 0
        self.is_last_stage = pipeline_stage_id == num_pipeline_stages - 1
        self.is_pipeline_parallel_enabled = num_pipeline_stages > 1
        self.tokenizer_name = tokenizer_name if tokenizer_name is not None else model_name
        self.engine = None  # set by wrap_model_container_for_distributed_training
        self._setup_config(pretrained_config)
        self._setup_tokenizer(additional_special_tokens)
        self._setup_model()
        self.router_aux_loss_coef = self.config.router_aux_loss_coef or 0

    # ------------------------------------------------------------------ construction
    def _setup_config(self, pretrained_config: dict | None) -> None:
        if pretrained_config is not None:
            self.config = config_from_dict(pretrained_config)
        else:
            assert self.model_name is not None and os.path.isdir(self.model_name), (
                "model_name must be a local directory with config.json and safetensors (there is no hub access)")
            self.config = CommonConfig.from_pretrained(self.model_name)
        self.is_custom_model = True
        self.tie_word_embeddings = self.config.tie_word_embeddings
        self.eos_token_id = self.config.eos_token_id

    def _setup_tokenizer(self, additional_special_tokens: list[str] | None) -> None:
        from ..tokenizers import get_tokenizer

        self.tokenizer = None
        if self.tokenizer_name is not None:
            try:
                self.tokenizer = get_tokenizer(self.tokenizer_name)
            except Exception as e:  # offline machine without the tokenizer files
                log_rank_0(logging.WARNING, f"tokenizer {self.tokenizer_name} unavailable ({e}); continuing without")
        if self.tokenizer is not None and additional_special_tokens:
            self.tokenizer.add_special_tokens({"additional_special_tokens": additional_special_tokens})

    def _model_kwargs(self) -> dict:
        return dict(use_padding_free_transformer=self.use_padding_free_transformer,
                    sequence_parallel=self.sequence_parallel, num_pipeline_stages=self.num_pipeline_stages,
                    pipeline_stage_id=self.pipeline_stage_id)

    def _setup_model(self) -> None:
        if self.efficient_initialization:
            with torch.device("meta"):
                self.model = build_model(self.config, **self._model_kwargs())
        else:
            self.model = build_model(self.config, **self._model_kwargs())
            if self.model_name is not None:
                from ..utils import SafeTensorsWeightsManager

                self.model.load_from_safetensors_weights_manager(SafeTensorsWeightsManager(self.model_name))
        n, active = self.calculate_num_parameters()
        log_rank_0(logging.INFO, f"num parameters in the model = {n:,} (active {active:,})")

    # ------------------------------------------------------------------ loss
    def get_loss(self, model_outputs, labels: torch.Tensor, shift_logits_and_labels: bool,
                 cu_seqlens: torch.Tensor | None = None, lm_loss_multiplier: float = 1) -> dict[str, torch.Tensor]:
        tp = ProcessGroupManager.is_tensor_parallel_enabled()
        fused = model_outputs.logits is None
        kw = dict(cu_seqlens=cu_seqlens, use_padding_free_transformer=self.use_padding_free_transformer,
                  reduction="sum", shift_logits_and_labels=shift_logits_and_labels)
        if fused:
            lm_loss = self.model.compute_lm_loss(model_outputs.last_hidden_state, labels, **kw)
        else:
            lm_loss = get_autoregressive_language_modeling_loss(
                lm_logits=model_outputs.logits, labels=labels, tensor_parallel_enabled=tp,
                vocab_size=self.config.vocab_size, **kw)
        lm_loss = lm_loss * lm_loss_multiplier
        aux = getattr(model_outputs, "aux_loss", 0)
        if is_aux_loss_zero(aux):
            return {"loss": lm_loss, "lm_loss": lm_loss}
        return {"loss": lm_loss + self.router_aux_loss_coef * aux, "lm_loss": lm_loss, "aux_loss": aux}

    def skip_logits(self) -> bool:
        return is_fused_linear_cross_entropy_enabled()

    # ------------------------------------------------------------------ misc
    def save_pretrained(self, save_path: str, state_dict: dict | None = None) -> None:
        from ..utils import SafeTensorsWeightsManager

        if state_dict is None:
            state_dict = self.engine.full_state_dict() if self.engine is not None else self.model.state_dict()
        state_dict = {(k[len("model."):] if k.startswith("model.") else k): v for k, v in state_dict.items()}
        SafeTensorsWeightsManager.save_state_dict(state_dict, save_path)
        self.config.save_pretrained(save_path)
        if self.tokenizer is not None and hasattr(self.tokenizer, "save_pretrained"):
            self.tokenizer.save_pretrained(save_path, legacy_format=False)

    def calculate_num_parameters(self) -> tuple[int, int]:
        """(total, active-per-token) parameter counts of the whole model (all pipeline stages, no TP split)."""
        with torch.device("meta"), ProcessGroupManager.set_dummy_tensor_parallel_world_size(1), \
                ProcessGroupManager.set_dummy_tensor_parallel_rank(0):
            full = build_model(self.config)
        total = sum(p.numel() for p in full.parameters())
        active = total
        for i, blk in enumerate(self.config.mlp_blocks):
            if blk.mlp_type == "MoE":
                mlp = full.transformer.h[str(i)].mlp_block
                per_expert = (mlp.c_fc.weight.numel() + mlp.c_proj.weight.numel()) // blk.num_experts
                active -= per_expert * (blk.num_experts - blk.num_experts_per_tok)
        return total, active

    def has_teacher_model(self) -> bool:
        return False

    def train(self, mode: bool = True):
        super().train(mode)
        return self
