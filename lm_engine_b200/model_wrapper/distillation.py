"""Distillation wrapper: the student trains on ``lm_loss + kl_divergence_weight * KL`` against a frozen teacher that
sees the same tokens (lm_engine/model_wrapper/distillation.py:24-212).

``kl_divergence_method``: ``forward`` = sum student * ln(student / teacher); ``backward`` = sum teacher *
ln(teacher / student); both averaged over tokens ("batchmean").  The student is sharded by the engine like any other
model; the teacher is a replicated, gradient-free copy in ``teacher_model_dtype`` placed on the device when the
student is wrapped (B200 keeps an 8B teacher in 16 GB of its 180 GB).  Tensor / pipeline parallel distillation is not
supported, as in the reference.
"""

from __future__ import annotations

import logging
import os

import torch
import torch.nn.functional as F

from ..enums import KLDivergenceMethod
from ..logging_utils import log_rank_0
from ..loss import get_autoregressive_language_modeling_loss
from ..models import CommonConfig, build_model, config_from_dict
from ..parallel.manager import ProcessGroupManager
from ..utils import string_to_torch_dtype
from .pretraining import ModelWrapperForPretraining


class ModelWrapperForDistillation(ModelWrapperForPretraining):
    def __init__(self, *args, teacher_model_name: str | None = None, teacher_pretrained_config: dict | None = None,
                 teacher_model_dtype: torch.dtype | str = torch.bfloat16,
                 kl_divergence_method: KLDivergenceMethod = KLDivergenceMethod.forward,
                 kl_divergence_weight: float = 1, **kwargs) -> None:
        self.teacher_model_name = teacher_model_name
        self.teacher_pretrained_config = teacher_pretrained_config
        self.teacher_model_dtype = (string_to_torch_dtype(teacher_model_dtype)
                                    if isinstance(teacher_model_dtype, str) else teacher_model_dtype)
        self.kl_divergence_method = KLDivergenceMethod(kl_divergence_method)
        self.kl_divergence_weight = kl_divergence_weight
        super().__init__(*args, **kwargs)
        if ProcessGroupManager.is_tensor_parallel_enabled() or self.num_pipeline_stages > 1:
            raise NotImplementedError("distillation supports data parallel sharding only")

    def _setup_config(self, pretrained_config: dict | None) -> None:
        super()._setup_config(pretrained_config)
        if self.teacher_pretrained_config is not None:
            self.teacher_config = config_from_dict(self.teacher_pretrained_config)
        else:
            assert self.teacher_model_name is not None and os.path.isdir(self.teacher_model_name), (
                "teacher model_name must be a local directory with config.json and safetensors")
            self.teacher_config = CommonConfig.from_pretrained(self.teacher_model_name)
        assert self.teacher_config.vocab_size == self.config.vocab_size, "teacher and student must share a vocabulary"

    def _setup_tokenizer(self, additional_special_tokens) -> None:
        super()._setup_tokenizer(additional_special_tokens)
        log_rank_0(logging.WARNING, "teacher and student are assumed to share one tokenizer; this is not checked")

    def _setup_model(self) -> None:
        super()._setup_model()
        kw = dict(use_padding_free_transformer=self.use_padding_free_transformer)
        teacher = build_model(self.teacher_config, **kw)
        if self.teacher_model_name is not None and self.teacher_pretrained_config is None:
            from ..utils import SafeTensorsWeightsManager

            teacher.load_from_safetensors_weights_manager(SafeTensorsWeightsManager(self.teacher_model_name))
        teacher = teacher.to(self.teacher_model_dtype).eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        # not a registered sub-module: the sharding runtime, the optimizer and checkpoints must not see the teacher
        object.__setattr__(self, "teacher_model", teacher)

    def place_teacher(self, device: torch.device) -> None:
        self.teacher_model.to(device)

    def forward(self, batch: dict | torch.Tensor, aux_loss_from_pipeline_parallel: torch.Tensor | float = 0,
                lm_loss_multiplier: float = 1) -> dict:
        if isinstance(batch, torch.Tensor):
            batch = {"text": batch}
        inputs, labels = self._prepare_model_inputs(batch)
        student_logits = self.model(**inputs).logits
        lm_loss = get_autoregressive_language_modeling_loss(
            lm_logits=student_logits, labels=labels, cu_seqlens=None,
            use_padding_free_transformer=self.use_padding_free_transformer, reduction="sum",
            shift_logits_and_labels=False, tensor_parallel_enabled=False) * lm_loss_multiplier
        with torch.no_grad():
            teacher_logits = self.teacher_model(**inputs).logits.float()
        V = teacher_logits.size(-1)
        t_lsm = F.log_softmax(teacher_logits, dim=-1).view(-1, V)
        s_lsm = F.log_softmax(student_logits.float(), dim=-1).view(-1, V)
        if self.kl_divergence_method == KLDivergenceMethod.forward:
            kl = F.kl_div(t_lsm, s_lsm, reduction="batchmean", log_target=True)
        else:
            kl = F.kl_div(s_lsm, t_lsm, reduction="batchmean", log_target=True)
        return {"loss": lm_loss + self.kl_divergence_weight * kl, "lm_loss": lm_loss, "kl_divergence": kl}

    def has_teacher_model(self) -> bool:
        return True

    def train(self, mode: bool = True):
        super().train(mode)
        self.teacher_model.eval()
        return self
