"""Task wrappers (lm_engine/model_wrapper/__init__.py:23-69)."""

from __future__ import annotations

from ..arguments import DistillationArgs, TrainingArgs
from ..containers import ModelContainer
from ..enums import TuningMethod
from ..parallel.manager import ProcessGroupManager
from .base import ModelWrapper
from .pretraining import ModelWrapperForPretraining

_WRAPPERS = {TuningMethod.pretraining: "pretraining.ModelWrapperForPretraining",
             TuningMethod.full_finetuning: "finetuning.ModelWrapperForFinetuning",
             TuningMethod.distillation: "distillation.ModelWrapperForDistillation"}


def _wrapper_class(method: TuningMethod):
    import importlib

    mod, cls = _WRAPPERS[method].split(".")
    return getattr(importlib.import_module(f"{__name__}.{mod}"), cls)


def get_model_container(args: TrainingArgs | DistillationArgs, efficient_initialization: bool | None = None,
                        keep_in_fp32: bool = True) -> ModelContainer:
    method = args.tuning_args.tuning_method
    if method not in _WRAPPERS:
        raise ValueError(f"unexpected tuning_method ({method})")
    d = args.distributed_args
    if d.num_pipeline_stages > 1:
        assert method == TuningMethod.pretraining, "pipeline parallel is only supported for pretraining"
    kwargs = dict(
        model_name=args.model_args.model_name, pretrained_config=args.model_args.pretrained_config,
        dtype=args.mixed_precision_args.dtype,
        efficient_initialization=(args.model_args.efficient_initialization if efficient_initialization is None
                                  else efficient_initialization),
        use_padding_free_transformer=args.model_args.use_padding_free_transformer,
        sequence_parallel=d.sequence_parallel, num_pipeline_stages=d.num_pipeline_stages,
        trust_remote_code=args.model_args.trust_remote_code, tokenizer_name=args.tokenizer_args.tokenizer_name,
        additional_special_tokens=args.tokenizer_args.additional_special_tokens, keep_in_fp32=keep_in_fp32)
    if method == TuningMethod.pretraining:
        seq = args.datasets[0].class_args.get("sequence_length")
        kwargs.update(micro_batch_size=args.training_parameters.micro_batch_size, sequence_length=seq,
                      reset_attention_mask=args.model_args.reset_attention_mask,
                      reset_position_ids=args.model_args.reset_position_ids)
    if method == TuningMethod.distillation:
        t = args.teacher_args
        kwargs.update(teacher_model_name=t.model_name, teacher_pretrained_config=t.pretrained_config,
                      teacher_model_dtype=t.dtype, kl_divergence_method=t.kl_divergence_method,
                      kl_divergence_weight=t.kl_divergence_weight,
                      micro_batch_size=args.training_parameters.micro_batch_size,
                      sequence_length=args.datasets[0].class_args.get("sequence_length"))
    cls = _wrapper_class(method)
    pp_rank = ProcessGroupManager.get_pipeline_parallel_rank()
    stage_ids = ProcessGroupManager.topology().pipeline_stage_ids(pp_rank, d.num_pipeline_stages)
    return ModelContainer([cls(**kwargs, pipeline_stage_id=i) for i in stage_ids])
