"""The YAML schema: ``TrainingArgs`` / ``DistillationArgs`` / ``UnshardingArgs`` and their sections.

Field names, defaults and cross-field rules follow the reference so that its config files load unchanged
(lm_engine/arguments/__init__.py:30-516).  Additions of this engine are marked "extension".
"""

from __future__ import annotations

from argparse import ArgumentParser
from typing import Any

from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ..enums import (
    ContextParallelLoadBalancerMethod,
    ExperimentsTrackerName,
    GradientCheckpointingMethod,
    Kernel,
    KLDivergenceMethod,
    LossMask,
    LRDecaySchedule,
    ParamsGroupMethod,
    TuningMethod,
)
from ..utils import divide_if_divisible, load_yaml, normalize_dtype_string
from .base import BaseArgs


def _require(**named: Any) -> None:
    for name, value in named.items():
        if value is None:
            raise AssertionError(f"{name} cannot be None")


class RandomArgs(BaseArgs):
    seed: int = 42


class TokenizerArgs(BaseArgs):
    tokenizer_name: str | None = None
    additional_special_tokens: list[str] | None = None


class ModelArgs(BaseArgs):
    model_name: str | None = None
    pretrained_config: dict | None = None
    trust_remote_code: bool = False
    use_padding_free_transformer: bool = False
    efficient_initialization: bool = False
    reset_attention_mask: bool = False
    reset_position_ids: bool = False

    def model_post_init(self, _ctx: Any) -> None:
        if self.model_name is None:
            _require(pretrained_config=self.pretrained_config)
        else:
            assert not self.efficient_initialization, "efficient_initialization is not supported with HF models"
            assert self.pretrained_config is None, "pretrained_config shouldn't be specified with model_name"


class TuningArgs(BaseArgs):
    tuning_method: TuningMethod | None = None

    def model_post_init(self, _ctx: Any) -> None:
        _require(tuning_method=self.tuning_method)


class TrainingParameters(BaseArgs):
    ignore_sampling_proportion_for_validation: bool = False
    num_training_steps: int | None = None
    micro_batch_size: int | None = None
    gradient_accumulation_steps: int | None = None
    global_batch_size: int | None = None
    eval_interval: int | None = None
    eval_during_training: bool = True
    loss_mask: LossMask = LossMask.output_only
    gradient_clipping: float | None = 1

    def model_post_init(self, _ctx: Any) -> None:
        _require(num_training_steps=self.num_training_steps)
        if self.eval_during_training:
            _require(eval_interval=self.eval_interval)
        given = [self.micro_batch_size, self.gradient_accumulation_steps, self.global_batch_size]
        if sum(v is not None for v in given) < 2:
            raise AssertionError(
                "two of micro_batch_size / gradient_accumulation_steps / global_batch_size cannot be None")

    def reset_training_parameters(self, data_loading_world_size: int) -> None:
        """Derives whichever of (micro batch, accumulation steps, global batch) is missing."""
        w = data_loading_world_size
        if self.micro_batch_size is None:
            self.micro_batch_size = divide_if_divisible(self.global_batch_size, self.gradient_accumulation_steps * w)
        elif self.gradient_accumulation_steps is None:
            self.gradient_accumulation_steps = divide_if_divisible(self.global_batch_size, self.micro_batch_size * w)
        elif self.global_batch_size is None:
            self.global_batch_size = self.micro_batch_size * self.gradient_accumulation_steps * w
        else:
            assert self.global_batch_size == self.micro_batch_size * self.gradient_accumulation_steps * w


class SaveArgs(BaseArgs):
    save_path: str | None = None
    save_interval: int | None = None
    save_optimizer: bool = True
    async_checkpointing: bool = False

    def model_post_init(self, _ctx: Any) -> None:
        _require(save_path=self.save_path, save_interval=self.save_interval)


class LoadArgs(BaseArgs):
    load_path: str | None = None
    iteration: int | None = None
    load_optimizer: bool = True
    load_lr_scheduler: bool = True
    load_rng_state: bool = True
    load_dataloader_state: bool = True
    load_experiments_tracker_state: bool = True
    load_starting_iteration: bool = True
    resume_learning_rate: bool = True

    def model_post_init(self, _ctx: Any) -> None:
        _require(load_path=self.load_path)
        if not self.load_optimizer:
            assert not self.load_lr_scheduler, "lr_scheduler loading doesn't make sense if you aren't loading optimizer"
        if self.load_lr_scheduler:
            assert self.resume_learning_rate, "resume learning rate needs to be True when reloading LR scheduler"


class DatasetArgs(BaseArgs):
    class_name: str | None = None
    class_args: dict = {}
    data_name: str | None = None
    input_format: str = INPUT_FORMAT
    output_format: str = OUTPUT_FORMAT
    data_sampling_ratio: int | None = None
    max_input_tokens: int | None = None
    max_output_tokens: int | None = None

    def model_post_init(self, _ctx: Any) -> None:
        _require(**{"dataset class_name": self.class_name, "data_name": self.data_name})
        if self.data_sampling_ratio is not None:
            assert self.data_sampling_ratio > 0, "data_sampling_ratio should be a positive integer"


class OptimizerArgs(BaseArgs):
    class_name: str = "TorchAdamW"
    params_group_method: ParamsGroupMethod | None = None
    use_optimizer_with_backward_hook: bool = False
    class_args: dict = {"lr": 1e-5, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10}

    def model_post_init(self, _ctx: Any) -> None:
        _require(**{"optimizer class_name": self.class_name})


class LRSchedulerArgs(BaseArgs):
    num_warmup_steps: int = 200
    num_constant_steps: int = 0
    num_decay_steps: int | None = None
    lr_decay_style: LRDecaySchedule = LRDecaySchedule.cosine
    lr_decay_factor: float = 0.1
    extra_lr_scheduler_args: dict = {}


class MixedPrecisionArgs(BaseArgs):
    dtype: str = "fp32"
    scaling_type_input: str = "dynamic"
    scaling_type_weight: str = "dynamic"
    scaling_type_grad_output: str = "dynamic"

    def model_post_init(self, _ctx: Any) -> None:
        self.dtype = normalize_dtype_string(self.dtype)


class ZeroTopologyArgs(BaseArgs):
    data_parallel_replication_world_size: int | None = None
    data_parallel_sharding_world_size: int | None = None

    def model_post_init(self, _ctx: Any) -> None:
        a, b = self.data_parallel_replication_world_size, self.data_parallel_sharding_world_size
        assert (a is None) == (b is None), (
            "data_parallel_replication_world_size and data_parallel_sharding_world_size need to be specified together")


class DistributedArgs(BaseArgs):
    stage: int = 3
    cpu_offload: bool = False
    gradient_checkpointing_method: GradientCheckpointingMethod | None = None
    gradient_checkpointing_args: dict = {}
    zero_topology: ZeroTopologyArgs = ZeroTopologyArgs()
    communication_dtype: str | None = None
    torch_compile: bool = False
    tensor_parallel_world_size: int = 1
    sequence_parallel: bool = False
    pipeline_parallel_world_size: int = 1
    context_parallel_world_size: int = 1
    context_parallel_load_balancing_method: ContextParallelLoadBalancerMethod | None = None
    timeout_minutes: int | None = None
    fsdp_algorithm: int | None = 2
    sync_every_gradient_accumulation_step: bool = False
    num_pipeline_stages: int = 1
    pipeline_parallel_schedule: str | None = None
    use_async_tensor_parallel: bool = False
    # extension: expert-parallel world size for MoE layers (experts sharded, tokens exchanged by all-to-all)
    expert_parallel_world_size: int = 1
    # extension: "ring" (K/V blocks around the cp ring), "ulysses" (all-to-all head exchange) or "auto" (ulysses
    # whenever the head counts divide over the cp group, else ring)
    context_parallel_attention: str = "auto"

    def model_post_init(self, _ctx: Any) -> None:
        if self.communication_dtype is not None:
            self.communication_dtype = normalize_dtype_string(self.communication_dtype)
        if self.sequence_parallel:
            assert self.tensor_parallel_world_size > 1, "tensor parallel needs to be enabled for sequence parallel"
        if self.tensor_parallel_world_size > 1:
            assert self.fsdp_algorithm in (2, 3), "FSDP-2/3 is required for using tensor parallel"
        if self.use_async_tensor_parallel:
            assert self.sequence_parallel, "sequence parallel should be enabled for using async-TP"
        assert self.num_pipeline_stages % self.pipeline_parallel_world_size == 0, (
            "num_pipeline_stages should be a multiple of pipeline_parallel_world_size")
        if self.num_pipeline_stages > 1:
            _require(pipeline_parallel_schedule=self.pipeline_parallel_schedule)


class AimArgs(BaseArgs):
    repo: str | None = None
    experiment: str | None = None

    def model_post_init(self, _ctx: Any) -> None:
        _require(repo=self.repo, experiment=self.experiment)


class WandBArgs(BaseArgs):
    project: str | None = None
    name: str | None = None
    entity: str | None = None
    tags: list[str] | None = None
    group: str | None = None
    notes: str | None = None

    def model_post_init(self, _ctx: Any) -> None:
        _require(project=self.project)


class LoggingArgs(BaseArgs):
    logging_level: str = "INFO"
    log_interval: int = 10
    aim_args: AimArgs | None = None
    wandb_args: WandBArgs | None = None
    experiments_tracker_name: ExperimentsTrackerName | None = None
    use_colored_logs: bool = False
    torch_profiler_trace_path: str | None = None
    cost_per_accelerator_per_hour: float | None = None

    def model_post_init(self, _ctx: Any) -> None:
        if self.experiments_tracker_name == ExperimentsTrackerName.aim:
            _require(aim_args=self.aim_args)
        elif self.experiments_tracker_name == ExperimentsTrackerName.wandb:
            _require(wandb_args=self.wandb_args)


class KernelArgs(BaseArgs):
    kernels: list[Kernel] = []

    def model_post_init(self, _ctx: Any) -> None:
        Kernel.validate_enabled(self.kernels)


class TeacherArgs(BaseArgs):
    model_name: str | None = None
    # extension: build the teacher from an inline config (offline runs / tests)
    pretrained_config: dict | None = None
    dtype: str = "fp32"
    kl_divergence_method: KLDivergenceMethod | None = None
    kl_divergence_weight: float = 1

    def model_post_init(self, _ctx: Any) -> None:
        self.dtype = normalize_dtype_string(self.dtype)
        _require(kl_divergence_method=self.kl_divergence_method)


class TrainingArgs(BaseArgs):
    random_args: RandomArgs = RandomArgs()
    tokenizer_args: TokenizerArgs = TokenizerArgs()
    model_args: ModelArgs | None = None
    tuning_args: TuningArgs | None = None
    optimizer_args: OptimizerArgs = OptimizerArgs()
    lr_scheduler_args: LRSchedulerArgs = LRSchedulerArgs()
    datasets: list[DatasetArgs] = []
    save_args: SaveArgs | None = None
    load_args: LoadArgs | None = None
    training_parameters: TrainingParameters | None = None
    logging_args: LoggingArgs = LoggingArgs()
    mixed_precision_args: MixedPrecisionArgs = MixedPrecisionArgs()
    distributed_args: DistributedArgs = DistributedArgs()
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, _ctx: Any) -> None:
        _require(model_args=self.model_args, tuning_args=self.tuning_args, save_args=self.save_args,
                 datasets=self.datasets)
        assert len(self.datasets) != 0, "datasets cannot be an empty list"
        names = [d.data_name for d in self.datasets]
        assert len(names) == len(set(names)), "data_name should be unique for each dataset"
        if self.distributed_args.num_pipeline_stages > 1 and self.training_parameters.eval_during_training:
            raise NotImplementedError("evaluation is not supported with pipeline parallel")
        if self.optimizer_args.use_optimizer_with_backward_hook:
            assert self.training_parameters.gradient_accumulation_steps == 1
            assert self.training_parameters.gradient_clipping is None


class UnshardingArgs(BaseArgs):
    load_args: LoadArgs | None = None
    unsharded_path: str | None = None
    mixed_precision_args: MixedPrecisionArgs = MixedPrecisionArgs()
    logging_args: LoggingArgs = LoggingArgs()
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, _ctx: Any) -> None:
        _require(load_args=self.load_args, unsharded_path=self.unsharded_path)


class DistillationArgs(TrainingArgs):
    teacher_args: TeacherArgs | None = None
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, _ctx: Any) -> None:
        _require(teacher_args=self.teacher_args)
        super().model_post_init(_ctx)


def args_from_yaml(path: str, args_class: type[BaseArgs]) -> BaseArgs:
    return args_class(**load_yaml(path))


def get_args(args_class: type[BaseArgs]) -> BaseArgs:
    """``--config path.yml`` -> validated args; also configures the root logger."""
    from ..logging_utils import set_logger

    parser = ArgumentParser()
    parser.add_argument("--config", type=str, required=True, help="path for the config")
    ns = parser.parse_args()
    args = args_from_yaml(ns.config, args_class)
    set_logger(args.logging_args.logging_level, colored_log=args.logging_args.use_colored_logs)
    return args
