"""Training entry point: ``python -m lm_engine_b200.train --config cfg.yml`` (role of lm_engine/train.py:49-794).

The step functions are importable on their own (the benchmark drives them directly):

* :func:`train_step_without_pipeline_parallel` - gradient accumulation over micro-batches, device-side global-norm
  clipping, fused sharded AdamW, LR schedule, metric reduction over data-parallel ranks;
* :func:`train_step_with_pipeline_parallel` - the same through the 1F1B pipeline schedule.

Loss scaling follows the reference: each micro-batch contributes ``sum(CE) / (micro_batch x local_sequence)`` and the
accumulated loss is divided by the number of accumulation steps before backward.
"""

from __future__ import annotations

import logging
import os
import time
from contextlib import nullcontext

import torch

from .accelerator import Accelerator
from .arguments import DistillationArgs, TrainingArgs, get_args
from .containers import LRSchedulerContainer, ModelContainer, OptimizerContainer
from .enums import TuningMethod
from .kernels import enable_kernels
from .logging_utils import ExperimentsTracker, MetricsTrackingDict, StepProfiler, log_environment, log_rank_0
from .logging_utils.profiler import DeviceTimer
from .parallel.manager import ProcessGroupManager
from .train_utils import (all_reduce_metrics_tracker, check_device_status, get_model_tflops, mfu,
                          track_metrics)
from .utils import disable_generation_cache, setup_tf32


def get_next_batch(dataloader) -> dict | None:
    if dataloader is None:
        return None
    return next(dataloader)


def train_step_without_pipeline_parallel(
    model_container: ModelContainer,
    optimizer_container: OptimizerContainer,
    lr_scheduler_container: LRSchedulerContainer,
    train_dataloader,
    gradient_accumulation_steps: int,
    gradient_clipping: float | None,
    forward_context=nullcontext,
    backward_context=nullcontext,
    sync_every_gradient_accumulation_step: bool = False,
    lm_loss_multiplier: float | None = None,
    tuning_method: TuningMethod = TuningMethod.pretraining,
    reduce_metrics: bool = True,
) -> MetricsTrackingDict:
    assert len(model_container) == 1
    model = model_container[0]
    optimizer = optimizer_container[0]
    optimizer.max_grad_norm = gradient_clipping
    optimizer.zero_grad()
    metrics = MetricsTrackingDict({})
    ga = gradient_accumulation_steps
    batches = [get_next_batch(train_dataloader) for _ in range(ga)]
    if lm_loss_multiplier is None:
        if tuning_method == TuningMethod.full_finetuning:
            # finetuning normalises by the number of target tokens in the whole accumulated batch
            n = sum(int((b["labels"][..., 1:] != -100).sum()) for b in batches if b is not None)
            lm_loss_multiplier = ga / max(n, 1)
        else:
            cp = ProcessGroupManager.get_context_parallel_world_size()
            lm_loss_multiplier = 1 / (model.micro_batch_size * model.sequence_length / cp)
    for batch in batches:
        with forward_context():
            loss_dict = model(batch, lm_loss_multiplier=lm_loss_multiplier)
        with backward_context():
            (loss_dict["loss"] / ga).backward()
        with torch.no_grad():
            metrics = metrics + {k: v.detach() if isinstance(v, torch.Tensor) else v for k, v in loss_dict.items()}
    grad_norm = optimizer.step()
    lr_scheduler_container.step()
    with torch.no_grad():
        metrics = metrics / ga
        metrics["grad_norm"] = grad_norm.reshape(()) if gradient_clipping is not None else 0.0
        if reduce_metrics:
            metrics = all_reduce_metrics_tracker(metrics)
    return metrics


def train_step_with_pipeline_parallel(model_container, pipeline_schedule, optimizer_container,
                                      lr_scheduler_container, train_dataloader, gradient_accumulation_steps: int,
                                      gradient_clipping: float | None, micro_batch_size: int,
                                      sequence_length: int) -> MetricsTrackingDict:
    from .parallel.pipeline_parallel import pipeline_train_step

    return pipeline_train_step(model_container, pipeline_schedule, optimizer_container, lr_scheduler_container,
                               train_dataloader, gradient_accumulation_steps, gradient_clipping, micro_batch_size,
                               sequence_length)


@torch.no_grad()
def evaluate(val_dataloaders, model_container: ModelContainer, global_step: int, experiments_tracker,
             eval_steps: int, group_names: list[str], lm_loss_multiplier: float | None = None) -> None:
    """Average loss over ``eval_steps`` batches of every validation group."""
    if not val_dataloaders:
        return
    model = model_container[0]
    model_container.eval()
    for name, loader in zip(group_names, val_dataloaders):
        metrics = MetricsTrackingDict({})
        n = 0
        for _ in range(eval_steps):
            try:
                batch = get_next_batch(loader)
            except StopIteration:
                break
            mult = lm_loss_multiplier
            if mult is None and hasattr(model, "micro_batch_size"):
                cp = ProcessGroupManager.get_context_parallel_world_size()
                mult = 1 / (model.micro_batch_size * model.sequence_length / cp)
            out = model(batch, lm_loss_multiplier=mult if mult is not None else 1)
            metrics = metrics + {k: v.detach() if isinstance(v, torch.Tensor) else v for k, v in out.items()}
            n += 1
        if n:
            metrics = all_reduce_metrics_tracker(metrics / n)
            track_metrics(global_step, experiments_tracker, metrics, context=f"val-{name}" if name else "val")
    model_container.train()


def train(args: TrainingArgs, model_container: ModelContainer, pipeline_schedule, optimizer_container,
          lr_scheduler_container, train_dataloader, val_dataloaders, test_dataloaders, experiments_tracker,
          starting_iteration: int = 0, val_group_names: list[str] | None = None) -> None:
    from .checkpointing import ensure_last_checkpoint_is_saved, save_checkpoint

    tp = args.training_parameters
    d = args.distributed_args
    ga = tp.gradient_accumulation_steps
    mbs = tp.micro_batch_size
    seq = args.datasets[0].class_args.get("sequence_length")
    log_interval = args.logging_args.log_interval
    world = ProcessGroupManager.get_world_size()
    tokens_per_step = tp.global_batch_size * (seq or 0)
    tflops_per_step = 0.0
    if seq is not None:
        tflops_per_step = get_model_tflops(model_container[0].config, tp.global_batch_size, seq,
                                           d.gradient_checkpointing_method, d.gradient_checkpointing_args)
    consumed = starting_iteration * tp.global_batch_size
    cost_rate = args.logging_args.cost_per_accelerator_per_hour
    cumulative_cost = 0.0
    model_container.train()
    timer = DeviceTimer()
    host_t0 = time.perf_counter()
    timer.start()
    window = MetricsTrackingDict({})
    step = starting_iteration
    # metrics of every logged step also go to <save_path>/../metrics.jsonl (the sweep tool reads it)
    from .train_utils import set_metrics_file

    set_metrics_file(os.path.join(os.path.dirname(os.path.abspath(args.save_args.save_path)), "metrics.jsonl"))
    # host-side failure detection: per-rank heartbeat file + watchdog thread (LME_STALL_SECONDS, LME_STALL_ABORT=1
    # ends a rank that made no progress so that the launcher can restart from the last checkpoint)
    from .utils.watchdog import Heartbeat

    from .utils.watchdog import abort_is_safe

    want_abort = os.environ.get("LME_STALL_ABORT", "0") == "1"
    if want_abort and not abort_is_safe():
        log_rank_0(logging.WARNING, "LME_STALL_ABORT=1 ignored: ending a rank whose memory is bound to an NVLink "
                   "multicast object faults its peers; set NCCL_NVLS_ENABLE=0 (and no LME_REDUCE_SCATTER=nvls), "
                   "or stop the job through the KILLSWITCH file")
        want_abort = False
    heartbeat = Heartbeat(os.environ.get("LME_HEARTBEAT_DIR", os.path.join(args.save_args.save_path, "heartbeats")),
                          ProcessGroupManager.get_global_rank(), ProcessGroupManager.get_world_size(),
                          stall_seconds=float(os.environ.get("LME_STALL_SECONDS", "1800")), poll_seconds=30.0,
                          abort=want_abort).start()
    device_status = None
    with StepProfiler(args.logging_args.torch_profiler_trace_path) as prof:
        while step < tp.num_training_steps:
            step += 1
            heartbeat.beat(step, device_status)
            if pipeline_schedule is not None:
                m = train_step_with_pipeline_parallel(model_container, pipeline_schedule, optimizer_container,
                                                      lr_scheduler_container, train_dataloader, ga,
                                                      tp.gradient_clipping, mbs, seq)
            else:
                m = train_step_without_pipeline_parallel(
                    model_container, optimizer_container, lr_scheduler_container, train_dataloader, ga,
                    tp.gradient_clipping,
                    sync_every_gradient_accumulation_step=d.sync_every_gradient_accumulation_step,
                    tuning_method=args.tuning_args.tuning_method)
            # the metric reduction above read values back, so the device is idle: one look at the status block tells
            # whether any bounded wait of the step (peer flags of the fused collectives, mbarriers) ran out
            device_status = check_device_status(step)
            window = window + m
            consumed += tp.global_batch_size
            prof.step()
            if step % log_interval == 0:
                timer.stop()
                dt = timer.elapsed_s() / log_interval          # device-timed
                host_dt = (time.perf_counter() - host_t0) / log_interval
                extra = {"learning_rate": lr_scheduler_container[0].get_last_lr()[0], "step_time (sec)": dt,
                         "host_step_time (sec)": host_dt}
                if tokens_per_step:
                    extra["tokens_per_sec_per_gpu"] = tokens_per_step / dt / world
                    extra["billion_tokens_per_day"] = tokens_per_step * 86400 / dt / 1e9
                if tflops_per_step:
                    extra["FLOPs"] = tflops_per_step / dt / world
                    extra["MFU"] = mfu(tflops_per_step, dt, world)
                if cost_rate is not None:
                    cumulative_cost += cost_rate * world * dt * log_interval / 3600
                    extra["cost (USD)"] = cumulative_cost
                avg = (window / log_interval).get_dict()
                track_metrics(step, experiments_tracker, {**avg, **extra}, context="train")
                window = MetricsTrackingDict({})
                host_t0 = time.perf_counter()
                timer.start()
            if tp.eval_during_training and tp.eval_interval and step % tp.eval_interval == 0:
                evaluate(val_dataloaders, model_container, step, experiments_tracker,
                         eval_steps=args.datasets[0].class_args.get("eval_steps", 1),
                         group_names=val_group_names or [""] * len(val_dataloaders or []))
            if step % args.save_args.save_interval == 0 or step == tp.num_training_steps:
                save_checkpoint(args, model_container, optimizer_container, lr_scheduler_container, train_dataloader,
                                experiments_tracker, step,
                                {"consumed_samples": consumed, "cumulative_cost_usd": cumulative_cost})
                host_t0 = time.perf_counter()
                timer.start()
    heartbeat.stop()
    ensure_last_checkpoint_is_saved()


def resumed_consumed_samples(args, metadata: dict | None) -> int:
    """Samples that the pretraining loaders skip on a resume: the checkpoint's count, or 0 when the checkpoint's
    data position is not wanted (``load_args.load_dataloader_state: false``; lm_engine/train.py:702-707)."""
    if metadata is None or args.load_args is None or not args.load_args.load_dataloader_state:
        return 0
    return int(metadata.get("consumed_samples", 0))


def main(args_class: type[TrainingArgs | DistillationArgs] = TrainingArgs) -> None:
    from .checkpointing import load_checkpoint_for_training
    from .data import get_finetuning_dataloader, get_pretraining_dataloaders
    from .distributed import wrap_model_container_for_distributed_training
    from .model_wrapper import get_model_container
    from .optimization import get_optimizer_container, get_scheduler_container

    setup_tf32()
    args = get_args(args_class)
    d = args.distributed_args
    if args_class is DistillationArgs:
        assert d.fsdp_algorithm in (2, 3), "distillation needs the sharded runtime (fsdp_algorithm 2 or 3)"
    ProcessGroupManager(
        tensor_parallel_world_size=d.tensor_parallel_world_size,
        pipeline_parallel_world_size=d.pipeline_parallel_world_size,
        data_parallel_replication_world_size=d.zero_topology.data_parallel_replication_world_size,
        data_parallel_sharding_world_size=d.zero_topology.data_parallel_sharding_world_size,
        context_parallel_world_size=d.context_parallel_world_size,
        context_parallel_load_balancing_method=d.context_parallel_load_balancing_method,
        zero_stage=d.stage, timeout_minutes=d.timeout_minutes,
        use_async_tensor_parallel=d.use_async_tensor_parallel,
        expert_parallel_world_size=d.expert_parallel_world_size,
        context_parallel_attention=d.context_parallel_attention)
    args.training_parameters.reset_training_parameters(ProcessGroupManager.get_data_loading_world_size())
    Accelerator.set_seed(args.random_args.seed)
    model_container = get_model_container(args, efficient_initialization=None, keep_in_fp32=True)
    model_container, pipeline_schedule = wrap_model_container_for_distributed_training(args, model_container)
    optimizer_container = get_optimizer_container(
        args.optimizer_args.class_name, args.optimizer_args.class_args, model_container,
        args.optimizer_args.params_group_method, args.optimizer_args.use_optimizer_with_backward_hook,
        max_grad_norm=args.training_parameters.gradient_clipping)
    ls = args.lr_scheduler_args
    lr_scheduler_container = get_scheduler_container(
        model_container, optimizer_container, ls.num_warmup_steps, ls.num_constant_steps, ls.num_decay_steps,
        args.training_parameters.num_training_steps, ls.lr_decay_style, ls.lr_decay_factor,
        ls.extra_lr_scheduler_args)
    starting_iteration, metadata, tracker_state = 0, None, None
    finetuning = args.tuning_args.tuning_method == TuningMethod.full_finetuning
    train_dl = None
    if finetuning:
        # built before the checkpoint is read, so that the saved sampler position is restored into it (the
        # reference does the same, lm_engine/train.py:719-728); the pretraining loaders are built afterwards from
        # the number of consumed samples instead
        train_dl = get_finetuning_dataloader(args, model_container[0].tokenizer, split="train")
    if args.load_args is not None:
        starting_iteration, metadata, tracker_state = load_checkpoint_for_training(
            args, args_class, model_container, optimizer_container, lr_scheduler_container, train_dl)
    consumed = resumed_consumed_samples(args, metadata)
    val_names: list[str] = []
    if finetuning:
        val_dls = [get_finetuning_dataloader(args, model_container[0].tokenizer, split="val")] \
            if args.training_parameters.eval_during_training else []
        test_dls = []
        val_names = [""]
    else:
        train_dl, val_dls, test_dls = get_pretraining_dataloaders(args, model_container[0].tokenizer, consumed)
        val_names = [""] * len(val_dls or [])
    tracker = ExperimentsTracker(args.logging_args.experiments_tracker_name, args.logging_args.aim_args,
                                 args.logging_args.wandb_args, checkpoint_metadata=tracker_state,
                                 is_tracking_rank=ProcessGroupManager.is_tracking_rank())
    tracker.log_args(args)
    log_rank_0(logging.INFO, str(ProcessGroupManager()) if False else "process groups ready")
    args.log_args()
    log_environment()
    log_rank_0(logging.INFO, str(model_container[0].model))
    with disable_generation_cache(), enable_kernels(args.kernel_args.kernels):
        train(args, model_container, pipeline_schedule, optimizer_container, lr_scheduler_container, train_dl, val_dls,
              test_dls, tracker, starting_iteration, val_names)
    tracker.finish()
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()
