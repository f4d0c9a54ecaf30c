"""Optimizers, parameter groups and learning-rate schedules."""

from ..containers import LRSchedulerContainer
from ..enums import LRDecaySchedule
from .lr_scheduler import LRScheduler, lr_factor
from .optimizer import ShardedOptimizer, get_optimizer_container
from .params_group import get_param_groups, get_param_groups_list


def get_scheduler_container(model_container, optimizer_container, num_warmup_steps: int, num_constant_steps: int,
                            num_decay_steps: int | None, num_training_steps: int, lr_decay_style: LRDecaySchedule,
                            lr_decay_factor: float, extra_lr_scheduler_args: dict,
                            use_optimizer_with_backward_hook: bool = False,
                            last_epoch: int = -1) -> LRSchedulerContainer:
    return LRSchedulerContainer([
        LRScheduler(opt, style=lr_decay_style, num_warmup_steps=num_warmup_steps,
                    num_constant_steps=num_constant_steps, num_decay_steps=num_decay_steps,
                    num_training_steps=num_training_steps, lr_decay_factor=lr_decay_factor, last_epoch=last_epoch,
                    **extra_lr_scheduler_args)
        for opt in optimizer_container])


def get_learning_rate(optimizer_container, lr_scheduler_container) -> float:
    return lr_scheduler_container[0].get_last_lr()[0]
