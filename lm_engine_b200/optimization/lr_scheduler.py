"""Learning-rate schedules: linear warm-up, optional constant phase, then cosine / linear / exponential / power /
constant decay down to ``lr_decay_factor`` (lm_engine/optimization/lr_scheduler/*.py).

``LRScheduler`` mirrors ``torch.optim.lr_scheduler.LambdaLR`` semantics: construction performs the step-0 update, so
the first optimizer step of a run with warm-up uses lr x 0, and ``step()`` is called after each optimizer step.
"""

from __future__ import annotations

import math

from ..enums import LRDecaySchedule


def lr_factor(step: int, *, style: LRDecaySchedule, num_warmup_steps: int, num_constant_steps: int,
              num_decay_steps: int | None, num_training_steps: int, lr_decay_factor: float, base_lr: float = 1.0,
              a: float | None = None, b: float | None = None, c: float | None = None) -> float:
    warm = num_warmup_steps
    const_end = warm + num_constant_steps
    decay_end = num_training_steps if num_decay_steps is None else const_end + num_decay_steps
    f = lr_decay_factor
    if style == LRDecaySchedule.power:
        assert num_constant_steps == 0, "num_constant_steps should be 0 for power law scheduler"
        peak = min(1.0, (a / base_lr) * (warm * c) ** b) if warm > 0 else 1.0
        if warm > 0 and step <= warm:
            return peak / warm * step
        return min(1.0, (a / base_lr) * (step * c) ** b)
    if warm > 0 and step <= warm:
        return step / warm
    if style == LRDecaySchedule.constant:
        assert num_decay_steps in (0, None) or True
        return 1.0
    if step <= const_end:
        return 1.0
    t, x = decay_end - const_end, step - const_end
    if style == LRDecaySchedule.exponential:
        e = math.e
        return (1 - f) * e / (e - 1) * math.exp(-x / t) + (f * e - 1) / (e - 1)
    if step <= decay_end:
        if style == LRDecaySchedule.cosine:
            return (1 - f) * (1 + math.cos(math.pi * x / t)) / 2 + f
        if style == LRDecaySchedule.linear:
            return (f - 1) / t * x + 1
        raise ValueError(f"invalid lr_decay_style ({style})")
    return f


class LRScheduler:
    def __init__(self, optimizer, *, style: LRDecaySchedule, num_warmup_steps: int, num_constant_steps: int,
                 num_decay_steps: int | None, num_training_steps: int, lr_decay_factor: float,
                 last_epoch: int = -1, **extra) -> None:
        if style == LRDecaySchedule.constant:
            assert not num_decay_steps, "num_decay_steps should be 0 for constant schedule"
        self.optimizer = optimizer
        self.base_lrs = [g.setdefault("initial_lr", g["lr"]) for g in optimizer.param_groups]
        self.kw = dict(style=style, num_warmup_steps=num_warmup_steps, num_constant_steps=num_constant_steps,
                       num_decay_steps=num_decay_steps, num_training_steps=num_training_steps,
                       lr_decay_factor=lr_decay_factor, **extra)
        self.last_epoch = last_epoch
        self.step()

    def factor(self, step: int) -> float:
        return lr_factor(step, base_lr=self.base_lrs[0], **self.kw)

    def step(self) -> None:
        self.last_epoch += 1
        f = self.factor(self.last_epoch)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * f

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch, "base_lrs": self.base_lrs}

    def load_state_dict(self, sd: dict) -> None:
        self.last_epoch = sd["last_epoch"]
        self.base_lrs = list(sd["base_lrs"])
        f = self.factor(self.last_epoch)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * f
