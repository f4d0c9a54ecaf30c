"""List containers for per-pipeline-stage models / optimizers / schedulers (lm_engine/containers.py:10-60)."""

from __future__ import annotations


class _Container:
    def __init__(self, items: list) -> None:
        self.items = list(items)

    def __iter__(self):
        return iter(self.items)

    def __getitem__(self, i: int):
        return self.items[i]

    def __setitem__(self, i: int, v) -> None:
        self.items[i] = v

    def __len__(self) -> int:
        return len(self.items)

    def __repr__(self) -> str:
        return "\n".join(repr(i) for i in self.items)


class ModelContainer(_Container):
    def train(self) -> "ModelContainer":
        for m in self:
            m.train()
        return self

    def eval(self) -> "ModelContainer":
        for m in self:
            m.eval()
        return self


class LRSchedulerContainer(_Container):
    def step(self) -> None:
        for s in self:
            s.step()


class OptimizerContainer(LRSchedulerContainer):
    def zero_grad(self) -> None:
        for o in self:
            o.zero_grad()


class BackwardHookOptimizerContainer(OptimizerContainer):
    """Optimizer that runs inside backward hooks: the explicit calls are no-ops."""

    def step(self) -> None:
        return None

    def zero_grad(self) -> None:
        return None
