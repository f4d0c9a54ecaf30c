"""Experiment tracking through wandb or aim, on the tracking rank only (reference: logging_utils/tracking.py:30-214).

State (run id / hash) round-trips through checkpoints so a resumed job continues the same run.
"""

from __future__ import annotations

import os
from typing import Any

from ..enums import ExperimentsTrackerName


class ExperimentsTracker:
    def __init__(self, tracker_name: ExperimentsTrackerName | None, aim_args=None, wandb_args=None,
                 checkpoint_metadata: dict | None = None, is_tracking_rank: bool = True) -> None:
        self.name = tracker_name
        self.enabled = tracker_name is not None and is_tracking_rank
        self.run = None
        self._state: dict[str, Any] = {}
        if not self.enabled:
            return
        meta = checkpoint_metadata or {}
        if tracker_name == ExperimentsTrackerName.wandb:
            import wandb

            kwargs = dict(project=wandb_args.project, name=wandb_args.name, entity=wandb_args.entity,
                          tags=wandb_args.tags, group=wandb_args.group, notes=wandb_args.notes)
            if "id" in meta:
                kwargs.update(id=meta["id"], resume="must")
            self.run = wandb.init(**kwargs)
            self.run.define_metric("iteration")
            self.run.define_metric("*", step_metric="iteration")
            self._state = {"id": self.run.id, "name": self.run.name, "project": wandb_args.project,
                           "entity": wandb_args.entity}
        elif tracker_name == ExperimentsTrackerName.aim:
            from aim import Run

            self.run = Run(run_hash=meta.get("run_hash"), repo=aim_args.repo, experiment=aim_args.experiment)
            self._state = {"run_hash": self.run.hash}
        job = os.environ.get("JOB_ID")
        if job is not None:
            self.log_args({"job_id": job})

    def log_args(self, args: Any) -> None:
        if not self.enabled:
            return
        payload = args.to_dict() if hasattr(args, "to_dict") else dict(args)
        if self.name == ExperimentsTrackerName.wandb:
            self.run.config.update(payload, allow_val_change=True)
        else:
            for k, v in payload.items():
                self.run[k] = v

    def track(self, values: dict[str, float], step: int, context: str | None = None) -> None:
        if not self.enabled:
            return
        if self.name == ExperimentsTrackerName.wandb:
            prefix = f"{context}/" if context else ""
            self.run.log({**{prefix + k: v for k, v in values.items()}, "iteration": step})
        else:
            for k, v in values.items():
                self.run.track(v, name=k, step=step, context={"subset": context} if context else None)

    def state_dict(self) -> dict[str, Any]:
        return dict(self._state)

    def finish(self) -> None:
        if self.enabled and self.name == ExperimentsTrackerName.wandb and self.run is not None:
            self.run.finish()
