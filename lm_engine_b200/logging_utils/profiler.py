"""Profiling hooks: torch profiler traces (same YAML knob as the reference, logging_utils/profiler.py:23-85), NVTX
ranges and device-side step timing with CUDA events."""

from __future__ import annotations

import contextlib

import torch


class StepProfiler:
    """``with StepProfiler(path) as p: ... p.step()``; rank 0 records one step after 5 wait + 5 warm-up steps into a
    TensorBoard/Chrome trace under ``path``.  ``path=None`` disables it."""

    def __init__(self, path: str | None, wait: int = 5, warmup: int = 5, active: int = 1) -> None:
        self.path = path
        self._prof = None
        self._sched = (wait, warmup, active)

    def __enter__(self) -> "StepProfiler":
        import os

        if self.path is not None and int(os.environ.get("RANK", "0")) == 0:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            wait, warmup, active = self._sched
            self._prof = torch.profiler.profile(
                activities=acts,
                schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active, repeat=1),
                on_trace_ready=torch.profiler.tensorboard_trace_handler(self.path),
                record_shapes=True,
                profile_memory=True,
            )
            self._prof.__enter__()
        return self

    def step(self) -> None:
        if self._prof is not None:
            self._prof.step()

    def __exit__(self, *exc) -> None:
        if self._prof is not None:
            self._prof.__exit__(*exc)
            self._prof = None


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class DeviceTimer:
    """Times a region on the device with CUDA events (falls back to the host clock on CPU)."""

    def __init__(self) -> None:
        self._cuda = torch.cuda.is_available()
        if self._cuda:
            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
        self._t0 = 0.0
        self._t1 = 0.0

    def start(self) -> None:
        if self._cuda:
            self._start.record()
        else:
            import time

            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self._cuda:
            self._end.record()
        else:
            import time

            self._t1 = time.perf_counter()

    def elapsed_s(self) -> float:
        if self._cuda:
            self._end.synchronize()
            return self._start.elapsed_time(self._end) * 1e-3
        return self._t1 - self._t0
