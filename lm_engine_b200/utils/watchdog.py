"""Failure detection on the host: a per-rank heartbeat file and a watchdog thread.

The training loop calls :meth:`Heartbeat.beat` once per optimizer step; the file ``<dir>/heartbeat-<rank>.json`` then
holds the step, a wall-clock stamp and the device status words of the kernel library.  A watchdog thread inside every
rank wakes up periodically and

* reports (and, when ``abort`` is set, ends the process with exit code 75 so that the launcher restarts the job from
  the last checkpoint) when its own rank has not completed a step within ``stall_seconds``;
* reports peers whose heartbeat file is older than ``stall_seconds`` (a rank that died or hangs in a collective shows
  up here before the process-group timeout fires).

Nothing here touches the GPU: a hung device is detected by the absence of progress, never by probing it.  The
reference only has the process-group timeout and the ``KILLSWITCH`` file (lm_engine/arguments/__init__.py:302-303,
lm_engine/checkpointing/__init__.py:40,148-149); both are kept.
"""

from __future__ import annotations

import json
import logging
import os
import threading
import time

EXIT_STALLED = 75   # EX_TEMPFAIL: "try again later"

log = logging.getLogger("lm_engine_b200.watchdog")


def _path(directory: str, rank: int) -> str:
    return os.path.join(directory, f"heartbeat-{rank}.json")


def abort_is_safe(environ=None) -> bool:
    """Ending a rank from the watchdog thread (``os._exit``) is only allowed when no memory of that rank can be bound
    to an NVLink multicast object: NCCL's in-switch reductions off and the gradient reduce-scatter on plain peer
    loads.  Otherwise the rank has to leave between steps (KILLSWITCH, process-group timeout)."""
    env = os.environ if environ is None else environ
    return env.get("NCCL_NVLS_ENABLE", "") == "0" and env.get("LME_REDUCE_SCATTER", "fused") != "nvls"


class Heartbeat:
    def __init__(self, directory: str, rank: int, world_size: int, stall_seconds: float = 600.0,
                 poll_seconds: float = 10.0, abort: bool = False, on_stall=None) -> None:
        self.directory, self.rank, self.world_size = directory, rank, world_size
        self.stall_seconds, self.poll_seconds, self.abort = stall_seconds, poll_seconds, abort
        self.on_stall = on_stall
        self.step = -1
        self._last = time.time()
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self.stalled_peers: list[int] = []
        os.makedirs(directory, exist_ok=True)

    # ------------------------------------------------------------------ called by the training loop
    def beat(self, step: int, device_status: list[int] | None = None) -> None:
        self.step, self._last = step, time.time()
        tmp = _path(self.directory, self.rank) + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"rank": self.rank, "step": step, "time": self._last, "device_status": device_status}, f)
        os.replace(tmp, _path(self.directory, self.rank))

    # ------------------------------------------------------------------ watchdog thread
    def start(self) -> "Heartbeat":
        self._thread = threading.Thread(target=self._run, name="lme-watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.poll_seconds + 1)

    def check(self, now: float | None = None) -> tuple[bool, list[int]]:
        """``(own rank stalled, peers whose heartbeat is stale or missing)``."""
        now = time.time() if now is None else now
        own = now - self._last > self.stall_seconds
        stale = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                with open(_path(self.directory, r)) as f:
                    t = json.load(f)["time"]
            except (OSError, ValueError, KeyError):
                t = None
            if t is None or now - t > self.stall_seconds:
                stale.append(r)
        return own, stale

    def _run(self) -> None:
        while not self._stop.wait(self.poll_seconds):
            own, stale = self.check()
            self.stalled_peers = stale
            if stale:
                log.warning("rank %d: no heartbeat from ranks %s for %.0f s", self.rank, stale, self.stall_seconds)
            if own:
                log.error("rank %d: no step completed for %.0f s (last step %d)", self.rank, self.stall_seconds,
                          self.step)
                if self.on_stall is not None:
                    self.on_stall(self)
                if self.abort:
                    os._exit(EXIT_STALLED)
