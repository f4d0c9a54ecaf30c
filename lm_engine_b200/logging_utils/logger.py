"""Rank-aware logging helpers (reference: lm_engine/logging_utils/logger.py:40-131)."""

from __future__ import annotations

import logging
import os
import sys
from importlib import metadata

_LOGGER: logging.Logger | None = None
_FORMAT = "%(asctime)s - [%(levelname)-8s] ▶ %(message)s"


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def set_logger(level: str | int = logging.INFO, colored_log: bool = False) -> None:
    global _LOGGER
    handler = logging.StreamHandler(sys.stdout)
    if colored_log:
        try:
            from colorlog import ColoredFormatter

            handler.setFormatter(ColoredFormatter("%(log_color)s" + _FORMAT))
        except ImportError:
            handler.setFormatter(logging.Formatter(_FORMAT))
    else:
        handler.setFormatter(logging.Formatter(_FORMAT))
    logger = logging.getLogger("lm_engine_b200")
    logger.handlers[:] = [handler]
    logger.setLevel(level)
    logger.propagate = False
    _LOGGER = logger


def get_logger() -> logging.Logger:
    if _LOGGER is None:
        set_logger()
    return _LOGGER


def log_rank_0(level: int, msg: str) -> None:
    if _rank() == 0:
        get_logger().log(level, msg, stacklevel=3)


def warn_rank_0(msg: str) -> None:
    log_rank_0(logging.WARNING, msg)


_WARNED: set[str] = set()


def warn_once(key: str, msg: str) -> None:
    """One warning per process and ``key`` on the first rank: used where an op leaves its hand-written kernel for
    a library kernel or a PyTorch statement, so that such a change of speed is visible in the log."""
    if key in _WARNED:
        return
    _WARNED.add(key)
    log_rank_0(logging.WARNING, msg)


def print_rank_0(*args, **kwargs) -> None:
    if _rank() == 0:
        print(*args, **kwargs)


def print_ranks_all(*args, **kwargs) -> None:
    """Every rank prints in rank order (needs an initialised process group to serialise)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        print(*args, **kwargs)
        return
    for r in range(dist.get_world_size()):
        if r == dist.get_rank():
            print(f"rank {r}:", *args, **kwargs)
        dist.barrier()


def log_metrics(level: int, msg: str) -> None:
    """Logs on the tracking rank only (first dp/tp/cp rank of the last pipeline stage)."""
    from ..parallel.manager import ProcessGroupManager

    if ProcessGroupManager.is_tracking_rank():
        get_logger().log(level, msg, stacklevel=3)


def log_environment() -> None:
    names = ["torch", "numpy", "transformers", "safetensors", "pydantic", "wandb", "aim", "datasets", "pyarrow"]
    log_rank_0(logging.INFO, "------------------------ packages ------------------------")
    for n in names:
        try:
            log_rank_0(logging.INFO, f"{n} = {metadata.version(n)}")
        except metadata.PackageNotFoundError:
            log_rank_0(logging.INFO, f"{n} is not installed")
    log_rank_0(logging.INFO, "-------------------- end of packages ---------------------")
