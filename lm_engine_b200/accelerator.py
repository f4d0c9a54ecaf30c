"""Device, seeding and RNG-state helpers.  This engine targets one accelerator family (CUDA sm_100a); CPU is kept
for tests and oracles (the reference's multi-vendor switch is lm_engine/accelerator.py:28-161)."""

from __future__ import annotations

import os
import random
from enum import Enum

import numpy as np
import torch


class Accelerator(str, Enum):
    cpu = "cpu"
    cuda = "cuda"

    @staticmethod
    def get_accelerator() -> "Accelerator":
        return Accelerator.cuda if torch.cuda.is_available() else Accelerator.cpu

    @staticmethod
    def get_device_type() -> str:
        return Accelerator.get_accelerator().value

    @staticmethod
    def get_current_device() -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def set_device(local_rank: int) -> None:
        if torch.cuda.is_available():
            torch.cuda.set_device(local_rank % torch.cuda.device_count())

    @staticmethod
    def set_seed(seed: int) -> None:
        random.seed(seed)
        np.random.seed(seed % (2**32))
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    @staticmethod
    def get_rng_state() -> dict:
        state = {"random": random.getstate(), "np": np.random.get_state(), "torch": torch.get_rng_state()}
        if torch.cuda.is_available():
            state["accelerator"] = torch.cuda.get_rng_state()
        return state

    @staticmethod
    def set_rng_state(state: dict) -> None:
        random.setstate(state["random"])
        np.random.set_state(state["np"])
        torch.set_rng_state(state["torch"])
        if torch.cuda.is_available() and state.get("accelerator") is not None:
            torch.cuda.set_rng_state(state["accelerator"])

    @staticmethod
    def synchronize() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @staticmethod
    def local_rank() -> int:
        return int(os.environ.get("LOCAL_RANK", "0"))
