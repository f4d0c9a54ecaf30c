"""Input distribution over the tensor-parallel group: only the first TP rank runs a dataloader; the token batch is
broadcast to the others (lm_engine/parallel/tensor_parallel.py:12-29)."""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..accelerator import Accelerator
from .manager import ProcessGroupManager


def broadcast_tensor_parallel_input(tokens: torch.Tensor | None, shape: tuple[int, int]) -> torch.Tensor:
    device = Accelerator.get_current_device()
    group = ProcessGroupManager.get_tensor_parallel_group()
    if group is None:
        return tokens.to(device, non_blocking=True)
    if ProcessGroupManager.is_tensor_parallel_first_rank():
        tokens = tokens.to(device, non_blocking=True)
    else:
        tokens = torch.empty(shape, dtype=torch.long, device=device)
    dist.broadcast(tokens, src=ProcessGroupManager.get_tensor_parallel_first_rank(), group=group)
    return tokens
