"""Context parallelism for non-linear recurrences: the ranks form a pipeline along the sequence.  Rank r waits for
the boundary state of rank r-1, runs its shard, hands its final state to rank r+1; in backward the state gradient
travels the other way and each rank recomputes its shard locally
(lm_engine/modeling_utils/sequence_pipeline.py:15-143, rotaters/{send,recv}.py)."""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from .manager import ProcessGroupManager


class _SequencePipeline(torch.autograd.Function):
    @staticmethod
    def forward(ctx, function: Callable, state_shape: tuple, group, *tensors: torch.Tensor):
        world, r = dist.get_world_size(group), dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        ref = tensors[0]
        h0 = torch.zeros(state_shape, dtype=ref.dtype, device=ref.device)
        if r > 0:
            dist.recv(h0, src=ranks[r - 1], group=group)
        with torch.no_grad():
            y, h = function(*tensors, h0)
        if r + 1 < world:
            dist.send(h.contiguous(), dst=ranks[r + 1], group=group)
        ctx.function, ctx.group = function, group
        ctx.save_for_backward(h0, *tensors)
        return y, h

    @staticmethod
    def backward(ctx, dy, dh_out):
        h0, *tensors = ctx.saved_tensors
        group = ctx.group
        world, r = dist.get_world_size(group), dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        dh = torch.zeros_like(h0) if dh_out is None else dh_out.clone()
        if r + 1 < world:
            incoming = torch.empty_like(h0)
            dist.recv(incoming, src=ranks[r + 1], group=group)
            dh = dh + incoming
        ins = [t.detach().requires_grad_(t.requires_grad or isinstance(t, torch.nn.Parameter)) for t in tensors]
        h0r = h0.detach().requires_grad_(True)
        with torch.enable_grad():
            y, h = ctx.function(*ins, h0r)
        torch.autograd.backward([y, h], [dy, dh])
        if r > 0:
            dist.send(h0r.grad.contiguous(), dst=ranks[r - 1], group=group)
        return (None, None, None, *[t.grad for t in ins])


def sequence_pipeline(function: Callable, tensors: tuple[torch.Tensor, ...], state_shape: tuple):
    """``function(*tensors, h0) -> (y, h_final)`` evaluated on this rank's sequence shard with the state carried
    across the context-parallel ranks."""
    group = ProcessGroupManager.get_context_parallel_group()
    if group is None:
        ref = tensors[0]
        return function(*tensors, torch.zeros(state_shape, dtype=ref.dtype, device=ref.device))
    return _SequencePipeline.apply(function, tuple(state_shape), group, *tensors)
