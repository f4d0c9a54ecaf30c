"""Context parallelism: sharding of inputs along the sequence over the ``cp`` group.

Two layouts (lm_engine/parallel/context_parallel/__init__.py:26-47, load_balancer.py:16-64):

* contiguous: rank r holds chunk r of ``cp`` equal chunks;
* head-tail : the sequence is cut in ``2 cp`` chunks and rank r holds chunks ``r`` and ``2 cp - 1 - r`` so that causal
  attention work is balanced.
"""

from __future__ import annotations

import torch

from ..enums import ContextParallelLoadBalancerMethod
from .manager import ProcessGroupManager


def shard_indices(seq_len: int, cp: int, rank: int, method: ContextParallelLoadBalancerMethod | None,
                  device=None) -> torch.Tensor:
    """Global positions held by ``rank`` (ascending within each chunk)."""
    if method == ContextParallelLoadBalancerMethod.headtail:
        assert seq_len % (2 * cp) == 0, "sequence length must be divisible by 2 x context parallel size"
        c = seq_len // (2 * cp)
        head = torch.arange(rank * c, (rank + 1) * c, device=device)
        tail = torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c, device=device)
        return torch.cat((head, tail))
    assert seq_len % cp == 0, "sequence length must be divisible by the context parallel size"
    c = seq_len // cp
    return torch.arange(rank * c, (rank + 1) * c, device=device)


def shard_sequence(tensors: tuple[torch.Tensor, ...], seq_dim: int = 1) -> tuple[torch.Tensor, ...]:
    """Returns this rank's context-parallel shard of every tensor (identity when cp = 1)."""
    cp = ProcessGroupManager.get_context_parallel_world_size()
    if cp == 1:
        return tensors
    rank = ProcessGroupManager.get_context_parallel_rank()
    method = ProcessGroupManager.get_context_parallel_load_balancing_method()
    out = []
    for t in tensors:
        idx = shard_indices(t.size(seq_dim), cp, rank, method, device=t.device)
        out.append(t.index_select(seq_dim, idx))
    return tuple(out)


prepare_context_parallel_input = shard_sequence
