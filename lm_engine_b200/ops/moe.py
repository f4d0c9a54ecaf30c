"""Mixture-of-experts token routing primitives: expert histogram, grouped (per-expert) linear, and the expert-parallel
all-to-all exchange.

``grouped_linear(x, weight, counts)`` applies ``weight[e]`` to the ``counts[e]`` consecutive rows of ``x`` that were
routed to expert ``e`` (rows sorted by expert) - the operation the reference gets from ScatterMoE
(lm_engine/modeling_utils/mlp_blocks/moe/experts.py:137-149,212-225) or, without it, from a per-expert loop.  On CUDA
bf16 every expert's product runs on the tcgen05 GEMM (including the transposed dgrad / wgrad forms through autograd).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .gemm import linear


def expert_histogram(sorted_expert_idxs: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Tokens per expert (int64 ``[num_experts]``); the input need not be sorted."""
    return torch.bincount(sorted_expert_idxs, minlength=num_experts)


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, counts: list[int],
                   bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x [sum(counts), in]``, ``weight [E, out, in]`` -> ``[sum(counts), out]``."""
    outs = []
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        outs.append(linear(x[start:start + n], weight[e], None if bias is None else bias[e]))
        start += n
    if not outs:
        return x.new_zeros((0, weight.size(1)))
    return torch.cat(outs, dim=0)


class _AllToAll(torch.autograd.Function):
    """Variable-size all-to-all of rows; backward is the all-to-all with the split lists swapped."""

    @staticmethod
    def forward(ctx, x, send_counts: list[int], recv_counts: list[int], group):
        ctx.group, ctx.send, ctx.recv = group, send_counts, recv_counts
        out = x.new_empty((sum(recv_counts), *x.shape[1:]))
        if x.is_cuda:
            dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts,
                                   input_split_sizes=send_counts, group=group)
        else:
            # gloo: emulate with all_gather of padded blocks
            world, r = dist.get_world_size(group), dist.get_rank(group)
            counts = [None] * world
            dist.all_gather_object(counts, send_counts, group=group)
            mx = max(max(c) for c in counts) if counts else 0
            pad = x.new_zeros((world, max(mx, 1), *x.shape[1:]))
            off = 0
            for j, n in enumerate(send_counts):
                pad[j, :n] = x[off:off + n]
                off += n
            gathered = [torch.empty_like(pad) for _ in range(world)]
            dist.all_gather(gathered, pad, group=group)
            pieces = [gathered[src][r, :counts[src][r]] for src in range(world)]
            out = torch.cat(pieces, dim=0) if pieces else out
        return out

    @staticmethod
    def backward(ctx, g):
        return _AllToAll.apply(g, ctx.recv, ctx.send, ctx.group), None, None, None


def all_to_all_rows(x: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    return _AllToAll.apply(x, send_counts, recv_counts, group)
