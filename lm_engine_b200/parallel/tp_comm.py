"""Differentiable tensor-parallel collectives on plain local tensors (no DTensor on the hot path).

Megatron-style sequence parallelism keeps activations sharded on the sequence dimension between a row-parallel
linear and the next column-parallel linear (reference: lm_engine/modeling_utils/TP.py:44-53,
lm_engine/modeling_utils/linear/{column,row}.py).  Each function is its own transpose in backward:

====================  ==========================  ==========================
 forward               backward                    used by
====================  ==========================  ==========================
 all-gather (seq)      reduce-scatter (seq)        column linear input (SP)
 reduce-scatter (seq)  all-gather (seq)            row linear output (SP)
 identity              all-reduce                  column linear input (no SP)
 all-reduce            identity                    row linear output (no SP)
====================  ==========================  ==========================

With ``use_async_tensor_parallel`` the linears bypass these and call the fused all-gather->GEMM /
GEMM->reduce-scatter kernels of :mod:`lm_engine_b200.parallel.symm` instead.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .manager import ProcessGroupManager


def _tp():
    return ProcessGroupManager.get_tensor_parallel_group()


def _all_gather_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    x = x.contiguous()
    if dim == 0:
        out = torch.empty((world * x.size(0), *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    parts = torch.empty((world, *x.shape), dtype=x.dtype, device=x.device)
    # flat view: the gloo backend only takes the concatenated output form
    dist.all_gather_into_tensor(parts.view(-1, *x.shape[1:]) if x.dim() > 0 else parts, x, group=group)
    return torch.cat(list(parts.unbind(0)), dim=dim)


def _reduce_scatter_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    if dim != 0:
        x = torch.cat(x.chunk(world, dim=dim), dim=0)
    x = x.contiguous()
    out = torch.empty((x.size(0) // world, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.device.type == "cpu":
        # gloo has no reduce_scatter_tensor: all-reduce then slice
        y = x.clone()
        dist.all_reduce(y, group=group)
        r = dist.get_rank(group)
        out.copy_(y.chunk(world, dim=0)[r])
    else:
        dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _all_gather_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim(g, ctx.dim, ctx.group), None, None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _reduce_scatter_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.dim, ctx.group), None, None


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLast(torch.autograd.Function):
    """all-gather along the last dim; backward keeps the local slice (used for logits when not output-parallel)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_dim(x, x.dim() - 1, group)

    @staticmethod
    def backward(ctx, g):
        world, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        return g.chunk(world, dim=-1)[r].contiguous(), None


def seq_dim(x: torch.Tensor, use_padding_free_transformer: bool) -> int:
    """sequence dimension of an activation: 0 for packed [T, H], 1 for [B, S, H]"""
    return 0 if (use_padding_free_transformer or x.dim() == 2) else 1


def gather_from_sequence_parallel(x, dim):
    g = _tp()
    return x if g is None else _GatherSeq.apply(x, dim, g)


def scatter_to_sequence_parallel(x, dim):
    g = _tp()
    return x if g is None else _ScatterSeq.apply(x, dim, g)


def copy_to_tensor_parallel(x):
    g = _tp()
    return x if g is None else _CopyToTP.apply(x, g)


def reduce_from_tensor_parallel(x):
    g = _tp()
    return x if g is None else _ReduceFromTP.apply(x, g)


def gather_last_dim_from_tensor_parallel(x):
    g = _tp()
    return x if g is None else _GatherLast.apply(x, g)


def split_to_sequence_parallel(x: torch.Tensor, dim: int) -> torch.Tensor:
    """Takes this TP rank's slice along the sequence dim (forward: slice, backward: all-gather)."""
    g = _tp()
    if g is None:
        return x

    class _Split(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t):
            return t.chunk(dist.get_world_size(g), dim=dim)[dist.get_rank(g)].contiguous()

        @staticmethod
        def backward(ctx, gr):
            return _all_gather_dim(gr, dim, g)

    return _Split.apply(x)
