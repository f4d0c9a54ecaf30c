"""Linear layers: plain, replicated, column- / row-parallel and low-rank.

All of them compute through :func:`lm_engine_b200.ops.linear` (tcgen05 GEMM with fused bias / residual epilogue on
CUDA bf16).  Column / row variants hold the local tensor-parallel shard as an ordinary parameter and exchange
activations with the collectives of :mod:`lm_engine_b200.parallel.tp_comm` (reference behaviour:
lm_engine/modeling_utils/linear/{base,column,row,replicated,low_rank}.py).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...parallel import tp_comm
from ...parallel.manager import ProcessGroupManager
from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_no_weight_decay,
    mark_tp_shard,
)
from ...utils import divide_if_divisible


def _fused_tp(x: torch.Tensor, padding_free: bool, world: int, gathered: bool, out_features: int) -> bool:
    """Fused collective kernels apply under ``use_async_tensor_parallel`` to activations whose sequence-parallel
    shards concatenate along rows: packed ``[T, H]`` or batch 1 (a ``[B > 1, S, H]`` batch would interleave the
    ranks' rows per batch entry and takes the two-step path)."""
    if not ProcessGroupManager.use_async_tensor_parallel():
        return False
    if not (x.dim() == 2 or padding_free or x.size(0) == 1):
        return False
    from ...parallel.symm import fused_tp_eligible, fused_tp_profitable

    rows = x.numel() // x.size(-1)
    if not fused_tp_eligible(x, rows // world if gathered else rows, world):
        return False
    m = rows if gathered else rows * world
    return fused_tp_profitable("reduce_scatter" if gathered else "all_gather", m, out_features, x.size(-1))


class ParameterizedLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.in_features, self.out_features, self.std = in_features, out_features, std
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if bias else None
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.weight.is_meta:
            return
        if self.std is None:
            nn.init.kaiming_uniform_(self.weight, a=5**0.5)
            if self.bias is not None:
                bound = 1 / self.in_features**0.5
                nn.init.uniform_(self.bias, -bound, bound)
        else:
            nn.init.normal_(self.weight, mean=0, std=self.std)
            if self.bias is not None:
                self.bias.zero_()
        mark_parameter_as_initialized(self.weight)
        mark_parameter_as_initialized(self.bias)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, residual)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class ReplicatedLinear(ParameterizedLinear):
    """Same weight on every tensor-parallel rank (router, shared small projections)."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        mark_tp_shard(self.weight, None)


class ColumnParallelLinear(ParameterizedLinear):
    """Output features split over TP ranks.  Input is sequence-sharded when ``sequence_parallel`` (all-gather in
    forward, reduce-scatter of the input gradient in backward), else replicated (all-reduce of the input gradient)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False, device=None,
                 dtype=None) -> None:
        tp = ProcessGroupManager.get_tensor_parallel_world_size()
        self.tp_world_size = tp
        self.global_out_features = out_features
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        super().__init__(in_features, divide_if_divisible(out_features, tp,
                         f"`out_features` ({out_features}) must be divisible by TP world size ({tp})"),
                         bias=bias, std=std, device=device, dtype=dtype)
        mark_tp_shard(self.weight, 0, (out_features, in_features))
        if self.bias is not None:
            mark_tp_shard(self.bias, 0, (out_features,))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.tp_world_size > 1:
            if self.sequence_parallel and residual is None and _fused_tp(x, self.use_padding_free_transformer,
                                                                         self.tp_world_size, gathered=False,
                                                                         out_features=self.weight.size(0)):
                # all-gather fused into the GEMM (copy CTAs pull the peers' rows over NVLink while the others multiply)
                from ...parallel import symm

                shape = x.shape
                y = symm.all_gather_linear(x.reshape(-1, shape[-1]), self.weight, self.bias,
                                           ProcessGroupManager.get_tensor_parallel_group())
                lead = (shape[0] * self.tp_world_size,) if x.dim() == 2 else (shape[0], shape[1] * self.tp_world_size)
                return y.view(*lead, self.weight.size(0))
            if self.sequence_parallel:
                x = tp_comm.gather_from_sequence_parallel(x, tp_comm.seq_dim(x, self.use_padding_free_transformer))
            else:
                x = tp_comm.copy_to_tensor_parallel(x)
        return ops.linear(x, self.weight, self.bias, residual)


class RowParallelLinear(ParameterizedLinear):
    """Input features split over TP ranks; partial outputs are reduce-scattered along the sequence
    (``sequence_parallel``) or all-reduced.  The bias is added once, after the reduction."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False, device=None,
                 dtype=None) -> None:
        tp = ProcessGroupManager.get_tensor_parallel_world_size()
        self.tp_world_size = tp
        self.global_in_features = in_features
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        super().__init__(divide_if_divisible(in_features, tp,
                         f"`in_features` ({in_features}) must be divisible by TP world size ({tp})"),
                         out_features, bias=bias, std=std, device=device, dtype=dtype)
        mark_tp_shard(self.weight, 1, (out_features, in_features))
        if self.bias is not None:
            mark_tp_shard(self.bias, None)
            # added after the reduce-scatter, i.e. to this rank's slice of the sequence only: its gradient is a
            # partial sum that the sharding runtime all-reduces over the tensor-parallel group
            self.bias.sequence_parallel_grad = sequence_parallel and tp > 1

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.tp_world_size == 1:
            return ops.linear(x, self.weight, self.bias, residual)
        if self.sequence_parallel and _fused_tp(x, self.use_padding_free_transformer, self.tp_world_size,
                                                gathered=True, out_features=self.weight.size(0)):
            # reduce-scatter (+ bias + residual) fused into the GEMM epilogue over NVLink peer stores
            from ...parallel import symm

            shape = x.shape
            r2 = residual.reshape(-1, self.weight.size(0)) if residual is not None else None
            y = symm.linear_reduce_scatter(x.reshape(-1, shape[-1]), self.weight, self.bias, r2,
                                           ProcessGroupManager.get_tensor_parallel_group())
            lead = (shape[0] // self.tp_world_size,) if x.dim() == 2 else (shape[0], shape[1] // self.tp_world_size)
            return y.view(*lead, self.weight.size(0))
        y = ops.linear(x, self.weight, None, None)
        if self.sequence_parallel:
            y = tp_comm.scatter_to_sequence_parallel(y, tp_comm.seq_dim(y, self.use_padding_free_transformer))
        else:
            y = tp_comm.reduce_from_tensor_parallel(y)
        if self.bias is not None:
            y = y + self.bias
        if residual is not None:
            y = y + residual
        return y


class LowRankLinear(nn.Module):
    """``up(down(x))`` with an inner dimension ``rank`` (lm_engine/modeling_utils/linear/low_rank.py:11-28)."""

    def __init__(self, in_features: int, out_features: int, rank: int, bias: bool = True,
                 std: float | None = None) -> None:
        super().__init__()
        self.l1 = ParameterizedLinear(in_features, rank, bias=False, std=std)
        self.l2 = ParameterizedLinear(rank, out_features, bias=bias, std=std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.l2(self.l1(x))
