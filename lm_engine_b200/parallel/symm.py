"""Fused compute + collective operators over NVLink peer memory (symmetric memory).

:func:`all_gather_matmul` is the sequence-parallel ``all-gather -> column-parallel GEMM`` as ONE kernel: a few CTAs
of the GEMM grid pull the peers' activation shards with bulk asynchronous copies (TMA engine, plain peer loads, no
multicast) into the local gathered operand while the remaining CTAs already multiply the row tiles that are present,
starting with this rank's own rows.  The reference reaches the same overlap through inductor's micro-pipeline pass and
``symm_mem.fused_all_gather_matmul`` (lm_engine/parallel/manager.py:241-243, modeling_utils/linear/column.py:59-60).

Buffers: per (process group, shard size) one symmetric allocation holds two staging slots for this rank's shard and a
16-word signal pad; ``seq`` counts the calls, the slot is ``seq & 1``.  All device-side waits are bounded; a timed-out
wait shows up in :func:`lm_engine_b200.ops._lib.read_status`.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import _max_ctas

_SEG = 32 * 1024
_PAD_WORDS = 16
_CONTEXTS: dict[tuple[int, int], "GatherContext"] = {}
N_COPY_CTAS = 8


class GatherContext:
    def __init__(self, group, shard_bytes: int, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.shard_bytes = group, shard_bytes
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= 8, "a gather group spans at most the 8 GPUs of one NVLink domain"
        assert shard_bytes % 16 == 0
        stage_bytes = (2 * shard_bytes + 255) // 256 * 256
        self.arena = symm_mem.empty(stage_bytes + _PAD_WORDS * 4, dtype=torch.uint8, device=device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, group)
        pad_off = stage_bytes // 4
        self.stage = [[self.handle.get_buffer(r, (shard_bytes,), torch.uint8, slot * shard_bytes).data_ptr()
                       for r in range(self.world)] for slot in range(2)]
        self.pads = [self.handle.get_buffer(r, (_PAD_WORDS,), torch.int32, pad_off).data_ptr()
                     for r in range(self.world)]
        nseg = (shard_bytes + _SEG - 1) // _SEG
        self.ready = torch.zeros(self.world * nseg, dtype=torch.int32, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.seq = 0
        self._pad_arr = (ctypes.c_void_p * 8)(*(self.pads + [None] * (8 - self.world)))
        self._stage_arr = [(ctypes.c_void_p * 8)(*(self.stage[s] + [None] * (8 - self.world))) for s in range(2)]
        # the zeroed pads must be in place everywhere before anybody signals
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


def gather_context(group, shard_bytes: int, device: torch.device) -> GatherContext:
    key = (id(group), shard_bytes)
    if key not in _CONTEXTS:
        _CONTEXTS[key] = GatherContext(group, shard_bytes, device)
    return _CONTEXTS[key]


def all_gather_matmul(x_shard: torch.Tensor, weight: torch.Tensor, group, *, bias: torch.Tensor | None = None,
                      swiglu: bool = False, preact: torch.Tensor | None = None,
                      n_copy: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``(concat_over_ranks(x_shard) @ weight.T [+ bias], concat_over_ranks(x_shard))``.
    ``x_shard`` is this rank's ``[t, K]`` bf16 rows; rank r's rows land at ``[r * t, (r + 1) * t)``."""
    assert x_shard.is_cuda and x_shard.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    x_shard = x_shard.contiguous()
    t, K = x_shard.shape
    N = weight.size(0)
    ctx = gather_context(group, t * K * 2, x_shard.device)
    M = t * ctx.world
    gathered = torch.empty((M, K), dtype=torch.bfloat16, device=x_shard.device)
    out = torch.empty((M, N // 2 if swiglu else N), dtype=torch.bfloat16, device=x_shard.device)
    flags = _lib.GEMM_SWIGLU if swiglu else 0
    ctx.seq += 1
    slot = ctx.seq & 1
    w = weight if weight.stride(1) == 1 and weight.stride(0) % 8 == 0 else weight.contiguous()
    rc = _lib.cuda_lib().lme_gemm_bf16_allgather_a(
        gathered.data_ptr(), K, w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K, flags,
        _lib.ptr(bias), None, 0, _lib.ptr(preact), preact.stride(0) if preact is not None else 0,
        x_shard.data_ptr(), ctx._stage_arr[slot], ctx._pad_arr, ctx.ready.data_ptr(), ctx.counters.data_ptr(),
        ctx.shard_bytes, ctx.rank, ctx.world, ctx.seq, n_copy or N_COPY_CTAS, _max_ctas(x_shard.device),
        _lib.stream_ptr())
    _lib.check(rc, f"lme_gemm_bf16_allgather_a M={M} N={N} K={K}")
    _lib.count_launch()
    return out, gathered
