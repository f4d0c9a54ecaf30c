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
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import _max_ctas

_SEG = 32 * 1024
_PAD_WORDS = 16
_CONTEXTS: dict[tuple[int, int], "GatherContext"] = {}
# copy CTAs inside the GEMM grid that pull the peers' rows; 0 = copy engines deliver them (see all_gather_matmul)
N_COPY_CTAS = int(os.environ.get("LME_GATHER_CTAS", "0"))
CE_CHUNK = 1 << int(os.environ.get("LME_GATHER_CHUNK_SHIFT", "22"))   # bytes per copy-engine chunk / readiness word


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
        self.stage_local = [self.arena[slot * shard_bytes:(slot + 1) * shard_bytes] for slot in range(2)]
        self.stage_peer = [[self.handle.get_buffer(r, (shard_bytes,), torch.uint8, slot * shard_bytes)
                            for r in range(self.world)] for slot in range(2)]
        self.ready_ce = torch.zeros(self.world * ((shard_bytes + CE_CHUNK - 1) // CE_CHUNK), dtype=torch.int32,
                                    device=device)
        self.side = torch.cuda.Stream(device)
        self._pad_arr = (ctypes.c_void_p * 8)(*(self.pads + [None] * (8 - self.world)))
        self._stage_arr = [(ctypes.c_void_p * 8)(*(self.stage[s] + [None] * (8 - self.world))) for s in range(2)]
        # the zeroed pads must be in place everywhere before anybody signals
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


class ScatterContext:
    """Receive slabs (two slots) and arrival flags for :func:`matmul_reduce_scatter` on one (group, shape)."""

    def __init__(self, group, rows_per_rank: int, n: int, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= 8 and rows_per_rank % 128 == 0
        slab_bytes = self.world * rows_per_rank * n * 2
        tiles_n = (n + (128 if n <= 128 else 256) - 1) // (128 if n <= 128 else 256)
        n_flags = self.world * (rows_per_rank // 128) * tiles_n * 4
        slabs = (2 * slab_bytes + 255) // 256 * 256
        self.arena = symm_mem.empty(slabs + n_flags * 4, dtype=torch.uint8, device=device)
        self.arena[slabs:].zero_()
        self.handle = symm_mem.rendezvous(self.arena, group)
        self.slab = [[self.handle.get_buffer(r, (slab_bytes,), torch.uint8, slot * slab_bytes).data_ptr()
                      for r in range(self.world)] for slot in range(2)]
        self.flags = [self.handle.get_buffer(r, (n_flags,), torch.int32, slabs // 4).data_ptr()
                      for r in range(self.world)]
        self._slab_arr = [(ctypes.c_void_p * 8)(*(self.slab[s] + [None] * (8 - self.world))) for s in range(2)]
        self._flag_arr = (ctypes.c_void_p * 8)(*(self.flags + [None] * (8 - self.world)))
        self.seq = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


_SCATTER: dict[tuple[int, int, int], ScatterContext] = {}


def matmul_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, group, *, bias: torch.Tensor | None = None,
                          residual: torch.Tensor | None = None, weight_mn: bool = False) -> torch.Tensor:
    """``reduce_scatter_rows(x @ weight.T) (+ bias) (+ residual)``: ``x`` is ``[M, K_local]``, every rank holds a
    K-slice; returns this rank's ``[M / world, N]`` rows of the sum.  One kernel: the epilogue of the tiles of a
    peer's rows stores into that peer's memory, the epilogue of own tiles adds what the peers sent."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    x = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 else x.contiguous()
    w = weight if weight.stride(1) == 1 and weight.stride(0) % 8 == 0 else weight.contiguous()
    M, K = x.shape
    N = w.size(1) if weight_mn else w.size(0)
    world = dist.get_world_size(group)
    key = (id(group), M // world, N)
    if key not in _SCATTER:
        _SCATTER[key] = ScatterContext(group, M // world, N, x.device)
    ctx = _SCATTER[key]
    out = torch.empty((M // world, N), dtype=torch.bfloat16, device=x.device)
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(1) == 1
    ctx.seq += 1
    rc = _lib.cuda_lib().lme_gemm_bf16_reduce_scatter(
        x.data_ptr(), x.stride(0), w.data_ptr(), int(weight_mn), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        ctx._slab_arr[ctx.seq & 1], ctx._flag_arr, ctx.rank, ctx.world, ctx.seq, _max_ctas(x.device),
        _lib.stream_ptr())
    _lib.check(rc, f"lme_gemm_bf16_reduce_scatter M={M} N={N} K={K}")
    _lib.count_launch()
    return out


def gather_context(group, shard_bytes: int, device: torch.device) -> GatherContext:
    key = (id(group), shard_bytes)
    if key not in _CONTEXTS:
        _CONTEXTS[key] = GatherContext(group, shard_bytes, device)
    return _CONTEXTS[key]


def all_gather_matmul(x_shard: torch.Tensor, weight: torch.Tensor, group, *, bias: torch.Tensor | None = None,
                      swiglu: bool = False, preact: torch.Tensor | None = None, n_copy: int | None = None,
                      weight_mn: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """``(concat_over_ranks(x_shard) @ weight.T [+ bias], concat_over_ranks(x_shard))``.
    ``x_shard`` is this rank's ``[t, K]`` bf16 rows; rank r's rows land at ``[r * t, (r + 1) * t)``.
    ``weight_mn``: ``weight`` is ``[K, N]`` (the product is ``x @ weight``), read in place by the tensor core."""
    assert x_shard.is_cuda and x_shard.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    x_shard = x_shard.contiguous()
    t, K = x_shard.shape
    N = weight.size(1) if weight_mn else weight.size(0)
    ctx = gather_context(group, t * K * 2, x_shard.device)
    M = t * ctx.world
    gathered = torch.empty((M, K), dtype=torch.bfloat16, device=x_shard.device)
    out = torch.empty((M, N // 2 if swiglu else N), dtype=torch.bfloat16, device=x_shard.device)
    flags = _lib.GEMM_SWIGLU if swiglu else 0
    ctx.seq += 1
    slot = ctx.seq & 1
    w = weight if weight.stride(1) == 1 and weight.stride(0) % 8 == 0 else weight.contiguous()
    lib = _lib.cuda_lib()
    n_copy = N_COPY_CTAS if n_copy is None else n_copy
    cur = torch.cuda.current_stream()
    # own rows: into the staging slot the peers read (before anything announces it) and, off the critical path, into
    # their place in the gathered operand (the GEMM itself reads them from x_shard)
    ctx.stage_local[slot].copy_(x_shard.view(torch.uint8).view(-1))
    ctx.side.wait_stream(cur)
    with torch.cuda.stream(ctx.side):
        side = _lib.stream_ptr()
        if n_copy == 0:
            # copy engines deliver the peers' rows: announce, then per peer wait for its announcement and copy chunk
            # by chunk, each chunk followed by a stream write of its readiness word
            _lib.check(lib.lme_gather_signal(ctx._pad_arr, ctx.rank, ctx.world, ctx.seq, side), "lme_gather_signal")
            flat = gathered.view(torch.uint8).view(-1)
            nchunk = (ctx.shard_bytes + CE_CHUNK - 1) // CE_CHUNK
            for i in range(1, ctx.world):
                p = (ctx.rank + i) % ctx.world
                _lib.check(lib.lme_gather_wait_peer(ctx.pads[ctx.rank], p, ctx.seq, side), "lme_gather_wait_peer")
                for c in range(nchunk):
                    lo, hi = c * CE_CHUNK, min((c + 1) * CE_CHUNK, ctx.shard_bytes)
                    flat[p * ctx.shard_bytes + lo:p * ctx.shard_bytes + hi].copy_(ctx.stage_peer[slot][p][lo:hi],
                                                                                    non_blocking=True)
                    _lib.check(lib.lme_stream_write_words(ctx.ready_ce.data_ptr() + 4 * (p * nchunk + c), 1, ctx.seq,
                                                          side), "lme_stream_write_words")
        gathered[ctx.rank * t:(ctx.rank + 1) * t].copy_(x_shard)
    ready = ctx.ready_ce if n_copy == 0 else ctx.ready
    rc = lib.lme_gemm_bf16_allgather_a(
        gathered.data_ptr(), K, w.data_ptr(), int(weight_mn), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        flags, _lib.ptr(bias), None, 0, _lib.ptr(preact), preact.stride(0) if preact is not None else 0,
        x_shard.data_ptr(), ctx._stage_arr[slot], ctx._pad_arr, ready.data_ptr(), ctx.counters.data_ptr(),
        ctx.shard_bytes, ctx.rank, ctx.world, ctx.seq, n_copy, CE_CHUNK.bit_length() - 1, _max_ctas(x_shard.device),
        _lib.stream_ptr())
    cur.wait_stream(ctx.side)
    x_shard.record_stream(ctx.side)
    _lib.check(rc, f"lme_gemm_bf16_allgather_a M={M} N={N} K={K}")
    _lib.count_launch()
    return out, gathered


# ---------------------------------------------------------------------------------------------------- autograd
class _AllGatherLinear(torch.autograd.Function):
    """Sequence-parallel column linear: ``y = all_gather_rows(x) @ W.T (+ b)`` with the gather fused into the GEMM;
    backward runs ``dx = reduce_scatter_rows(dy @ W)`` with the scatter fused into that GEMM's epilogue."""

    @staticmethod
    def forward(ctx, x, weight, bias, group):
        y, xg = all_gather_matmul(x, weight, group, bias=bias)
        ctx.save_for_backward(xg, weight)
        ctx.group, ctx.has_bias = group, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import _wgrad_into, gemm

        xg, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_reduce_scatter(dy, weight, ctx.group, weight_mn=True)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                _wgrad_into(main_grad, weight, dy, xg)
            else:
                dw = gemm(dy, xg, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(0, dtype=torch.float32).to(dy.dtype)
        return dx, dw, db, None


class _LinearReduceScatter(torch.autograd.Function):
    """Sequence-parallel row linear: ``y = reduce_scatter_rows(x @ W.T) (+ b) (+ residual)`` in one kernel; backward
    gathers ``dy`` inside the input-gradient GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, group):
        y = matmul_reduce_scatter(x, weight, group, bias=bias, residual=residual)
        ctx.save_for_backward(x, weight)
        ctx.group, ctx.has_bias, ctx.has_residual = group, bias is not None, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import _wgrad_into, gemm

        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx, dy_full = all_gather_matmul(dy, weight, ctx.group, weight_mn=True)
        dw = db = dres = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                _wgrad_into(main_grad, weight, dy_full, x)
            else:
                dw = gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(0, dtype=torch.float32).to(dy.dtype)   # over this rank's rows; all-reduced by the engine
        if ctx.has_residual and ctx.needs_input_grad[3]:
            dres = dy
        return (dx if ctx.needs_input_grad[0] else None), dw, db, dres, None


def fused_tp_eligible(x: torch.Tensor, rows_local: int, world: int) -> bool:
    """The fused kernels take packed bf16 rows whose per-rank block is a whole number of 128-row tiles."""
    return x.is_cuda and x.dtype == torch.bfloat16 and 2 <= world <= 8 and rows_local % 128 == 0


# Measured on B200 (tp 2 / 4 / 8, 8192 tokens): the fused kernels beat "NCCL collective + GEMM" once the GEMM is long
# enough to hide the transfer and the host-side enqueue of the chunk copies; below that the two-step path wins.
_MIN_MNK = {"all_gather": 1.0e11, "reduce_scatter": 6.0e10}


def fused_tp_profitable(kind: str, m: int, n: int, k: int) -> bool:
    mode = os.environ.get("LME_FUSED_TP", "auto")
    if mode == "always":
        return True
    if mode == "never":
        return False
    return float(m) * n * k >= _MIN_MNK[kind]


def all_gather_linear(x, weight, bias, group):
    return _AllGatherLinear.apply(x, weight, bias, group)


def linear_reduce_scatter(x, weight, bias, residual, group):
    return _LinearReduceScatter.apply(x, weight, bias, residual, group)
