"""Context-parallel attention with the key / value exchange fused into the attention kernel.

The reference rotates K / V blocks around a ring of flash-attention calls and merges the partial results by their
log-sum-exps, with the gradient accumulators travelling the ring in the backward pass
(lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/ring_attention.py:41-199, 202-434).  Here every
rank's K / V shard is published in symmetric memory; copy engines pull the peers' shards over NVLink into this GPU's
own position-ordered K / V buffer, chunk by chunk, and the stream writes one readiness word per chunk.  ONE launch of
the tcgen05 attention kernel per run of local query positions then walks the whole key range: its TMA producer waits
(bounded) for the word of a chunk before it loads the first tile of that chunk, so the exchange overlaps the tiles
that are already there, the online softmax simply continues across chunks (no partial outputs, no log-sum-exp merge),
and no SM is spent on the transfer.  The kernel's tensor maps cover local memory only.

Backward: the dQ kernel and the dK / dV kernel run over the gathered K / V; every rank's dK / dV for the whole key
range land in symmetric memory and each rank sums its own chunks from all ranks with the peer-load reduce-scatter
kernel (fp32 sums in rank order), the kernel that also serves the ZeRO gradient path.

Layouts: contiguous sharding (rank r holds chunk r) and head-tail balancing (chunks r and 2 cp - 1 - r); in both the
gathered buffer is in global position order, so a run of local queries is an ordinary causal problem whose last
query is aligned with the last key it may see.
"""

from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist

from ..enums import ContextParallelLoadBalancerMethod
from ..ops import _lib
from .manager import ProcessGroupManager

_PAD_WORDS = 16
_CONTEXTS: dict[tuple, "_KVExchange"] = {}


def chunk_layout(cp: int, rank: int, method) -> list[int]:
    """Global chunk ids held by ``rank``, in the order of its local rows."""
    if method == ContextParallelLoadBalancerMethod.headtail:
        return [rank, 2 * cp - 1 - rank]
    return [rank]


class _KVExchange:
    """Symmetric buffers of one (group, K / V shard shape): two staging slots for this rank's K / V, two slots for the
    dK / dV partial results over the whole key range, a signal pad, the readiness words and a side stream."""

    def __init__(self, group, B: int, S_local: int, Hkv: int, D: int, method, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.method = group, method
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= 8, "a context-parallel group spans at most the 8 GPUs of one NVLink domain"
        self.B, self.S_local, self.Hkv, self.D = B, S_local, Hkv, D
        self.chunks_per_rank = 2 if method == ContextParallelLoadBalancerMethod.headtail else 1
        self.chunk_rows = S_local // self.chunks_per_rank
        self.n_chunks = self.world * self.chunks_per_rank
        self.S_total = S_local * self.world
        shard = 2 * B * S_local * Hkv * D                      # bf16 elements of one rank's K and V
        full = 2 * B * self.S_total * Hkv * D                  # dK and dV over the whole key range
        self.shard_elems, self.full_elems = shard, full
        total = 2 * shard + 2 * full
        self.arena = symm_mem.empty(total * 2 + 2 * _PAD_WORDS * 4, dtype=torch.uint8, device=device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, group)
        bf = torch.bfloat16
        self.stage_peer = [[self.handle.get_buffer(r, (2, B, S_local, Hkv * D), bf, slot * shard)
                            for r in range(self.world)] for slot in range(2)]
        self.grad_peer = [[self.handle.get_buffer(r, (2, B, self.S_total, Hkv * D), bf, 2 * shard + slot * full)
                           for r in range(self.world)] for slot in range(2)]
        pad0 = total * 2 // 4
        self.pads = [self.handle.get_buffer(r, (_PAD_WORDS,), torch.int32, pad0).data_ptr()
                     for r in range(self.world)]
        self.rs_pads = [self.handle.get_buffer(r, (_PAD_WORDS,), torch.int32, pad0 + _PAD_WORDS).data_ptr()
                        for r in range(self.world)]
        self._pad_arr = (ctypes.c_void_p * 8)(*(self.pads + [None] * (8 - self.world)))
        self._rs_pad_arr = (ctypes.c_void_p * 8)(*(self.rs_pads + [None] * (8 - self.world)))
        self.ready = torch.zeros((B, self.n_chunks), dtype=torch.int32, device=device)
        self.side = torch.cuda.Stream(device)
        self.seq = 0          # forward calls (staging slot = seq & 1)
        self.rs_seq = 0       # reduce-scatter launches of the backward pass
        self.bwd_calls = 0    # backward calls (gradient slot = bwd_calls & 1)
        self.stream_waits = True
        # the attention kernel waits for chunks that a peer sends when IT reaches this layer
        _lib.raise_peer_wait_limit()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


def _exchange(group, k: torch.Tensor, method) -> _KVExchange:
    B, S_local, Hkv, D = k.shape
    key = (id(group), B, S_local, Hkv, D, str(method))
    if key not in _CONTEXTS:
        _CONTEXTS[key] = _KVExchange(group, B, S_local, Hkv, D, method, k.device)
    return _CONTEXTS[key]


def eligible(q: torch.Tensor, k: torch.Tensor, causal: bool, sliding_window, method) -> bool:
    """bf16, head dim 128, no window, causal, and chunks that are whole 128-row tiles."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.size(-1) == 128):
        return False
    if sliding_window is not None or not causal or q.dim() != 4 or q.size(1) != k.size(1):
        return False
    per = 2 if method == ContextParallelLoadBalancerMethod.headtail else 1
    return q.size(1) % (128 * per) == 0 and q.size(2) % k.size(2) == 0


def _gather_kv(ex: _KVExchange, k: torch.Tensor, v: torch.Tensor) -> tuple[torch.Tensor, int]:
    """Publishes this rank's K / V, starts the pulls of the peers' chunks on the side stream and returns the
    position-ordered ``[2, B, S_total, Hkv * D]`` buffer that fills up behind the readiness words."""
    lib = _lib.cuda_lib()
    B, S_l, HD, c = ex.B, ex.S_local, ex.Hkv * ex.D, ex.chunk_rows
    ex.seq += 1
    seq, slot = ex.seq, ex.seq & 1
    cur = torch.cuda.current_stream()
    stage = ex.stage_peer[slot][ex.rank]
    stage[0].copy_(k.reshape(B, S_l, HD))
    stage[1].copy_(v.reshape(B, S_l, HD))
    kv_all = torch.empty((2, B, ex.S_total, HD), dtype=torch.bfloat16, device=k.device)
    # This rank's own chunks go into the gathered buffer on the COMPUTE stream, ahead of the attention launches: a
    # copy inside one device may run as a kernel, and a kernel queued on the side stream is not scheduled while an
    # attention grid that fills every SM spins on exactly that chunk's word (seen as waits that ran out for a rank's
    # own chunk on 4 GPUs, where the grid has 1280 CTAs; the peers' chunks arrive by copy engines over NVLink).
    for j, g in enumerate(chunk_layout(ex.world, ex.rank, ex.method)):
        for b in range(B):
            for t in range(2):
                kv_all[t, b, g * c:(g + 1) * c].copy_(stage[t, b, j * c:(j + 1) * c], non_blocking=True)
            _lib.check(lib.lme_stream_write_words(ex.ready.data_ptr() + 4 * (b * ex.n_chunks + g), 1, seq,
                                                  _lib.stream_ptr()), "lme_stream_write_words")
    ex.side.wait_stream(cur)
    with torch.cuda.stream(ex.side):
        side = _lib.stream_ptr()
        # two staging slots need no "done" handshake: slot seq & 1 was last read by the peers in call seq - 2, and in
        # call seq - 1 this stream waited for every peer's announcement of seq - 1, which a peer makes on the stream
        # that carries its pulls of seq - 2, behind them
        _lib.check(lib.lme_gather_signal(ex._pad_arr, ex.rank, ex.world, seq, side), "lme_gather_signal")
        # The announcement is the only kernel of this stream.  The attention kernel is held back until it has run:
        # an attention grid that filled every SM first and then waited for the peers' chunks would keep this rank's
        # own announcement - which the peers wait for - from ever being scheduled.
        announced = torch.cuda.Event()
        announced.record(ex.side)
        cur.wait_event(announced)
        for i in range(1, ex.world):
            p = (ex.rank + i) % ex.world
            # a stream memory operation, not a kernel: it needs no SM while the attention CTAs hold theirs
            rc = lib.lme_stream_wait_word(ex.pads[ex.rank] + 4 * p, seq, side) if ex.stream_waits else -1
            if rc != _lib.LME_OK:
                ex.stream_waits = False      # not available for this memory: a one-thread bounded wait kernel
                _lib.check(lib.lme_gather_wait_peer(ex.pads[ex.rank], p, seq, side), "lme_gather_wait_peer")
            src = ex.stage_peer[slot][p]
            for j, g in enumerate(chunk_layout(ex.world, p, ex.method)):
                for b in range(B):      # one contiguous copy-engine transfer per (tensor, batch entry, chunk)
                    for t in range(2):
                        kv_all[t, b, g * c:(g + 1) * c].copy_(src[t, b, j * c:(j + 1) * c], non_blocking=True)
                    _lib.check(lib.lme_stream_write_words(ex.ready.data_ptr() + 4 * (b * ex.n_chunks + g), 1, seq,
                                                          side), "lme_stream_write_words")
    if not ex.stream_waits:
        # the peers' announcements are awaited by one-thread KERNELS on the side stream: an attention grid that fills
        # every SM and spins on a chunk would keep such a kernel from ever starting, so without stream memory
        # operations the attention launches wait for the whole exchange (correct, but nothing overlaps)
        cur.wait_stream(ex.side)
    k.record_stream(ex.side)
    v.record_stream(ex.side)
    kv_all.record_stream(ex.side)
    return kv_all, seq


def _runs(ex: _KVExchange) -> list[tuple[int, int, int]]:
    """``(first local row, rows, visible keys)`` of every run of this rank's queries."""
    c = ex.chunk_rows
    return [(j * c, c, (g + 1) * c) for j, g in enumerate(chunk_layout(ex.world, ex.rank, ex.method))]


class _GatheredKVAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, group, method):
        from ..ops.attention_cuda import flash_attention_forward

        ex = _exchange(group, k, method)
        B, S_l, Hq, D = q.shape
        kv_all, seq = _gather_kv(ex, k.contiguous(), v.contiguous())
        K = kv_all[0].view(B, ex.S_total, ex.Hkv, D)
        V = kv_all[1].view(B, ex.S_total, ex.Hkv, D)
        out = torch.empty_like(q)
        lse = torch.empty((B, Hq, S_l), dtype=torch.float32, device=q.device)
        for row0, rows, kv_len in _runs(ex):
            for b in range(B):      # one launch per batch entry: the gathered buffer's batch pitch is S_total
                o, l = flash_attention_forward(q[b:b + 1, row0:row0 + rows], K[b:b + 1, :kv_len], V[b:b + 1, :kv_len],
                                               causal=True, softmax_scale=scale, return_lse=True,
                                               kv_ready=ex.ready[b], kv_chunk_rows=ex.chunk_rows, kv_seq=seq)
                out[b, row0:row0 + rows] = o[0]
                lse[b, :, row0:row0 + rows] = l[0]
        torch.cuda.current_stream().wait_stream(ex.side)
        ctx.save_for_backward(q, kv_all, out, lse)
        ctx.cfg = (scale, ex)
        return out

    @staticmethod
    def backward(ctx, do):
        from ..ops.attention_cuda import flash_attention_backward

        q, kv_all, out, lse = ctx.saved_tensors
        scale, ex = ctx.cfg
        B, S_l, Hq, D = q.shape
        lib = _lib.cuda_lib()
        HD, c = ex.Hkv * D, ex.chunk_rows
        K = kv_all[0].view(B, ex.S_total, ex.Hkv, D)
        V = kv_all[1].view(B, ex.S_total, ex.Hkv, D)
        ex.bwd_calls += 1
        slot = ex.bwd_calls & 1
        grads = ex.grad_peer[slot][ex.rank]          # [2, B, S_total, HD] in symmetric memory
        grads.zero_()                                # key rows that no local query sees contribute nothing
        do = do.contiguous()
        dq = torch.empty_like(q)
        first = True
        for row0, rows, kv_len in _runs(ex):
            for b in range(B):
                dq_r, dk_r, dv_r = flash_attention_backward(
                    do[b:b + 1, row0:row0 + rows], q[b:b + 1, row0:row0 + rows], K[b:b + 1, :kv_len],
                    V[b:b + 1, :kv_len], out[b:b + 1, row0:row0 + rows],
                    lse[b:b + 1, :, row0:row0 + rows].contiguous(), causal=True, softmax_scale=scale)
                dq[b, row0:row0 + rows] = dq_r[0]
                if first:
                    grads[0, b, :kv_len] = dk_r[0].view(kv_len, HD)
                    grads[1, b, :kv_len] = dv_r[0].view(kv_len, HD)
                else:
                    grads[0, b, :kv_len] += dk_r[0].view(kv_len, HD)
                    grads[1, b, :kv_len] += dv_r[0].view(kv_len, HD)
            first = False
        # every rank sums its own chunks of dK / dV over all ranks' partial results (peer loads, fp32, rank order).
        # Two slots: a rank overwrites slot s only two backward calls later, and every reduction below first waits
        # for all peers' announcements, which a peer makes after its reads of the previous reductions.
        dkv = torch.empty((2, B, S_l, HD), dtype=torch.bfloat16, device=q.device)
        n = c * HD
        for t in range(2):
            for b in range(B):
                for j, g in enumerate(chunk_layout(ex.world, ex.rank, ex.method)):
                    srcs = (ctypes.c_void_p * 8)(*([ex.grad_peer[slot][r][t, b, g * c:(g + 1) * c].data_ptr()
                                                    for r in range(ex.world)] + [None] * (8 - ex.world)))
                    ex.rs_seq += 1
                    _lib.check(lib.lme_reduce_scatter_peers(
                        srcs, ex._rs_pad_arr, None, ex.rank, ex.world, ex.rs_seq,
                        dkv[t, b, j * c:(j + 1) * c].data_ptr(), n, 1, 1.0, 0, None, 32, _lib.stream_ptr()),
                        "lme_reduce_scatter_peers")
                    _lib.count_launch()
        Hkv = ex.Hkv
        return dq, dkv[0].view(B, S_l, Hkv, D), dkv[1].view(B, S_l, Hkv, D), None, None, None


def gathered_kv_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, softmax_scale: float | None = None
                          ) -> torch.Tensor:
    """Causal attention over the context-parallel group; q / k / v are this rank's shards ``[B, S / cp, H, 128]``."""
    group = ProcessGroupManager.get_context_parallel_group()
    method = ProcessGroupManager.get_context_parallel_load_balancing_method()
    scale = softmax_scale if softmax_scale is not None else 1 / math.sqrt(q.size(-1))
    return _GatheredKVAttention.apply(q, k, v, scale, group, method)
