"""Context-parallel ring attention.

Every rank keeps its query shard and passes its K/V shard around the ``cp`` ring; partial results are merged with
their log-sum-exp in fp32, so the result equals single-device attention over the full sequence.  The backward pass
rotates K/V together with fp32 dK/dV accumulators so each gradient block ends up on its owner.  Masking is driven by
global token positions, which makes contiguous and head-tail sharding (and sliding windows) the same code path;
blocks that a causal mask would zero entirely are skipped.

Role of lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/ring_attention.py:41-538 (which wraps
flash-attn kernels in a Python ring over all-to-all); here the per-block math is the tcgen05 attention kernels
(:func:`kernel_block_forward` / :func:`kernel_block_backward`, one launch per pair of position runs) when the block
decomposes into whole runs of 128-row multiples, else the PyTorch statements :func:`block_attention_forward` /
:func:`block_attention_backward`.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .context_parallel import shard_indices
from .manager import ProcessGroupManager


def _mask(qpos: torch.Tensor, kpos: torch.Tensor, causal: bool, window: int | None) -> torch.Tensor | None:
    if not causal and window is None:
        return None
    qi, kj = qpos[:, None], kpos[None, :]
    m = torch.ones(qpos.numel(), kpos.numel(), dtype=torch.bool, device=qpos.device)
    if causal:
        m &= kj <= qi
        if window is not None:
            m &= kj > qi - window
    elif window is not None:
        m &= (kj - qi).abs() < window
    return m


def block_attention_forward(q, k, v, qpos, kpos, scale, causal, window):
    """One (query shard, key shard) block.  q ``[B, Sq, Hq, D]``, k/v ``[B, Sk, Hkv, D]``.
    Returns fp32 ``out [B, Sq, Hq, D]`` normalised within the block and ``lse [B, Sq, Hq]`` (-inf rows allowed)."""
    G = q.size(2) // k.size(2)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(G, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(G, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    m = _mask(qpos, kpos, causal, window)
    if m is not None:
        s = s.masked_fill(~m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    out = torch.matmul(p, vf)
    return out.transpose(1, 2), lse.transpose(1, 2)


def block_attention_backward(do, q, k, v, out, lse, qpos, kpos, scale, causal, window):
    """Gradients of one block given the **global** ``out`` / ``lse`` (fp32).  Returns fp32 ``dq, dk, dv``."""
    Hq, Hkv = q.size(2), k.size(2)
    G = Hq // Hkv
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(G, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(G, dim=1)
    dof = do.float().transpose(1, 2)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    m = _mask(qpos, kpos, causal, window)
    if m is not None:
        s = s.masked_fill(~m, float("-inf"))
    l = lse.transpose(1, 2)
    p = torch.exp(s - torch.where(torch.isinf(l), torch.zeros_like(l), l)[..., None])
    p = torch.where(torch.isinf(l)[..., None], torch.zeros_like(p), p)
    delta = (dof * out.float().transpose(1, 2)).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    B, _, Sk, D = dk.shape
    dk = dk.view(B, Hkv, G, Sk, D).sum(2)
    dv = dv.view(B, Hkv, G, Sk, D).sum(2)
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)


def merge_partial(out, lse, out_b, lse_b):
    """Combines two partial softmax results (fp32).  ``new = logaddexp(lse, lse_b)``."""
    if out is None:
        return out_b, lse_b
    new = torch.logaddexp(lse, lse_b)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    wa = torch.exp(lse - safe)[..., None]
    wb = torch.exp(lse_b - safe)[..., None]
    wa = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(wa), wa)
    wb = torch.where(torch.isinf(lse_b)[..., None], torch.zeros_like(wb), wb)
    return out * wa + out_b * wb, new


def _block_needed(qpos, kpos, causal, window) -> bool:
    if not causal:
        return True
    if int(kpos.min()) > int(qpos.max()):
        return False
    if window is not None and int(kpos.max()) <= int(qpos.min()) - window:
        return False
    return True


def shard_runs(seq_len: int, cp: int, rank: int, method) -> list[tuple[int, int]]:
    """The shard of ``rank`` as (first position, length) runs, in shard order: one run for contiguous sharding,
    two for head-tail (host-side twin of :func:`shard_indices`)."""
    from ..enums import ContextParallelLoadBalancerMethod

    if method == ContextParallelLoadBalancerMethod.headtail:
        c = seq_len // (2 * cp)
        return [(rank * c, c), ((2 * cp - 1 - rank) * c, c)]
    c = seq_len // cp
    return [(rank * c, c)]


def _relation(qrun: tuple[int, int], krun: tuple[int, int], causal: bool) -> str | None:
    """How a run of keys relates to a run of queries: every key visible, the causal diagonal, nothing visible, or
    ``None`` for a partial overlap the kernels have no mask for."""
    if not causal:
        return "full"
    (qs, ql), (ks, kl) = qrun, krun
    if ks + kl - 1 <= qs:
        return "full"
    if ks == qs and kl == ql:
        return "causal"
    if ks > qs + ql - 1:
        return "skip"
    return None


def kernel_blocks_usable(q: torch.Tensor, k: torch.Tensor, qruns, kruns, causal: bool, window) -> bool:
    """The tcgen05 attention kernels (ops/attention_cuda.py) serve a block when it decomposes into whole runs."""
    from ..ops import attention_cuda

    if window is not None or not q.is_cuda or q.dtype != torch.bfloat16 or q.size(-1) != 128:
        return False
    if any(length % 128 for _, length in list(qruns) + list(kruns)):
        return False
    if any(_relation(a, b, causal) is None for a in qruns for b in kruns):
        return False
    return attention_cuda.shapes_supported(q[:, :128], k[:, :128], k[:, :128])


def kernel_block_forward(q, k, v, qruns, kruns, scale, causal):
    """:func:`block_attention_forward` on the attention kernels: one launch per (query run, key run) pair that has
    visible keys, merged per query run by their log-sum-exps."""
    from ..ops.attention_cuda import flash_attention_forward

    B, Sq, Hq, D = q.shape
    out = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    lse = torch.full((B, Sq, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    qo = 0
    for qrun in qruns:
        o_run = l_run = None
        ko = 0
        for krun in kruns:
            rel = _relation(qrun, krun, causal)
            if rel != "skip":
                o_b, l_b = flash_attention_forward(q[:, qo:qo + qrun[1]], k[:, ko:ko + krun[1]], v[:, ko:ko + krun[1]],
                                                   causal=rel == "causal", softmax_scale=scale, return_lse=True)
                o_run, l_run = merge_partial(o_run, l_run, o_b.float(), l_b.transpose(1, 2))
            ko += krun[1]
        if o_run is not None:
            out[:, qo:qo + qrun[1]] = o_run
            lse[:, qo:qo + qrun[1]] = l_run
        qo += qrun[1]
    return out, lse


def kernel_block_backward(do, q, k, v, out, lse, qruns, kruns, scale, causal):
    """:func:`block_attention_backward` on the attention kernels (global ``out`` / ``lse``)."""
    from ..ops.attention_cuda import flash_attention_backward

    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    do16, out16 = do.to(q.dtype), out.to(q.dtype)
    qo = 0
    for qrun in qruns:
        qs = slice(qo, qo + qrun[1])
        l_run = lse[:, qs].transpose(1, 2).contiguous()
        ko = 0
        for krun in kruns:
            rel = _relation(qrun, krun, causal)
            ks = slice(ko, ko + krun[1])
            if rel != "skip":
                dq_b, dk_b, dv_b = flash_attention_backward(do16[:, qs], q[:, qs], k[:, ks], v[:, ks], out16[:, qs],
                                                            l_run, causal=rel == "causal", softmax_scale=scale)
                dq[:, qs] += dq_b
                dk[:, ks] += dk_b
                dv[:, ks] += dv_b
            ko += krun[1]
        qo += qrun[1]
    return dq, dk, dv


def _rotate(t: torch.Tensor, group, shift: int = 1) -> tuple[torch.Tensor, list]:
    """Starts sending ``t`` to rank+shift and receiving from rank-shift; returns (recv buffer, work handles)."""
    world, r = dist.get_world_size(group), dist.get_rank(group)
    ranks = dist.get_process_group_ranks(group)
    recv = torch.empty_like(t)
    ops = [dist.P2POp(dist.isend, t.contiguous(), ranks[(r + shift) % world], group),
           dist.P2POp(dist.irecv, recv, ranks[(r - shift) % world], group)]
    return recv, dist.batch_isend_irecv(ops)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, group, method, seq_len):
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        pos = [shard_indices(seq_len, cp, j, method, device=q.device) for j in range(cp)]
        runs = [shard_runs(seq_len, cp, j, method) for j in range(cp)]
        out = lse = None
        kv = torch.stack((k, v)).contiguous()
        for step in range(cp):
            nxt = works = None
            if step < cp - 1:
                nxt, works = _rotate(kv, group)
            src = (r - step) % cp
            if kernel_blocks_usable(q, kv[0], runs[r], runs[src], causal, window):
                if any(_relation(a, b, causal) != "skip" for a in runs[r] for b in runs[src]):
                    o_b, l_b = kernel_block_forward(q, kv[0], kv[1], runs[r], runs[src], scale, causal)
                    out, lse = merge_partial(out, lse, o_b, l_b)
            elif _block_needed(pos[r], pos[src], causal, window):
                if q.is_cuda:
                    from ..logging_utils.logger import warn_once

                    warn_once("ring-attention-pytorch-block", "ring attention: a block is windowed, not bf16 with "
                              "head dim 128, or not made of 128-row runs; it runs as a PyTorch statement that "
                              "materialises its fp32 score matrix")
                o_b, l_b = block_attention_forward(q, kv[0], kv[1], pos[r], pos[src], scale, causal, window)
                out, lse = merge_partial(out, lse, o_b, l_b)
            if works is not None:
                for w in works:
                    w.wait()
                kv = nxt
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (scale, causal, window, group, method, seq_len)
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        scale, causal, window, group, method, seq_len = ctx.cfg
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        pos = [shard_indices(seq_len, cp, j, method, device=q.device) for j in range(cp)]
        runs = [shard_runs(seq_len, cp, j, method) for j in range(cp)]
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)
        dkv_works = None        # rotation of the dK / dV accumulators started in the previous step
        for step in range(cp):
            src = (r - step) % cp
            nxt_kv = works = None
            if step < cp - 1:
                nxt_kv, works = _rotate(kv, group)
            blk = None
            if kernel_blocks_usable(q, kv[0], runs[r], runs[src], causal, window):
                if any(_relation(a, b, causal) != "skip" for a in runs[r] for b in runs[src]):
                    blk = kernel_block_backward(do, q, kv[0], kv[1], out, lse, runs[r], runs[src], scale, causal)
            elif _block_needed(pos[r], pos[src], causal, window):
                blk = block_attention_backward(do, q, kv[0], kv[1], out, lse, pos[r], pos[src], scale, causal, window)
            # the accumulators of the previous step were sent on while this block was computed (the reference
            # awaits its dK / dV rotation after the block as well, ring_attention.py:202-434)
            if dkv_works is not None:
                for w in dkv_works:
                    w.wait()
            if blk is not None:
                dq += blk[0]
                dkv[0] += blk[1]
                dkv[1] += blk[2]
            if works is not None:
                for w in works:
                    w.wait()
                kv = nxt_kv
            # the accumulators travel with their K/V block; after cp hops they are back at the owner
            dkv, dkv_works = _rotate(dkv, group)
        for w in dkv_works:
            w.wait()
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None, None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
                   softmax_scale: float | None = None, sliding_window: int | None = None) -> torch.Tensor:
    """q/k/v are this rank's context-parallel shards ``[B, S/cp, H, D]``; returns the local output shard."""
    group = ProcessGroupManager.get_context_parallel_group()
    scale = softmax_scale if softmax_scale is not None else 1 / math.sqrt(q.size(-1))
    if group is None:
        from ..ops import attention

        return attention(q, k, v, causal=causal, softmax_scale=scale, sliding_window=sliding_window)
    cp = dist.get_world_size(group)
    method = ProcessGroupManager.get_context_parallel_load_balancing_method()
    return _RingAttention.apply(q, k, v, scale, causal, sliding_window, group, method, q.size(1) * cp)
