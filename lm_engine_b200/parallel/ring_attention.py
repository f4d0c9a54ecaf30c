"""Context-parallel ring attention.

Every rank keeps its query shard and passes its K/V shard around the ``cp`` ring; partial results are merged with
their log-sum-exp in fp32, so the result equals single-device attention over the full sequence.  The backward pass
rotates K/V together with fp32 dK/dV accumulators so each gradient block ends up on its owner.  Masking is driven by
global token positions, which makes contiguous and head-tail sharding (and sliding windows) the same code path;
blocks that a causal mask would zero entirely are skipped.

Role of lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/ring_attention.py:41-538 (which wraps
flash-attn kernels in a Python ring over all-to-all); here the per-block math is
:func:`block_attention_forward` / :func:`block_attention_backward`.
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
        out = lse = None
        kv = torch.stack((k, v)).contiguous()
        for step in range(cp):
            nxt = works = None
            if step < cp - 1:
                nxt, works = _rotate(kv, group)
            src = (r - step) % cp
            if _block_needed(pos[r], pos[src], causal, window):
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
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)
        for step in range(cp):
            src = (r - step) % cp
            nxt_kv = works = None
            if step < cp - 1:
                nxt_kv, works = _rotate(kv, group)
            if _block_needed(pos[r], pos[src], causal, window):
                dq_b, dk_b, dv_b = block_attention_backward(do, q, kv[0], kv[1], out, lse, pos[r], pos[src], scale,
                                                            causal, window)
                dq += dq_b
                dkv[0] += dk_b
                dkv[1] += dv_b
            if works is not None:
                for w in works:
                    w.wait()
                kv = nxt_kv
            # the accumulators travel with their K/V block; after cp hops they are back at the owner
            dkv, w2 = _rotate(dkv, group)
            for w in w2:
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
