"""Context-parallel attention by head exchange ("Ulysses").

Each rank holds ``S / cp`` tokens of every head.  One all-to-all turns that into all ``S`` tokens of ``H / cp`` heads,
attention runs locally over the full sequence with the single-device kernel, and a second all-to-all returns the
output to the sequence-sharded layout.  Compared with the ring (ring_attention.py in this package, which plays the
role of lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/ring_attention.py:41-538) this moves
``(Hq + 2 Hkv + Hq) / cp`` head-slices per token instead of ``2 Hkv (cp - 1)`` and needs no partial-softmax merging,
at the price of requiring ``Hq % cp == 0``.  Over NVSwitch the all-to-all runs at full per-GPU bandwidth, so this is
the default whenever the head counts allow it.

Head-tail load-balanced sharding (context_parallel.py) stores the sequence in a permuted order; the exchange undoes
the permutation before attention and re-applies it afterwards, so causal masking sees natural positions.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .context_parallel import shard_indices
from .manager import ProcessGroupManager


def _all_to_all_equal(x: torch.Tensor, group) -> torch.Tensor:
    """``x [world, ...]``: slice j goes to rank j; returns ``[world, ...]`` with slice j received from rank j."""
    x = x.contiguous()
    out = torch.empty_like(x)
    if x.is_cuda:
        dist.all_to_all_single(out, x, group=group)
        return out
    # gloo has no all_to_all_single: gather everything and keep this rank's column
    world, r = dist.get_world_size(group), dist.get_rank(group)
    gathered = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(gathered, x, group=group)
    for src in range(world):
        out[src] = gathered[src][r]
    return out


class _SeqToHeads(torch.autograd.Function):
    """``[B, s, H, D]`` (local tokens, all heads) -> ``[B, cp * s, H / cp, D]`` (rank-major token order)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        cp = dist.get_world_size(group)
        B, s, H, D = x.shape
        send = x.reshape(B, s, cp, H // cp, D).permute(2, 0, 1, 3, 4)
        got = _all_to_all_equal(send, group)                      # [cp(src), B, s, h, D]
        return got.permute(1, 0, 2, 3, 4).reshape(B, cp * s, H // cp, D)

    @staticmethod
    def backward(ctx, g):
        return _HeadsToSeq.apply(g, ctx.group), None


class _HeadsToSeq(torch.autograd.Function):
    """Inverse of :class:`_SeqToHeads`."""

    @staticmethod
    def forward(ctx, y, group):
        ctx.group = group
        cp = dist.get_world_size(group)
        B, S, h, D = y.shape
        s = S // cp
        send = y.reshape(B, cp, s, h, D).permute(1, 0, 2, 3, 4)
        got = _all_to_all_equal(send, group)                      # [cp(head group), B, s, h, D]
        return got.permute(1, 2, 0, 3, 4).reshape(B, s, cp * h, D)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads.apply(g, ctx.group), None


def ulysses_eligible(num_q_heads: int, num_kv_heads: int, cp: int) -> bool:
    """The query heads must split evenly; K/V heads are replicated up to a multiple of ``cp`` when the GQA group
    size allows it."""
    if num_q_heads % cp:
        return False
    f = cp // math.gcd(num_kv_heads, cp)
    return (num_q_heads // num_kv_heads) % f == 0


def _natural_order(seq_len: int, cp: int, method, device) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """(to_natural, to_sharded) index vectors for the rank-major concatenation, or (None, None) when it already is
    the natural order."""
    if method is None:
        return None, None
    concat = torch.cat([shard_indices(seq_len, cp, j, method, device=device) for j in range(cp)])
    if bool((concat == torch.arange(seq_len, device=device)).all()):
        return None, None
    return torch.argsort(concat), concat


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
                      softmax_scale: float | None = None, sliding_window: int | None = None,
                      dropout_p: float = 0.0) -> torch.Tensor:
    """q ``[B, S/cp, Hq, D]``, k/v ``[B, S/cp, Hkv, D]`` are this rank's sequence shards; returns ``[B, S/cp, Hq, D]``."""
    from ..ops import attention

    group = ProcessGroupManager.get_context_parallel_group()
    scale = softmax_scale if softmax_scale is not None else 1 / math.sqrt(q.size(-1))
    if group is None:
        return attention(q, k, v, causal=causal, softmax_scale=scale, sliding_window=sliding_window,
                         dropout_p=dropout_p)
    cp = dist.get_world_size(group)
    Hq, Hkv = q.size(2), k.size(2)
    assert ulysses_eligible(Hq, Hkv, cp), f"cannot split {Hq} query / {Hkv} key-value heads over {cp} ranks"
    f = cp // math.gcd(Hkv, cp)
    if f > 1:
        k = k.repeat_interleave(f, dim=2)
        v = v.repeat_interleave(f, dim=2)
        Hkv *= f
    B, s, _, D = q.shape
    hq, hkv = Hq // cp, Hkv // cp
    # one exchange for q, k and v: heads of destination j are laid side by side
    packed = torch.cat((q.reshape(B, s, cp, hq, D), k.reshape(B, s, cp, hkv, D), v.reshape(B, s, cp, hkv, D)),
                       dim=3).reshape(B, s, cp * (hq + 2 * hkv), D)
    full = _SeqToHeads.apply(packed, group)                       # [B, S, hq + 2 hkv, D]
    method = ProcessGroupManager.get_context_parallel_load_balancing_method()
    to_natural, to_sharded = _natural_order(s * cp, cp, method, q.device)
    if to_natural is not None:
        full = full.index_select(1, to_natural)
    qf, kf, vf = full.split((hq, hkv, hkv), dim=2)
    out = attention(qf.contiguous(), kf.contiguous(), vf.contiguous(), causal=causal, softmax_scale=scale,
                    sliding_window=sliding_window, dropout_p=dropout_p)
    if to_sharded is not None:
        out = out.index_select(1, to_sharded)
    return _HeadsToSeq.apply(out, group)
