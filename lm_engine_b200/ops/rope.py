"""Fused split of the per-KV-group interleaved QKV projection + NeoX rotary embedding.

The fused projection's output is laid out per KV head as ``[q_0 .. q_{G-1} | k | v]`` (each ``D`` wide), the
checkpoint-visible convention of the reference (lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/
module.py:174-196); RoPE rotates the **last** ``rope_dim`` channels of every q / k head with fp32 math
(lm_engine/modeling_utils/position_embedding/rope.py:15-171).  One kernel reads the packed tensor once and writes
contiguous ``q [.., Hq, D]``, ``k``, ``v [.., Hkv, D]``; the backward kernel is the inverse rotation + re-pack.
"""

from __future__ import annotations

import torch

from . import _lib


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = torch.chunk(x, 2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., T-like dims, heads, D]; cos/sin broadcastable [..., 1, rope_dim] (fp32)."""
    rd = cos.size(-1)
    D = x.size(-1)
    xf = x.float()
    if rd == D:
        return (xf * cos + rotate_half(xf) * sin).to(x.dtype)
    nope, rope = xf[..., : D - rd], xf[..., D - rd:]
    rope = rope * cos + rotate_half(rope) * sin
    return torch.cat((nope, rope), dim=-1).to(x.dtype)


def qkv_split_rope_reference(qkv, Hkv, G, D, cos, sin):
    """qkv [..., Hkv*(G+2)*D] -> q [..., Hkv*G, D], k [..., Hkv, D], v [..., Hkv, D]; cos/sin [..., rope_dim] or None."""
    lead = qkv.shape[:-1]
    x = qkv.view(*lead, Hkv, (G + 2) * D)
    q, k, v = torch.split(x, (G * D, D, D), dim=-1)
    q = q.reshape(*lead, Hkv * G, D)
    if cos is not None:
        c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
        q = apply_rope_reference(q, c, s)
        k = apply_rope_reference(k, c, s)
    return q, k.contiguous(), v.contiguous()


class _QKVRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos_table, sin_table, positions, S, Hkv, G, D, rope_dim):
        lead = qkv.shape[:-1]
        x = qkv.reshape(-1, qkv.size(-1)).contiguous()
        T = x.size(0)
        max_pos = cos_table.size(0) if cos_table is not None else 0
        if positions is not None and positions.numel() != T:
            raise ValueError(f"qkv_split_rope: {positions.numel()} positions for {T} tokens")
        q = torch.empty((T, Hkv * G, D), dtype=x.dtype, device=x.device)
        k = torch.empty((T, Hkv, D), dtype=x.dtype, device=x.device)
        v = torch.empty((T, Hkv, D), dtype=x.dtype, device=x.device)
        _lib.check(_lib.cuda_lib().lme_qkv_rope(x.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                _lib.ptr(cos_table), _lib.ptr(sin_table), _lib.ptr(positions), T, S,
                                                Hkv, G, D, rope_dim, max_pos, 0, _lib.stream_ptr()), "lme_qkv_rope")
        _lib.count_launch()
        ctx.tables = (cos_table, sin_table, positions)
        ctx.dims = (T, S, Hkv, G, D, rope_dim, max_pos)
        ctx.in_shape = qkv.shape
        return q.view(*lead, Hkv * G, D), k.view(*lead, Hkv, D), v.view(*lead, Hkv, D)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        T, S, Hkv, G, D, rope_dim, max_pos = ctx.dims
        cos_table, sin_table, positions = ctx.tables
        dq, dk, dv = dq.contiguous(), dk.contiguous(), dv.contiguous()
        dqkv = torch.empty((T, Hkv * (G + 2) * D), dtype=dq.dtype, device=dq.device)
        _lib.check(_lib.cuda_lib().lme_qkv_rope(dqkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                                _lib.ptr(cos_table), _lib.ptr(sin_table), _lib.ptr(positions), T, S,
                                                Hkv, G, D, rope_dim, max_pos, 1, _lib.stream_ptr()),
                   "lme_qkv_rope(inverse)")
        _lib.count_launch()
        return dqkv.view(ctx.in_shape), None, None, None, None, None, None, None, None


def qkv_split_rope(qkv: torch.Tensor, Hkv: int, G: int, D: int, cos_table: torch.Tensor | None,
                   sin_table: torch.Tensor | None, position_ids: torch.Tensor | None, seq_len: int):
    """``cos_table/sin_table``: fp32 ``[max_pos, rope_dim]``; ``position_ids``: flattened like ``qkv``'s leading dims
    (or None: position = token index modulo ``seq_len``)."""
    rope_dim = 0 if cos_table is None else cos_table.size(-1)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and D % 8 == 0 and rope_dim % 16 == 0:
        pos = None
        if position_ids is not None:
            lead = qkv.shape[:-1]
            if position_ids.dim() == len(lead) and tuple(position_ids.shape) != tuple(lead):
                position_ids = position_ids.expand(lead)   # [1, S] positions shared by the whole batch
            pos = position_ids.reshape(-1).to(torch.int32).contiguous()
        return _QKVRope.apply(qkv, cos_table, sin_table, pos, seq_len, Hkv, G, D, rope_dim)
    cos = sin = None
    if cos_table is not None:
        lead = qkv.shape[:-1]
        if position_ids is None:
            n = 1
            for d in lead:
                n *= d
            position_ids = (torch.arange(n, device=qkv.device) % seq_len).view(lead)
        cos, sin = cos_table[position_ids.view(lead)], sin_table[position_ids.view(lead)]
    return qkv_split_rope_reference(qkv, Hkv, G, D, cos, sin)
