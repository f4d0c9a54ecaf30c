"""Sequence packing: left-padded ``[B, S, ...]`` batches <-> packed ``[T, ...]`` token streams described by
``cu_seqlens`` (role of lm_engine/modeling_utils/sequence_packing.py:18-93).

The valid tokens of row ``b`` are its last ``cu_seqlens[b + 1] - cu_seqlens[b]`` positions.  The gather / scatter
index of every packed token is computed on the device from ``cu_seqlens`` with one ``searchsorted`` (no per-row loop,
no host synchronisation when the total token count is given), so both directions are single indexed copies and
differentiable.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def compute_cu_seqlens_and_max_seqlen_from_attention_mask(attention_mask: torch.Tensor) -> tuple[torch.Tensor, int]:
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    cu_seqlens = F.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    return cu_seqlens, int(seqlens.max())


def _flat_index(cu_seqlens: torch.Tensor, S: int, total: int | None) -> torch.Tensor:
    """Flat position ``b * S + s`` of every packed token inside the padded ``[B, S]`` grid."""
    cu = cu_seqlens.to(torch.int64)
    if total is None:
        total = int(cu[-1])
    t = torch.arange(total, device=cu.device)
    b = torch.searchsorted(cu[1:], t, right=True)
    lens = cu[1:] - cu[:-1]
    return b * S + (S - lens[b]) + (t - cu[b])


def _row_kernels_apply(x: torch.Tensor, row_shape) -> bool:
    row_bytes = x.element_size()
    for d in row_shape:
        row_bytes *= d
    return x.is_cuda and len(row_shape) > 0 and row_bytes % 16 == 0 and x.numel() > 0


class _PackRows(torch.autograd.Function):
    """CUDA path (csrc/kernels/rows.cu): one vectorised copy kernel per direction; each is the other's gradient."""

    @staticmethod
    def forward(ctx, x, cu_seqlens, total: int):
        from . import _lib

        x = x.contiguous()
        B, S = x.shape[:2]
        cu = cu_seqlens.to(torch.int32).contiguous()
        out = torch.empty((total, *x.shape[2:]), dtype=x.dtype, device=x.device)
        row_bytes = x[0, 0].numel() * x.element_size()
        if total > 0:
            _lib.check(_lib.cuda_lib().lme_pack_rows(x.data_ptr(), cu.data_ptr(), out.data_ptr(), B, S, total,
                                                     row_bytes, _lib.stream_ptr()), "lme_pack_rows")
            _lib.count_launch()
        ctx.save_for_backward(cu)
        ctx.shape = tuple(x.shape)
        return out

    @staticmethod
    def backward(ctx, g):
        (cu,) = ctx.saved_tensors
        return _UnpackRows.apply(g, cu, ctx.shape), None, None


class _UnpackRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, cu_seqlens, output_shape):
        from . import _lib

        packed = packed.contiguous()
        B, S = output_shape[:2]
        cu = cu_seqlens.to(torch.int32).contiguous()
        out = torch.empty(tuple(output_shape), dtype=packed.dtype, device=packed.device)
        row_bytes = out[0, 0].numel() * out.element_size()
        _lib.check(_lib.cuda_lib().lme_unpack_rows(packed.data_ptr(), cu.data_ptr(), out.data_ptr(), B, S, row_bytes,
                                                   _lib.stream_ptr()), "lme_unpack_rows")
        _lib.count_launch()
        ctx.save_for_backward(cu)
        ctx.total = packed.size(0)
        return out

    @staticmethod
    def backward(ctx, g):
        (cu,) = ctx.saved_tensors
        return _PackRows.apply(g, cu, ctx.total), None, None


def pack_sequence(inputs, cu_seqlens: torch.Tensor, total_tokens: int | None = None):
    single = isinstance(inputs, torch.Tensor)
    xs = [inputs] if single else list(inputs)
    out = []
    for x in xs:
        assert x.dim() >= 2 and x.size(0) == cu_seqlens.numel() - 1
        if _row_kernels_apply(x, x.shape[2:]):
            total = int(cu_seqlens[-1]) if total_tokens is None else total_tokens
            out.append(_PackRows.apply(x, cu_seqlens, total))
            continue
        idx = _flat_index(cu_seqlens, x.size(1), total_tokens)
        out.append(x.reshape(x.size(0) * x.size(1), *x.shape[2:]).index_select(0, idx))
    return out[0] if single else out


def unpack_sequence(inputs, cu_seqlens: torch.Tensor, output_shape: tuple[int, ...]):
    single = isinstance(inputs, torch.Tensor)
    xs = [inputs] if single else list(inputs)
    B, S = output_shape[:2]
    assert cu_seqlens.numel() - 1 == B
    out = []
    for x in xs:
        if _row_kernels_apply(x, output_shape[2:]):
            out.append(_UnpackRows.apply(x, cu_seqlens, tuple(output_shape)))
            continue
        idx = _flat_index(cu_seqlens, S, x.size(0))
        flat = torch.zeros((B * S, *output_shape[2:]), dtype=x.dtype, device=x.device)
        out.append(flat.index_copy(0, idx, x).view(*output_shape))
    return out[0] if single else out
