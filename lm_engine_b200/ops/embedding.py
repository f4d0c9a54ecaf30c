"""Embedding lookup (optionally the masked lookup of one vocabulary shard) and its gradient on CUDA
(csrc/kernels/rows.cu).  Role of ``F.embedding`` on DTensors in the reference
(lm_engine/modeling_utils/embedding.py:37-92); the gradient is a sort by token id followed by one pass that adds the
rows of every id in a fixed order, so it is deterministic."""

from __future__ import annotations

import torch
import torch.nn.functional as F


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, lo: int, hi: int):
        from . import _lib

        flat = ids.reshape(-1).to(torch.int64).contiguous()
        H = weight.size(1)
        out = torch.empty((flat.numel(), H), dtype=weight.dtype, device=weight.device)
        _lib.check(_lib.cuda_lib().lme_embedding_fwd(flat.data_ptr(), weight.data_ptr(), out.data_ptr(), flat.numel(),
                                                     H, lo, hi, _lib.stream_ptr()), f"lme_embedding_fwd H={H}")
        _lib.count_launch()
        ctx.save_for_backward(flat)
        ctx.meta = (weight.size(0), lo, hi)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dy):
        from . import _lib

        (flat,) = ctx.saved_tensors
        rows, lo, hi = ctx.meta
        H = dy.size(-1)
        dy = dy.reshape(-1, H).contiguous()
        sorted_ids, order = torch.sort(flat)
        dW = torch.zeros((rows, H), dtype=dy.dtype, device=dy.device)
        _lib.check(_lib.cuda_lib().lme_embedding_bwd(sorted_ids.data_ptr(), order.data_ptr(), dy.data_ptr(),
                                                     dW.data_ptr(), flat.numel(), H, lo, hi, _lib.stream_ptr()),
                   f"lme_embedding_bwd H={H}")
        _lib.count_launch()
        return None, dW, None, None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0, vocab_end: int | None = None):
    """``weight[ids - vocab_start]`` with zeros for ids outside ``[vocab_start, vocab_end)``."""
    hi = vocab_start + weight.size(0) if vocab_end is None else vocab_end
    if (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.is_contiguous() and weight.size(1) % 8 == 0
            and ids.numel() > 0):
        return _Embedding.apply(ids, weight, vocab_start, hi)
    inside = (ids >= vocab_start) & (ids < hi)
    x = F.embedding((ids - vocab_start).masked_fill(~inside, 0), weight)
    return x if bool(inside.all()) else x * inside.unsqueeze(-1).to(weight.dtype)
