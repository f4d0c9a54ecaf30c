"""SwiGLU on the packed interleaved layout: ``y = x[..., 1::2] * silu(x[..., ::2])``.

Same layout as the reference's GLU activations (lm_engine/modeling_utils/activations/glu.py:52-59): gate at even
columns, up-projection at odd columns, which is what lets the GEMM epilogue fuse the activation (each accumulator
row holds adjacent gate/up pairs).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


def swiglu_packed_reference(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return (xf[..., 1::2] * F.silu(xf[..., ::2])).to(x.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        I2 = x.size(-1)
        x2 = x.reshape(-1, I2).contiguous()
        y = torch.empty((x2.size(0), I2 // 2), dtype=x.dtype, device=x.device)
        _lib.check(_lib.cuda_lib().lme_swiglu_fwd(x2.data_ptr(), y.data_ptr(), x2.size(0), I2 // 2,
                                                  _lib.stream_ptr()), "lme_swiglu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], I2 // 2)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        dy2 = dy.reshape(x2.size(0), -1).contiguous()
        dx = torch.empty_like(x2)
        _lib.check(_lib.cuda_lib().lme_swiglu_bwd(x2.data_ptr(), dy2.data_ptr(), dx.data_ptr(), x2.size(0),
                                                  dy2.size(1), _lib.stream_ptr()), "lme_swiglu_bwd")
        _lib.count_launch()
        return dx.view(ctx.shape)


def swiglu_packed(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.size(-1) % 16 == 0:
        return _SwiGLU.apply(x)
    return swiglu_packed_reference(x)


def swiglu_backward(preact: torch.Tensor, dy: torch.Tensor, tile_group: torch.Tensor | None = None) -> torch.Tensor:
    """d(preact) given the packed pre-activation and d(out) (used by the fused MLP op).  ``tile_group`` (int32, one
    entry per 128 rows): only tiles with an entry >= 0 are read and written (the grouped GEMMs' padded layout)."""
    if preact.is_cuda and preact.dtype == torch.bfloat16:
        p2 = preact.reshape(-1, preact.size(-1))
        d2 = dy.reshape(p2.size(0), -1).contiguous()
        dx = torch.empty_like(p2)
        if tile_group is not None and p2.size(0) == tile_group.numel() * 128:
            _lib.check(_lib.cuda_lib().lme_swiglu_bwd_tiles(p2.data_ptr(), d2.data_ptr(), dx.data_ptr(), p2.size(0),
                                                            d2.size(1), tile_group.data_ptr(), _lib.stream_ptr()),
                       "lme_swiglu_bwd_tiles")
            _lib.count_launch()
            return dx.view(preact.shape)
        _lib.check(_lib.cuda_lib().lme_swiglu_bwd(p2.data_ptr(), d2.data_ptr(), dx.data_ptr(), p2.size(0),
                                                  d2.size(1), _lib.stream_ptr()), "lme_swiglu_bwd")
        _lib.count_launch()
        return dx.view(preact.shape)
    g = preact[..., ::2].float()
    u = preact[..., 1::2].float()
    s = torch.sigmoid(g)
    d = dy.float()
    out = torch.empty_like(preact, dtype=torch.float32)
    out[..., ::2] = d * u * s * (1 + g * (1 - s))
    out[..., 1::2] = d * g * s
    return out.to(preact.dtype)
