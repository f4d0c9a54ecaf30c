"""RMSNorm with an optional fused residual add (forward) and fused residual-gradient add (backward).

Counterpart of the reference's ``nn.RMSNorm`` / ``rmsnorm`` kernels (lm_engine/modeling_utils/normalization.py:64-124).
The backward kernel reduces the weight gradient through an fp32 scratch of per-CTA partial sums.
"""

from __future__ import annotations

import torch

from . import _lib


def rmsnorm_reference(x, weight, eps, residual=None):
    h = x if residual is None else x + residual
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype), h


def _use_kernel(x: torch.Tensor, weight: torch.Tensor | None) -> bool:
    H = x.size(-1)
    return (x.is_cuda and x.dtype == torch.bfloat16 and H % 8 == 0 and H <= 16384
            and (weight is None or weight.dtype == torch.bfloat16))


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        H = x.size(-1)
        x2 = x.reshape(-1, H).contiguous()
        r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
        T = x2.size(0)
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if r2 is not None else None
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        w = weight.contiguous() if weight is not None else None
        _lib.check(_lib.cuda_lib().lme_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(r2), _lib.ptr(w), y.data_ptr(),
                                                   _lib.ptr(h), rstd.data_ptr(), T, H, eps, _lib.stream_ptr()),
                   "lme_rmsnorm_fwd")
        _lib.count_launch()
        hs = h if h is not None else x2
        ctx.save_for_backward(hs, w if w is not None else torch.empty(0, device=x.device), rstd)
        ctx.has_w = w is not None
        ctx.has_res = r2 is not None
        ctx.shape = x.shape
        ctx.mark_non_differentiable(rstd)
        if h is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        hs, w, rstd = ctx.saved_tensors
        T, H = hs.shape
        dy2 = dy.reshape(T, H).contiguous()
        dh2 = dh.reshape(T, H).contiguous() if dh is not None else None
        dx = torch.empty_like(hs)
        lib = _lib.cuda_lib()
        dw = partial = None
        weight = None
        if ctx.has_w:
            rows = lib.lme_rmsnorm_bwd_partial_rows(T)
            partial = torch.empty((rows, H), dtype=torch.float32, device=hs.device)
            dw = torch.empty(H, dtype=torch.float32, device=hs.device)
            weight = w
        _lib.check(lib.lme_rmsnorm_bwd(dy2.data_ptr(), hs.data_ptr(), _lib.ptr(weight), rstd.data_ptr(),
                                       _lib.ptr(dh2), dx.data_ptr(), _lib.ptr(partial), _lib.ptr(dw), 0, T, H,
                                       _lib.stream_ptr()), "lme_rmsnorm_bwd")
        _lib.count_launch(2 if ctx.has_w else 1)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), (dw.to(w.dtype) if ctx.has_w else None), None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float,
            residual: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(rmsnorm(x + residual) * weight, x + residual)`` (second element is ``x`` when no residual)."""
    if _use_kernel(x, weight):
        y, h = _RMSNorm.apply(x, residual, weight, eps)
        return y, (h if residual is not None else x)
    return rmsnorm_reference(x, weight, eps, residual)
