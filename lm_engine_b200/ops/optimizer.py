"""Fused AdamW on flat fp32 shards, squared-norm reduction and clip coefficient (device-side, no host sync).

Replaces ``torch.optim.AdamW`` + ``clip_grad_norm_`` of the reference (lm_engine/optimization/optimizer.py:89-94,
lm_engine/train.py:211) for the flat-buffer parameter layout of :mod:`lm_engine_b200.parallel.fsdp`.
"""

from __future__ import annotations

import math

import torch

from . import _lib


def adamw_reference(p, m, v, g, p_lp, lr, b1, b2, eps, wd, step, gscale=None):
    gf = g.float()
    if gscale is not None:
        gf = gf * gscale
    p.mul_(1 - lr * wd)
    m.mul_(b1).add_(gf, alpha=1 - b1)
    v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
    bc1 = 1 - b1**step
    bc2 = 1 - b2**step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if p_lp is not None:
        p_lp.copy_(p)


def adamw_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, p_lp: torch.Tensor | None, *,
               lr: float, betas: tuple[float, float], eps: float, weight_decay: float, step: int,
               gscale: torch.Tensor | None = None) -> None:
    """One AdamW step on flat tensors: ``p/m/v`` fp32 master + moments, ``g`` bf16 or fp32 gradient, ``p_lp`` the
    bf16 compute copy refreshed in the same pass; ``gscale`` a 1-element device tensor multiplied into ``g``."""
    if not p.is_cuda:
        adamw_reference(p, m, v, g, p_lp, lr, betas[0], betas[1], eps, weight_decay, step, gscale)
        return
    assert p.dtype == m.dtype == v.dtype == torch.float32 and g.dtype in (torch.bfloat16, torch.float32)
    assert p.is_contiguous() and m.is_contiguous() and v.is_contiguous() and g.is_contiguous()
    _lib.check(_lib.cuda_lib().lme_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                         int(g.dtype == torch.bfloat16), _lib.ptr(p_lp), p.numel(), lr, betas[0],
                                         betas[1], eps, weight_decay, step, _lib.ptr(gscale), _lib.stream_ptr()),
               "lme_adamw")
    _lib.count_launch()


_partials: dict[torch.device, torch.Tensor] = {}


def sumsq_(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[0] (+)= sum(x^2) in fp32, deterministic two-stage reduction."""
    if not x.is_cuda:
        s = x.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
        return
    scratch = _partials.get(x.device)
    if scratch is None:
        scratch = _partials[x.device] = torch.empty(_lib.SUMSQ_MAX_PARTIALS, dtype=torch.float32, device=x.device)
    assert x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float32)
    _lib.check(_lib.cuda_lib().lme_sumsq(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(),
                                         scratch.data_ptr(), out.data_ptr(), int(accumulate), _lib.stream_ptr()),
               "lme_sumsq")
    _lib.count_launch(2)


def clip_coef_(sumsq: torch.Tensor, max_norm: float | None, norm_out: torch.Tensor, coef_out: torch.Tensor) -> None:
    """norm = sqrt(sumsq); coef = min(1, max_norm / (norm + 1e-6)) (torch ``clip_grad_norm_`` semantics)."""
    mn = float(max_norm) if max_norm is not None else 0.0
    if not sumsq.is_cuda:
        n = sumsq[0].sqrt()
        norm_out[0] = n
        coef_out[0] = min(1.0, mn / (float(n) + 1e-6)) if mn > 0 else 1.0
        return
    _lib.check(_lib.cuda_lib().lme_clip_coef(sumsq.data_ptr(), mn, norm_out.data_ptr(), coef_out.data_ptr(),
                                             _lib.stream_ptr()), "lme_clip_coef")
    _lib.count_launch()
