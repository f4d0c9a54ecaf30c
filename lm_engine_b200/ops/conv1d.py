"""Depthwise causal convolution ``y[t, c] = act(b[c] + sum_j w[c, j] * x[t - (K-1) + j, c])`` with an optional
initial state holding the ``K-1`` inputs before ``t = 0``.  Counterpart of ``causal_conv1d_fn`` /
``causal_conv1d_update`` used by the reference (lm_engine/modeling_utils/depthwise_causal_convolution.py:110-206)."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_conv1d_reference(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                            initial_state: torch.Tensor | None, activation: str | None) -> torch.Tensor:
    """x ``[B, S, C]``, weight ``[C, K]``, initial_state ``[B, C, K-1]`` -> ``[B, S, C]``."""
    B, S, C = x.shape
    K = weight.size(1)
    xt = x.transpose(1, 2)
    if initial_state is None:
        xt = F.pad(xt, (K - 1, 0))
    else:
        xt = torch.cat((initial_state.to(xt.dtype), xt), dim=-1)
    y = F.conv1d(xt, weight.unsqueeze(1), bias, groups=C)
    y = y.transpose(1, 2)
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y


class _CausalConv1d(torch.autograd.Function):
    """CUDA path: one pass forward (activation fused), one pass backward that recomputes the pre-activation."""

    @staticmethod
    def forward(ctx, x, weight, bias, initial_state, silu: bool):
        from . import _lib

        x = x.contiguous()
        B, S, C = x.shape
        K = weight.size(1)
        w = weight.contiguous()
        init = initial_state.to(x.dtype).contiguous() if initial_state is not None else None
        y = torch.empty_like(x)
        _lib.check(_lib.cuda_lib().lme_causal_conv1d_fwd(x.data_ptr(), w.data_ptr(), _lib.ptr(bias), _lib.ptr(init),
                                                         y.data_ptr(), B, S, C, K, int(silu), _lib.stream_ptr()),
                   f"lme_causal_conv1d_fwd B={B} S={S} C={C} K={K}")
        _lib.count_launch()
        ctx.save_for_backward(x, w, bias, init)
        ctx.silu = silu
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _lib

        x, w, bias, init = ctx.saved_tensors
        B, S, C = x.shape
        K = w.size(1)
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros((C, K), dtype=torch.float32, device=x.device)
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if bias is not None else None
        dinit = (torch.empty((B, C, K - 1), dtype=torch.float32, device=x.device)
                 if init is not None and ctx.needs_input_grad[3] else None)
        _lib.check(_lib.cuda_lib().lme_causal_conv1d_bwd(
            x.data_ptr(), w.data_ptr(), _lib.ptr(bias), _lib.ptr(init), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(),
            _lib.ptr(db), _lib.ptr(dinit), B, S, C, K, int(ctx.silu), _lib.stream_ptr()),
            f"lme_causal_conv1d_bwd B={B} S={S} C={C} K={K}")
        _lib.count_launch()
        return (dx, dw.to(w.dtype), db.to(bias.dtype) if db is not None else None,
                dinit.to(init.dtype) if dinit is not None else None, None)


def causal_conv1d(x, weight, bias=None, initial_state=None, activation=None):
    """x ``[B, S, C]``, weight ``[C, K]``, bias ``[C]``, initial_state ``[B, C, K-1]`` -> ``[B, S, C]``."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.size(-1) % 8 == 0
            and weight.size(1) <= 8 and activation in (None, "silu", "swish")
            and (bias is None or bias.dtype == torch.bfloat16)):
        return _CausalConv1d.apply(x, weight, bias, initial_state, activation is not None)
    return causal_conv1d_reference(x, weight, bias, initial_state, activation)
