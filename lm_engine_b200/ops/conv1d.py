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


def causal_conv1d(x, weight, bias=None, initial_state=None, activation=None):
    return causal_conv1d_reference(x, weight, bias, initial_state, activation)
