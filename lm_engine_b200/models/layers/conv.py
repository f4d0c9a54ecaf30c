"""Depthwise causal 1-D convolution with carried state (prefill, single-token update, multi-token continuation),
optional fused activation, padding-mask zeroing and the context-parallel halo exchange
(lm_engine/modeling_utils/depthwise_causal_convolution.py:28-254).  The parameter layout is ``nn.Conv1d``'s:
``weight [C, 1, K]``, ``bias [C]``."""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ...ops.conv1d import causal_conv1d
from ...parallel.manager import ProcessGroupManager
from ...parameter import mark_parameter_as_initialized, mark_parameter_as_no_weight_decay
from .activations import get_activation_function


def apply_mask_to_padding_states(x: torch.Tensor, attention_mask: torch.Tensor | None) -> torch.Tensor:
    if attention_mask is not None and attention_mask.shape[1] > 1 and attention_mask.shape[0] > 1:
        return (x * attention_mask[:, :, None]).to(x.dtype)
    return x


class _HaloFromPreviousRank(torch.autograd.Function):
    """Last ``K-1`` timesteps of the previous context-parallel rank (zeros on the first rank); the gradient flows
    back to the rank that produced them."""

    @staticmethod
    def forward(ctx, tail, group):
        ctx.group = group
        world, r = dist.get_world_size(group), dist.get_rank(group)
        parts = [torch.empty_like(tail) for _ in range(world)]
        dist.all_gather(parts, tail.contiguous(), group=group)
        return parts[r - 1] if r > 0 else torch.zeros_like(tail)

    @staticmethod
    def backward(ctx, g):
        world, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        parts = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(parts, (g if r > 0 else torch.zeros_like(g)).contiguous(), group=ctx.group)
        return (parts[r + 1] if r + 1 < world else torch.zeros_like(g)), None


class DepthwiseCausalConvolution(nn.Module):
    def __init__(self, hidden_size: int, kernel_size: int, activation_function: str | None, add_bias: bool,
                 std: float | None, use_padding_free_transformer: bool = False) -> None:
        super().__init__()
        assert kernel_size > 1
        if use_padding_free_transformer:
            raise NotImplementedError()
        self.hidden_size, self.kernel_size, self.std = hidden_size, kernel_size, std
        self.weight = nn.Parameter(torch.empty(hidden_size, 1, kernel_size))
        self.bias = nn.Parameter(torch.empty(hidden_size)) if add_bias else None
        mark_parameter_as_no_weight_decay(self.bias)
        self.activation_string = activation_function
        self.fused_activation = activation_function in (None, "silu", "swish", "identity")
        self.activation_function = (nn.Identity() if activation_function is None
                                    else get_activation_function(activation_function))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.weight.is_meta:
            return
        if self.std is None:
            bound = 1 / self.kernel_size**0.5
            nn.init.uniform_(self.weight, -bound, bound)
            if self.bias is not None:
                nn.init.uniform_(self.bias, -bound, bound)
        else:
            nn.init.normal_(self.weight, mean=0, std=self.std)
            if self.bias is not None:
                self.bias.zero_()
        mark_parameter_as_initialized(self.weight)
        mark_parameter_as_initialized(self.bias)

    def forward(self, x: torch.Tensor, input_state: torch.Tensor | None, attention_mask: torch.Tensor | None,
                output_state: bool) -> tuple[torch.Tensor, torch.Tensor | None]:
        """x ``[B, S, C]``; state ``[B, C, K-1]`` (the last K-1 raw inputs).  Returns ``(y [B, S, C], new state)``."""
        K = self.kernel_size
        x = apply_mask_to_padding_states(x, attention_mask)
        cp_group = ProcessGroupManager.get_context_parallel_group()
        if cp_group is not None:
            assert input_state is None and not output_state
            assert ProcessGroupManager.get_context_parallel_load_balancing_method() is None
            assert x.size(1) >= K - 1
            input_state = _HaloFromPreviousRank.apply(x[:, 1 - K:], cp_group).transpose(1, 2)
        new_state = None
        if output_state:
            hist = x.transpose(1, 2) if input_state is None else torch.cat((input_state, x.transpose(1, 2)), dim=-1)
            new_state = hist[..., 1 - K:] if hist.size(-1) >= K - 1 else F.pad(hist, (K - 1 - hist.size(-1), 0))
        act = self.activation_string if self.fused_activation else None
        y = causal_conv1d(x, self.weight.squeeze(1), self.bias, input_state, act)
        if not self.fused_activation:
            y = self.activation_function(y)
        y = apply_mask_to_padding_states(y, attention_mask)
        return y, new_state
