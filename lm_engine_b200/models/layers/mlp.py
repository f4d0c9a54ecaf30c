"""Dense MLP block: ``c_fc`` (column-parallel; doubled width for GLU activations, gate/up interleaved) ->
activation -> ``c_proj`` (row-parallel) -> dropout (lm_engine/modeling_utils/mlp_blocks/mlp/module.py:22-129).

On CUDA bf16 with SwiGLU and no bias the activation is fused into the ``c_fc`` GEMM epilogue and the residual add
into the ``c_proj`` epilogue.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...parameter import mark_parameter_as_mup_learning_rate
from ..config import MLPArgs
from .activations import GLUActivation, get_activation_function, is_glu
from .dropout import Dropout
from .init_utils import std_for_linear
from .linear import ColumnParallelLinear, RowParallelLinear


def interleave_up_gate(up: torch.Tensor, gate: torch.Tensor, is_glu_: bool = True) -> torch.Tensor:
    """Packs separate up / gate projection weights ``[I, H]`` into the ``c_fc`` layout: row 2j = gate_j,
    row 2j+1 = up_j (lm_engine/modeling_utils/mlp_blocks/mlp/utils.py:10-30)."""
    I = up.size(0)
    out = torch.empty((2 * I, *up.shape[1:]), dtype=up.dtype, device=up.device)
    out[0::2] = gate
    out[1::2] = up
    return out


def split_up_gate(c_fc: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`interleave_up_gate`; returns ``(up, gate)``."""
    return c_fc[1::2].contiguous(), c_fc[0::2].contiguous()


class MLP(nn.Module):
    def __init__(self, hidden_size: int, config: MLPArgs, init_method: str, initializer_range: float,
                 m_width: float | None, num_layers: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False) -> None:
        super().__init__()
        I = config.intermediate_size
        self.is_glu = is_glu(config.activation_function)
        std_fc = std_for_linear(initializer_range, init_method, m_width, hidden_size, num_layers, False)
        std_proj = std_for_linear(initializer_range, init_method, m_width, I, num_layers, use_depth_scaled_init)
        self.c_fc = ColumnParallelLinear(hidden_size, 2 * I if self.is_glu else I, bias=config.add_bias, std=std_fc,
                                         use_padding_free_transformer=use_padding_free_transformer,
                                         sequence_parallel=sequence_parallel)
        self.act = get_activation_function(config.activation_function)
        self.c_proj = RowParallelLinear(I, hidden_size, bias=config.add_bias, std=std_proj,
                                        use_padding_free_transformer=use_padding_free_transformer,
                                        sequence_parallel=sequence_parallel)
        self.dropout = Dropout(config.dropout)
        self._fusable = isinstance(self.act, GLUActivation) and self.act.is_swiglu and not config.add_bias
        mark_parameter_as_mup_learning_rate(self.c_fc.weight)
        mark_parameter_as_mup_learning_rate(self.c_proj.weight)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if (self._fusable and x.is_cuda and x.dtype == torch.bfloat16 and self.c_fc.tp_world_size == 1):
            x = ops.linear_swiglu(x, self.c_fc.weight)
        else:
            x = self.act(self.c_fc(x))
        fuse_res = residual is not None and self.dropout.p == 0
        x = self.c_proj(x, residual if fuse_res else None)
        x = self.dropout(x)
        if residual is not None and not fuse_res:
            x = x + residual
        return x
