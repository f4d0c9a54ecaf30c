"""Activation functions by name: base activations and the GLU family on the packed interleaved layout
(lm_engine/modeling_utils/activations/*.py).  ``swiglu`` runs the CUDA kernel (or is fused into the producing GEMM's
epilogue by :class:`~lm_engine_b200.models.layers.mlp.MLP`)."""

from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops


class ReLUSquared(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = torch.relu(x)
        return y * y


class _Upcast(nn.Module):
    """fp32 evaluation of a saturating activation, cast back to the input dtype."""

    def __init__(self, fn) -> None:
        super().__init__()
        self.fn = fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fn(x.float()).to(x.dtype)


_BASE = {
    "celu": nn.CELU, "elu": nn.ELU, "gelu": nn.GELU, "gelu_pytorch_tanh": lambda: nn.GELU(approximate="tanh"),
    "selu": nn.SELU, "hard_shrink": nn.Hardshrink, "hard_sigmoid": nn.Hardsigmoid, "hard_swish": nn.Hardswish,
    "hard_tanh": nn.Hardtanh, "identity": nn.Identity, "leaky_reLU": nn.LeakyReLU, "log_sigmoid": nn.LogSigmoid,
    "mish": nn.Mish, "prelu": nn.PReLU, "relu": nn.ReLU, "relu2": ReLUSquared, "relu_squared": ReLUSquared,
    "relu6": nn.ReLU6, "rrelu": nn.RReLU, "sigmoid": nn.Sigmoid, "silu": nn.SiLU, "swish": nn.SiLU,
    "softplus": nn.Softplus, "soft_plus": nn.Softplus, "soft_shrink": nn.Softshrink, "soft_sign": nn.Softsign,
    "tanh": nn.Tanh, "tanh_shrink": nn.Tanhshrink,
}
_GLU_BASE = {"glu": "sigmoid", "sigmoid_glu": "sigmoid", "ceglu": "celu", "eglu": "elu", "geglu": "gelu",
             "miglu": "mish", "mishglu": "mish", "preglu": "prelu", "reglu": "relu", "rreglu": "rrelu",
             "seglu": "selu", "swiglu": "swish"}


def get_base_activation(name: str) -> nn.Module:
    if name not in _BASE:
        raise ValueError("invalid activation function")
    return _BASE[name]()


class GLUActivation(nn.Module):
    """``up * act(gate)`` where gate / up are the even / odd columns of the packed input."""

    def __init__(self, base: nn.Module) -> None:
        super().__init__()
        self.base_activation = base
        self.is_swiglu = isinstance(base, nn.SiLU)

    def forward(self, x: torch.Tensor | None, u: torch.Tensor | None = None, g: torch.Tensor | None = None):
        if x is None:
            return u * self.base_activation(g)
        if self.is_swiglu:
            return ops.swiglu_packed(x)
        return x[..., 1::2] * self.base_activation(x[..., ::2])


def is_glu(name: str) -> bool:
    return name.endswith("glu")


def get_glu_activation(name: str) -> GLUActivation:
    if name in _GLU_BASE:
        base = _GLU_BASE[name]
    elif name.endswith("_glu"):
        base = name[: -len("_glu")]
    else:
        raise ValueError("invalid activation function")
    return GLUActivation(get_base_activation(base))


def get_activation_function(name: str) -> nn.Module:
    return get_glu_activation(name) if is_glu(name) else get_base_activation(name)


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return torch.sigmoid(x.float()).to(x.dtype)


def silu(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(x.float()).to(x.dtype)


def tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.tanh(x.float()).to(x.dtype)


class _ClipGradients(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, limit):
        ctx.limit = limit
        return x

    @staticmethod
    def backward(ctx, g):
        return g.clamp(-ctx.limit, ctx.limit), None


def clip_gradients(x: torch.Tensor, limit: float | None) -> torch.Tensor:
    """Identity in forward; clamps the gradient flowing back through ``x`` to [-limit, limit]."""
    return x if limit is None else _ClipGradients.apply(x, limit)
