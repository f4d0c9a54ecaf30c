"""Tensor-wise dynamically scaled FP8 linear layers on the 8-bit tcgen05 path.

Recipe (the one torchao's ``convert_to_float8_training`` applies in the reference, lm_engine/fp8.py:53-75):
activations and weights are cast to e4m3, output gradients to e5m2, each with one scale ``fmax / amax`` per tensor
computed from the tensor itself ("dynamic" scaling); master weights, optimizer state and every non-GEMM op stay in
bf16 / fp32.  The three GEMMs of a linear layer contract over different axes and the tensor core reads 8-bit operands
K-major only, so the quantiser emits a tensor and its transpose in one pass:

==========  ======================  =============================================
 forward     ``y  = x  @ W.T``       ``gemm_fp8(q(x)  [T,K], q(W)  [N,K])``
 dgrad       ``dx = dy @ W``         ``gemm_fp8(q(dy) [T,N], q(W).T [K,N])``
 wgrad       ``dW = dy.T @ x``       ``gemm_fp8(q(dy).T [N,T], q(x).T [K,T])``
==========  ======================  =============================================

The saved activation of a layer is its 1-byte transposed cast (half the bf16 footprint).  De-quantisation
(``scale_a * scale_b``) happens on the fp32 accumulator in the GEMM epilogue, before bias / residual / SwiGLU.
On CPU (tests) the same arithmetic runs through ``torch.float8_*`` casts.
"""

from __future__ import annotations

import torch

from . import _lib
from .gemm import _max_ctas, gemm_reference

E4M3, E5M2 = 0, 1
_FMAX = {E4M3: 448.0, E5M2: 57344.0}
_TORCH = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}


class Fp8Tensor:
    """A quantised matrix: ``q`` [rows, cols] and / or ``qt`` [cols, rows] (uint8 storage), its format and the
    one-element fp32 de-quantisation scale."""

    __slots__ = ("q", "qt", "scale_inv", "fmt", "shape")

    def __init__(self, q, qt, scale_inv, fmt, shape):
        self.q, self.qt, self.scale_inv, self.fmt, self.shape = q, qt, scale_inv, fmt, shape

    def dequantize(self, transposed: bool = False) -> torch.Tensor:
        t = self.qt if transposed else self.q
        return t.view(_TORCH[self.fmt]).float() * self.scale_inv


def quantize_reference(x: torch.Tensor, fmt: int, rowwise: bool = True, transposed: bool = False) -> Fp8Tensor:
    xf = x.float()
    amax = xf.abs().max().clamp_min(1e-12)
    scale = _FMAX[fmt] / amax
    q = (xf * scale).clamp(-_FMAX[fmt], _FMAX[fmt]).to(_TORCH[fmt]).view(torch.uint8)
    return Fp8Tensor(q if rowwise else None, q.t().contiguous() if transposed else None,
                     (amax / _FMAX[fmt]).reshape(1), fmt, tuple(x.shape))


def quantize(x: torch.Tensor, fmt: int = E4M3, rowwise: bool = True, transposed: bool = False) -> Fp8Tensor:
    """Casts a bf16 matrix to FP8 with its own amax as the scale (two kernels: amax, scaled cast [+ transpose])."""
    assert x.dim() == 2
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return quantize_reference(x, fmt, rowwise, transposed)
    R, C = x.shape
    if not x.is_contiguous() or x.data_ptr() % 16:
        x = x.contiguous().clone() if x.data_ptr() % 16 else x.contiguous()
    lib = _lib.cuda_lib()
    amax = torch.zeros(1, dtype=torch.float32, device=x.device)
    scale_inv = torch.empty(1, dtype=torch.float32, device=x.device)
    st = _lib.stream_ptr()
    _lib.check(lib.lme_fp8_amax(x.data_ptr(), x.numel(), amax.data_ptr(), st), "lme_fp8_amax")
    q = torch.empty((R, C), dtype=torch.uint8, device=x.device) if rowwise else None
    qt = torch.empty((C, R), dtype=torch.uint8, device=x.device) if transposed else None
    _lib.check(lib.lme_fp8_quantize(x.data_ptr(), R, C, x.stride(0), amax.data_ptr(), fmt, _lib.ptr(q), C,
                                    _lib.ptr(qt), R, scale_inv.data_ptr(), st), f"lme_fp8_quantize {R}x{C}")
    _lib.count_launch(2)
    return Fp8Tensor(q, qt, scale_inv, fmt, (R, C))


def gemm_fp8(a: torch.Tensor, a_fmt: int, a_scale: torch.Tensor, b: torch.Tensor, b_fmt: int, b_scale: torch.Tensor,
             *, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, accumulate: bool = False,
             bias=None, residual=None, swiglu: bool = False, preact=None) -> torch.Tensor:
    """``C[M, N] = (A[M, K] @ B[N, K].T) * a_scale * b_scale`` with uint8-stored FP8 operands, both K-major."""
    M, K = a.shape
    N = b.size(0)
    assert b.size(1) == K
    if not a.is_cuda:
        A = a.view(_TORCH[a_fmt]).float() * a_scale
        B = b.view(_TORCH[b_fmt]).float() * b_scale
        return gemm_reference(A, B, out=out, out_dtype=out_dtype or torch.bfloat16, accumulate=accumulate, bias=bias,
                              residual=residual, swiglu=swiglu, preact=preact)
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    flags = 0
    if out.dtype == torch.float32:
        flags |= _lib.GEMM_OUT_F32
    if accumulate:
        flags |= _lib.GEMM_ACCUMULATE
    if swiglu:
        flags |= _lib.GEMM_SWIGLU
    lib = _lib.cuda_lib()
    rc = lib.lme_gemm_fp8(a.data_ptr(), a_fmt, a.stride(0), b.data_ptr(), b_fmt, b.stride(0), a_scale.data_ptr(),
                          b_scale.data_ptr(), out.data_ptr(), out.stride(0), M, N, K, flags, _lib.ptr(bias),
                          _lib.ptr(residual), residual.stride(0) if residual is not None else 0, _lib.ptr(preact),
                          preact.stride(0) if preact is not None else 0, _max_ctas(a.device), _lib.stream_ptr())
    _lib.check(rc, f"lme_gemm_fp8 M={M} N={N} K={K}")
    _lib.count_launch()
    return out


def fp8_eligible(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Every contraction / pitch of the three GEMMs must be a multiple of 16 bytes."""
    T = x.numel() // x.size(-1)
    return T % 16 == 0 and weight.size(0) % 16 == 0 and weight.size(1) % 16 == 0


def _backward(ctx, dy2: torch.Tensor, xq: Fp8Tensor, wq_t: Fp8Tensor, weight: torch.Tensor, need_dx: bool,
              need_dw: bool):
    gq = quantize(dy2, E5M2, rowwise=need_dx, transposed=need_dw)
    dx = dw = None
    if need_dx:
        dx = gemm_fp8(gq.q, E5M2, gq.scale_inv, wq_t.qt, E4M3, wq_t.scale_inv)
    if need_dw:
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            stale = getattr(weight, "main_grad_stale", False)
            gemm_fp8(gq.qt, E5M2, gq.scale_inv, xq.qt, E4M3, xq.scale_inv, out=main_grad, accumulate=not stale)
            if stale:
                weight.main_grad_stale = False
        else:
            dw = gemm_fp8(gq.qt, E5M2, gq.scale_inv, xq.qt, E4M3, xq.scale_inv, out_dtype=weight.dtype)
    return dx, dw


class _LinearFp8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, weight.size(0)) if residual is not None else None
        xq = quantize(x2, E4M3, rowwise=True, transposed=True)
        wq = quantize(weight, E4M3, rowwise=True, transposed=False)
        y = gemm_fp8(xq.q, E4M3, xq.scale_inv, wq.q, E4M3, wq.scale_inv, bias=bias, residual=r2)
        ctx.xq = Fp8Tensor(None, xq.qt, xq.scale_inv, E4M3, xq.shape)   # only the transposed cast is kept
        ctx.weight = weight   # re-quantised (transposed) in backward: the gathered weight buffer may be recycled
        ctx.has_bias, ctx.has_residual, ctx.in_shape = bias is not None, residual is not None, shape
        return y.view(*shape[:-1], weight.size(0))

    @staticmethod
    def backward(ctx, dy):
        weight = ctx.weight
        dy2 = dy.reshape(-1, dy.size(-1))
        wq_t = quantize(weight, E4M3, rowwise=False, transposed=True) if ctx.needs_input_grad[0] else None
        dx, dw = _backward(ctx, dy2, ctx.xq, wq_t, weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        db = dres = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy.dtype)
        if ctx.has_residual and ctx.needs_input_grad[3]:
            dres = dy
        return (dx.view(ctx.in_shape) if dx is not None else None), dw, db, dres


class _LinearSwiGLUFp8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        N = weight.size(0)
        xq = quantize(x2, E4M3, rowwise=True, transposed=True)
        wq = quantize(weight, E4M3, rowwise=True, transposed=False)
        pre = torch.empty((x2.size(0), N), dtype=x.dtype, device=x.device)
        y = gemm_fp8(xq.q, E4M3, xq.scale_inv, wq.q, E4M3, wq.scale_inv, swiglu=True, preact=pre)
        ctx.xq = Fp8Tensor(None, xq.qt, xq.scale_inv, E4M3, xq.shape)
        ctx.weight, ctx.in_shape = weight, shape
        ctx.save_for_backward(pre)
        return y.view(*shape[:-1], N // 2)

    @staticmethod
    def backward(ctx, dy):
        from .activation import swiglu_backward

        (pre,) = ctx.saved_tensors
        weight = ctx.weight
        dpre = swiglu_backward(pre, dy.reshape(pre.size(0), -1))
        wq_t = quantize(weight, E4M3, rowwise=False, transposed=True) if ctx.needs_input_grad[0] else None
        dx, dw = _backward(ctx, dpre, ctx.xq, wq_t, weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return (dx.view(ctx.in_shape) if dx is not None else None), dw


def linear_fp8(x, weight, bias=None, residual=None):
    return _LinearFp8.apply(x, weight, bias, residual)


def linear_swiglu_fp8(x, weight):
    return _LinearSwiGLUFp8.apply(x, weight)
