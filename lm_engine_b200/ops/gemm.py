"""bf16 GEMM on tcgen05 tensor cores with fused epilogues, and the ``linear`` autograd op built on it.

``gemm(a, b)`` computes ``C[M, N] = sum_k A(m, k) * B(n, k)``.  Each operand is either *K-major* (a row-major
``[rows, K]`` tensor) or *MN-major* (a row-major ``[K, rows]`` tensor, flag ``a_mn`` / ``b_mn``) - the tensor core
consumes both layouts directly from shared memory, so the backward GEMMs of a linear layer never materialise a
transpose:

==========  =======================  ======================
 forward     ``y  = x  @ W.T``        ``gemm(x, W)``
 dgrad       ``dx = dy @ W``          ``gemm(dy, W, b_mn=True)``
 wgrad       ``dW = dy.T @ x``        ``gemm(dy, x, a_mn=True, b_mn=True)``
==========  =======================  ======================

Plays the role of ``F.linear`` / QuACK ``gemm``/``gemm_act``/``gemm_gated`` in the reference
(lm_engine/modeling_utils/linear/base.py:17-49, lm_engine/modeling_utils/quack.py:19-132).
"""

from __future__ import annotations

import os

import torch

from . import _lib

# SMs left free for communication kernels that run concurrently with the persistent GEMMs (set by the sharding
# runtime when collectives overlap compute).  A persistent kernel that cannot place all of its CTAs at once would
# otherwise wait for the collective to release its SMs.
RESERVED_SMS = 0
_NUM_SMS: dict[int, int] = {}


def _max_ctas(device: torch.device) -> int:
    if RESERVED_SMS <= 0:
        return 0
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _NUM_SMS:
        _NUM_SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return max(_NUM_SMS[idx] - RESERVED_SMS, 8)


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("gemm operands must be 2-D")
    if t.stride(1) != 1 or t.stride(0) < t.size(1) or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def gemm_reference(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, accumulate=False, bias=None,
                   residual=None, swiglu=False, preact=None):
    """PyTorch statement of :func:`gemm` (CPU path and numerical oracle)."""
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if A.is_cuda and A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16:
        try:        # library GEMM on the tensor cores with an fp32 result (shapes the tcgen05 kernel does not take)
            acc = torch.mm(A, B.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            acc = torch.mm(A, B.t()).float()
    else:
        acc = A.float() @ B.float().t()
    if bias is not None:
        acc = acc + bias.float()
    if swiglu:
        pre = acc.to(a.dtype)
        if preact is not None:
            preact.copy_(pre)
        pre = pre.float()
        res = (pre[:, 1::2] * torch.nn.functional.silu(pre[:, 0::2])).to(out_dtype)
    else:
        if residual is not None:
            acc = acc + residual.float()
        if accumulate:
            acc = acc + out.float()
        res = acc.to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    swiglu: bool = False,
    preact: torch.Tensor | None = None,
    max_ctas: int = 0,
    probe: int = 0,
) -> torch.Tensor:
    """``probe``: timing-probe flags of the micro-benchmarks (64: stages are never loaded, 128: never multiplied);
    the result is meaningless with either."""
    if not (a.is_cuda and a.dtype == torch.bfloat16):
        return gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=out_dtype, accumulate=accumulate,
                              bias=bias, residual=residual, swiglu=swiglu, preact=preact)
    a = _rowmajor(a)
    b = _rowmajor(b)
    if b.dtype != torch.bfloat16:
        raise TypeError("gemm: both operands must be bf16")
    K, M = (a.size(0), a.size(1)) if a_mn else (a.size(1), a.size(0))
    Kb, N = (b.size(0), b.size(1)) if b_mn else (b.size(1), b.size(0))
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    n_out = N // 2 if swiglu else N
    # the kernel moves operands with TMA: leading dimensions and N in units of 16 bytes.  Other shapes (an output
    # width that is not a multiple of 8, e.g. a projection that carries one scalar gate per head) take the library
    # GEMM with the same epilogue semantics.
    if (N % 8 or (swiglu and N % 16) or a.stride(0) % 8 or b.stride(0) % 8
            or (out is not None and (out.stride(1) != 1 or out.stride(0) % 4))
            or (residual is not None and residual.stride(0) % 8) or (preact is not None and preact.stride(0) % 8)):
        from ..logging_utils.logger import warn_once

        warn_once(f"gemm-library-{N}-{K}", f"gemm: M={M} N={N} K={K} (strides {a.stride(0)}, {b.stride(0)}) does "
                  "not meet the 16-byte rule of the TMA operand loads; this product runs on the library GEMM")
        return gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=out_dtype, accumulate=accumulate,
                              bias=bias, residual=residual, swiglu=swiglu, preact=preact)
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    elif out.stride(1) != 1 or out.shape != (M, n_out):
        raise ValueError("gemm: out must be a row-major [M, N] tensor")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm: out must be bf16 or fp32")
    flags = int(probe) & 192
    if out.dtype == torch.float32:
        flags |= _lib.GEMM_OUT_F32
    if accumulate:
        flags |= _lib.GEMM_ACCUMULATE
    if swiglu:
        flags |= _lib.GEMM_SWIGLU
        if preact is not None and (preact.shape != (M, N) or preact.stride(1) != 1):
            raise ValueError("gemm: preact must be row-major [M, N]")
    if residual is not None:
        if residual.shape != (M, N) or residual.stride(1) != 1 or residual.dtype != torch.bfloat16:
            raise ValueError("gemm: residual must be a row-major bf16 [M, N] tensor")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("gemm: bias must be a contiguous bf16 [N] tensor")
    lib = _lib.cuda_lib()
    rc = lib.lme_gemm_bf16(
        a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0), out.data_ptr(), out.stride(0),
        M, N, K, flags, _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        _lib.ptr(preact), preact.stride(0) if preact is not None else 0, max_ctas or _max_ctas(a.device),
        _lib.stream_ptr(),
    )
    _lib.check(rc, f"lme_gemm_bf16 M={M} N={N} K={K}")
    _lib.count_launch()
    return out


def _wgrad_into(main_grad: torch.Tensor, weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> None:
    """dW = dy^T x written into the parameter's gradient buffer by the GEMM epilogue.  The first write of a step
    overwrites (the buffer was not cleared, flag ``main_grad_stale``), later ones accumulate."""
    stale = getattr(weight, "main_grad_stale", False)
    gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=not stale)
    if stale:
        weight.main_grad_stale = False


class _Linear(torch.autograd.Function):
    """y = x W^T (+ b) (+ residual).  The weight gradient is accumulated straight into ``weight.main_grad`` by the
    GEMM epilogue when that buffer exists (gradient accumulation fused into wgrad), else returned to autograd."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, weight.size(0)) if residual is not None else None
        y = gemm(x2, weight, bias=bias, residual=r2)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_residual = residual is not None
        ctx.in_shape = shape
        return y.view(*shape[:-1], weight.size(0))

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                _wgrad_into(main_grad, weight, dy2, x2)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy.dtype)
        if ctx.has_residual and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear`` with an optional fused residual add; tcgen05 GEMMs on CUDA bf16, PyTorch elsewhere."""
    if getattr(weight, "fp8", False) == "block":
        from . import fp8_block

        if fp8_block.block_eligible(x, weight):
            return fp8_block.linear_block_scaled(x, weight, bias, residual)
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        if getattr(weight, "fp8", False) is True:
            from . import fp8

            if fp8.fp8_eligible(x, weight):
                return fp8.linear_fp8(x, weight, bias, residual)
        return _Linear.apply(x, weight, bias, residual)
    y = torch.nn.functional.linear(x, weight, bias)
    return y if residual is None else y + residual


class _LinearSwiGLU(torch.autograd.Function):
    """``swiglu_packed(x W^T)`` with the activation fused into the GEMM epilogue.  The bf16 pre-activation is kept
    for backward (the reference's QuACK path does the same with ``store_preact``)."""

    @staticmethod
    def forward(ctx, x, weight):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        N = weight.size(0)
        pre = torch.empty((x2.size(0), N), dtype=x.dtype, device=x.device)
        y = gemm(x2, weight, swiglu=True, preact=pre)
        ctx.save_for_backward(x2, weight, pre)
        ctx.in_shape = shape
        return y.view(*shape[:-1], N // 2)

    @staticmethod
    def backward(ctx, dy):
        from .activation import swiglu_backward

        x2, weight, pre = ctx.saved_tensors
        dpre = swiglu_backward(pre, dy.reshape(pre.size(0), -1))
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dpre, weight, b_mn=True).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                _wgrad_into(main_grad, weight, dpre, x2)
            else:
                dw = gemm(dpre, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        return dx, dw


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``up * silu(gate)`` of the packed projection ``x W^T`` (gate/up interleaved along the output features)."""
    if getattr(weight, "fp8", False) == "block":
        from . import fp8_block
        from .activation import swiglu_packed

        if fp8_block.block_eligible(x, weight):
            return swiglu_packed(fp8_block.linear_block_scaled(x, weight))
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.size(0) % 16 == 0:
        if getattr(weight, "fp8", False) is True:
            from . import fp8

            if fp8.fp8_eligible(x, weight):
                return fp8.linear_swiglu_fp8(x, weight)
        return _LinearSwiGLU.apply(x, weight)
    from .activation import swiglu_packed

    return swiglu_packed(torch.nn.functional.linear(x, weight))


# ---------------------------------------------------------------------------------------------- batched products
def _batched_operand(t: torch.Tensor) -> torch.Tensor:
    """3-D bf16 operand with unit inner stride and row / batch pitches that TMA accepts (multiples of 16 bytes)."""
    if t.dim() != 3:
        raise ValueError("bmm operands must be 3-D")
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    if (t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.stride(1) < t.size(2) or t.data_ptr() % 16
            or (t.size(0) > 1 and t.stride(0) < t.size(1) * t.stride(1))):
        t = t.contiguous()
    return t


def bmm_reference(a, b, *, a_mn=False, b_mn=False, out_dtype=torch.float32):
    A = a.transpose(1, 2) if a_mn else a
    B = b if b_mn else b.transpose(1, 2)
    return torch.bmm(A.float(), B.float()).to(out_dtype)


def _bmm_kernel(a, b, a_mn, b_mn, out_dtype):
    a, b = _batched_operand(a), _batched_operand(b)
    batch = a.size(0)
    K, M = (a.size(1), a.size(2)) if a_mn else (a.size(2), a.size(1))
    Kb, N = (b.size(1), b.size(2)) if b_mn else (b.size(2), b.size(1))
    if K != Kb or b.size(0) != batch:
        raise ValueError(f"bmm: shapes {tuple(a.shape)} (a_mn={a_mn}) x {tuple(b.shape)} (b_mn={b_mn}) do not match")
    out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
    if batch == 0 or M == 0 or N == 0:
        return out
    flags = _lib.GEMM_OUT_F32 if out_dtype == torch.float32 else 0
    rc = _lib.cuda_lib().lme_gemm_bf16_batched(
        a.data_ptr(), int(a_mn), a.stride(1), a.stride(0), b.data_ptr(), int(b_mn), b.stride(1), b.stride(0),
        out.data_ptr(), out.stride(1), out.stride(0), batch, M, N, K, flags, _max_ctas(a.device), _lib.stream_ptr())
    _lib.check(rc, f"lme_gemm_bf16_batched batch={batch} M={M} N={N} K={K}")
    _lib.count_launch()
    return out


def _bmm_kernel_usable(a, b, a_mn, b_mn) -> bool:
    if not (a.is_cuda and a.dim() == 3 and b.dim() == 3):
        return False
    K, M = (a.size(1), a.size(2)) if a_mn else (a.size(2), a.size(1))
    N = b.size(2) if b_mn else b.size(1)
    # innermost extents of the tensor maps and the output pitch in units of 16 bytes
    return N % 8 == 0 and (M if a_mn else K) % 8 == 0 and (N if b_mn else K) % 8 == 0


class _Bmm(torch.autograd.Function):
    """``C[i] = A[i] B[i]^T`` over a batch on the tcgen05 GEMM (3-D tensor maps), fp32 or bf16 result; the two
    gradients are the same kernel with the layouts swapped, so no operand is ever transposed in memory."""

    @staticmethod
    def forward(ctx, a, b, a_mn, b_mn, out_dtype):
        ctx.save_for_backward(a, b)
        ctx.cfg = (a_mn, b_mn)
        return _bmm_kernel(a, b, a_mn, b_mn, out_dtype)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        a_mn, b_mn = ctx.cfg
        g = g.to(torch.bfloat16)
        da = db = None
        if ctx.needs_input_grad[0]:
            # dA = dC B  (stored like A: [M, K], or [K, M] when A is MN-major)
            da = (_bmm_kernel(b, g, not b_mn, False, torch.bfloat16) if a_mn
                  else _bmm_kernel(g, b, False, not b_mn, torch.bfloat16)).to(a.dtype)
        if ctx.needs_input_grad[1]:
            # dB = dC^T A  (stored like B: [N, K], or [K, N] when B is MN-major)
            db = (_bmm_kernel(a, g, not a_mn, True, torch.bfloat16) if b_mn
                  else _bmm_kernel(g, a, True, not a_mn, torch.bfloat16)).to(b.dtype)
        return da, db, None, None, None


def bmm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
        out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Batched ``C[i, M, N] = sum_k A_i(m, k) B_i(n, k)``: ``a`` is ``[batch, M, K]`` (or ``[batch, K, M]`` with
    ``a_mn``), ``b`` is ``[batch, N, K]`` (or ``[batch, K, N]`` with ``b_mn``); bf16 operands, fp32 accumulation.
    Differentiable.  Shapes that the TMA loads cannot take run as a PyTorch statement."""
    if not _bmm_kernel_usable(a, b, a_mn, b_mn):
        if a.is_cuda:
            from ..logging_utils.logger import warn_once

            warn_once(f"bmm-library-{tuple(a.shape[1:])}-{tuple(b.shape[1:])}",
                      f"bmm: operands {tuple(a.shape)} x {tuple(b.shape)} do not meet the 16-byte rule of the TMA "
                      "loads; this product runs on the library GEMM")
            A = a.transpose(1, 2) if a_mn else a
            B = b if b_mn else b.transpose(1, 2)
            return torch.bmm(A.to(torch.bfloat16), B.to(torch.bfloat16)).to(out_dtype)
        return bmm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype)
    return _Bmm.apply(a, b, a_mn, b_mn, out_dtype)
