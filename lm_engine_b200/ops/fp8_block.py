"""Block-scaled 8-bit (e4m3) numerics: 1 x 128 scales for activations and gradients, 128 x 128 scales for weights.

This module is the NUMERICS of that recipe and its oracle, not yet its speed: operands are quantised to e4m3 with
per-block scales and de-quantised again, and the products run on the bf16 / fp32 GEMMs (``LME_FP8_SCALING=block``
together with ``mixed_precision_args.dtype: fp8``).  The 8-bit tensor-core kernel that applies the scales per
128-element K block is not built; ``block_scaled_matmul_reference`` states what it has to compute.

Per GEMM of a linear layer, with the contraction dimension named first:
  forward   y  = x W^T      x rows in 1 x 128 blocks along K,       W in 128 x 128 tiles
  dgrad     dx = dy W       dy rows in 1 x 128 blocks along N,      the same W tiles (read transposed)
  wgrad     dW = dy^T x     dy and x in 128 x 1 blocks along the token axis (re-quantised: the blocks of the
                            forward pass run along the wrong axis for this product)
"""

from __future__ import annotations

import torch

BLOCK = 128
E4M3_MAX = 448.0
_F8 = torch.float8_e4m3fn


def _blocks_last_dim(x: torch.Tensor) -> torch.Tensor:
    assert x.size(-1) % BLOCK == 0, f"last dimension {x.size(-1)} is not a multiple of {BLOCK}"
    return x.float().reshape(*x.shape[:-1], x.size(-1) // BLOCK, BLOCK)


def quantize_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [..., K]`` -> ``(q e4m3 [..., K], scale_inv fp32 [..., K / 128])`` with ``x ~ q * scale_inv`` per 1 x 128
    block (the scale maps the block's absolute maximum onto the largest e4m3 value)."""
    xb = _blocks_last_dim(x)
    amax = xb.abs().amax(-1).clamp_min(1e-12)
    scale = E4M3_MAX / amax
    q = (xb * scale[..., None]).to(_F8).reshape(x.shape)
    return q, 1.0 / scale


def dequantize_rows(q: torch.Tensor, scale_inv: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    qb = q.float().reshape(*q.shape[:-1], q.size(-1) // BLOCK, BLOCK)
    return (qb * scale_inv[..., None]).reshape(q.shape).to(dtype)


def quantize_tiles(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` -> ``(q e4m3 [N, K], scale_inv fp32 [N / 128, K / 128])``, one scale per 128 x 128 tile."""
    N, K = w.shape
    assert N % BLOCK == 0 and K % BLOCK == 0, f"weight {N} x {K} is not made of {BLOCK} x {BLOCK} tiles"
    t = w.float().reshape(N // BLOCK, BLOCK, K // BLOCK, BLOCK)
    amax = t.abs().amax((1, 3)).clamp_min(1e-12)
    scale = E4M3_MAX / amax
    q = (t * scale[:, None, :, None]).to(_F8).reshape(N, K)
    return q, 1.0 / scale


def dequantize_tiles(q: torch.Tensor, scale_inv: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    N, K = q.shape
    t = q.float().reshape(N // BLOCK, BLOCK, K // BLOCK, BLOCK) * scale_inv[:, None, :, None]
    return t.reshape(N, K).to(dtype)


def block_scaled_matmul_reference(xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    """What the block-scaled kernel computes, K block by K block: ``y[m, n] = sum_kb sx[m, kb] * sw[n / 128, kb] *
    sum_{k in kb} xq[m, k] wq[n, k]`` with the inner sums exact in fp32 (``xq [M, K]``, ``wq [N, K]``)."""
    M, K = xq.shape
    N = wq.size(0)
    y = torch.zeros((M, N), dtype=torch.float32, device=xq.device)
    xf, wf = xq.float(), wq.float()
    for kb in range(K // BLOCK):
        part = xf[:, kb * BLOCK:(kb + 1) * BLOCK] @ wf[:, kb * BLOCK:(kb + 1) * BLOCK].t()
        y += part * sx[:, kb, None] * sw[:, kb].repeat_interleave(BLOCK)[None, :]
    return y


def fake_quant_rows(x: torch.Tensor) -> torch.Tensor:
    """``x`` rounded to what the 1 x 128 e4m3 representation holds, in ``x``'s dtype."""
    q, s = quantize_rows(x)
    return dequantize_rows(q, s, x.dtype)


def fake_quant_tiles(w: torch.Tensor) -> torch.Tensor:
    q, s = quantize_tiles(w)
    return dequantize_tiles(q, s, w.dtype)


def fake_quant_token_axis(x2: torch.Tensor) -> torch.Tensor:
    """Blocks of 128 TOKENS per feature (the contraction axis of the weight gradient); a last partial block is
    scaled on its own."""
    T = x2.size(0)
    pad = (-T) % BLOCK
    xt = torch.nn.functional.pad(x2, (0, 0, 0, pad)).t().contiguous()
    return fake_quant_rows(xt).t()[:T].contiguous()


def block_eligible(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return weight.dim() == 2 and weight.size(0) % BLOCK == 0 and weight.size(1) % BLOCK == 0


class _LinearBlockScaled(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        from .gemm import linear

        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        wq = fake_quant_tiles(weight)
        y = linear(fake_quant_rows(x2), wq, bias)
        ctx.save_for_backward(x2, wq, weight)
        ctx.in_shape, ctx.has_bias = shape, bias is not None
        return y.view(*shape[:-1], weight.size(0))

    @staticmethod
    def backward(ctx, dy):
        from .gemm import _wgrad_into, linear

        x2, wq, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = linear(fake_quant_rows(dy2), wq.t().contiguous()).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dyq, xq = fake_quant_token_axis(dy2), fake_quant_token_axis(x2)
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None and dy2.is_cuda:      # the sharding engine's gradient buffer (see ops/gemm.py)
                _wgrad_into(main_grad, weight, dyq, xq)
            else:
                dw = linear(dyq.t().contiguous(), xq.t().contiguous()).to(wq.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy.dtype)
        return dx, dw, db


def linear_block_scaled(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                        residual: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear`` whose three products see 1 x 128 / 128 x 128 block-scaled e4m3 operands (module docstring)."""
    y = _LinearBlockScaled.apply(x, weight, bias)
    return y if residual is None else y + residual
