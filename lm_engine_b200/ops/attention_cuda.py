"""Binding of the tcgen05 flash-attention forward kernel (csrc/kernels/attention.cu): head dim 128, bf16, causal or
full, grouped K/V heads, log-sum-exp output.

There is no backward kernel yet, so the dispatcher in :mod:`lm_engine_b200.ops.attention` takes this path only where
no gradient is recorded - evaluation, generation prefill, and the first forward pass of a block under activation
checkpointing (which runs under ``no_grad``; the recomputation and the backward use the library kernel) - and only
when ``LME_ATTENTION=own`` asks for it: it is not yet faster than the library forward."""

from __future__ import annotations

import os

import torch

from . import _lib


def enabled() -> bool:
    return os.environ.get("LME_ATTENTION", "") == "own"


def shapes_supported(q, k, v) -> bool:
    return (q.is_cuda and q.dim() == 4 and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and v.dtype == torch.bfloat16 and q.size(-1) == 128 and v.size(-1) == 128
            and q.size(1) % 128 == 0 and k.size(1) % 128 == 0 and k.size(1) >= q.size(1)
            and q.size(2) % k.size(2) == 0 and k.size(2) == v.size(2))


def supports(q, k, v, *, causal, sliding_window, attention_mask, cu_seqlens, dropout_p) -> bool:
    if not enabled() or not shapes_supported(q, k, v):
        return False
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if causal and q.size(1) != k.size(1):
        return False
    return (not needs_grad and attention_mask is None and dropout_p == 0 and sliding_window is None
            and cu_seqlens is None)


def _token_major(t: torch.Tensor) -> torch.Tensor:
    """[B, S, H, 128] with heads contiguous inside a token and batches back to back (any token pitch), else a copy."""
    B, S, H, D = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == D and t.stride(1) % 8 == 0 and (B == 1 or t.stride(0) == S * t.stride(1))
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def flash_attention_forward(q, k, v, *, causal: bool, softmax_scale: float, return_lse: bool = False):
    q, k, v = _token_major(q), _token_major(k), _token_major(v)
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.size(1), k.size(2)
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    _lib.check(_lib.cuda_lib().lme_attention_fwd(q.data_ptr(), q.stride(1), k.data_ptr(), k.stride(1), v.data_ptr(),
                                                 v.stride(1), out.data_ptr(), Hq * D, _lib.ptr(lse), B, Sq, Skv, Hq,
                                                 Hkv, int(causal), float(softmax_scale), _lib.stream_ptr()),
               f"lme_attention_fwd B={B} Sq={Sq} Skv={Skv} Hq={Hq} Hkv={Hkv}")
    _lib.count_launch()
    return (out, lse) if return_lse else out


def flash_attention(q, k, v, *, causal, softmax_scale, sliding_window=None, cu_seqlens=None, max_seqlen=None):
    assert sliding_window is None and cu_seqlens is None
    return flash_attention_forward(q, k, v, causal=causal, softmax_scale=softmax_scale)
