"""Binding of the tcgen05 flash-attention kernels (csrc/kernels/attention.cu, attention_bwd.cu): head dim 128, bf16,
causal or full, grouped K/V heads; forward with log-sum-exp output, backward as a dQ kernel and a dK / dV kernel
that own their output rows (no atomics, deterministic).

The kernels are opt-in (``LME_ATTENTION=own``): they are not yet as fast as the library kernels the default path
calls (cuDNN through ``scaled_dot_product_attention``)."""

from __future__ import annotations

import os

import torch

from . import _lib


def enabled() -> bool:
    return os.environ.get("LME_ATTENTION", "") == "own"


def shapes_supported(q, k, v, packed: bool = False) -> bool:
    """Batches ``[B, S, H, 128]`` with S a multiple of 128, or packed sequences ``[T, H, 128]`` of any lengths."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.size(-1) == 128 and v.size(-1) == 128 and q.size(-2) % k.size(-2) == 0
            and k.size(-2) == v.size(-2)):
        return False
    if packed:
        return q.dim() == 3 and q.size(0) == k.size(0)
    return q.dim() == 4 and q.size(1) % 128 == 0 and k.size(1) % 128 == 0 and k.size(1) >= q.size(1)


def supports(q, k, v, *, causal, sliding_window, attention_mask, cu_seqlens, dropout_p) -> bool:
    """The switch selects these kernels; causal sliding-window attention takes them regardless, because the library
    path has no windowed kernel and the alternative materialises the full score matrix."""
    packed = cu_seqlens is not None
    if not shapes_supported(q, k, v, packed) or attention_mask is not None or dropout_p != 0:
        return False
    if sliding_window is not None and not causal:
        return False
    if packed:                      # the default for packed sequences is the library's varlen kernel
        return enabled()
    if sliding_window is not None:
        return True
    return enabled() and (not causal or q.size(1) == k.size(1))


def why_unsupported(q, k, v, *, causal, sliding_window, attention_mask, cu_seqlens, dropout_p) -> str:
    """Short reason why :func:`supports` said no (for the one-time fallback warning)."""
    packed = cu_seqlens is not None
    if q.size(-1) != 128 or v.size(-1) != 128:
        return f"head dim {q.size(-1)}"
    if q.dtype != torch.bfloat16:
        return f"dtype {q.dtype}"
    if attention_mask is not None:
        return "padding mask"
    if dropout_p != 0:
        return "dropout"
    if sliding_window is not None and not causal:
        return "non-causal window"
    if not shapes_supported(q, k, v, packed):
        return "sequence length not a multiple of 128" if not packed else "packed layout"
    if not enabled():
        return "library kernels are the default, LME_ATTENTION=own selects the tcgen05 kernels"
    return "query / key lengths differ"


def _token_major(t: torch.Tensor) -> torch.Tensor:
    """[B, S, H, 128] with heads contiguous inside a token and batches back to back (any token pitch), else a copy."""
    B, S, H, D = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == D and t.stride(1) % 8 == 0 and (B == 1 or t.stride(0) == S * t.stride(1))
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def _packed_view(t: torch.Tensor) -> torch.Tensor:
    """[T, H, 128] packed tokens as a one-batch [1, T, H, 128] operand."""
    return _token_major(t.unsqueeze(0))


def _padded(n: int) -> int:
    return (n + 127) // 128 * 128


def flash_attention_forward(q, k, v, *, causal: bool, softmax_scale: float, return_lse: bool = False,
                            sliding_window: int | None = None, cu_seqlens: torch.Tensor | None = None,
                            max_seqlen: int | None = None, kv_ready: torch.Tensor | None = None,
                            kv_chunk_rows: int = 0, kv_seq: int = 0):
    """Batches ``[B, S, H, 128]``, or packed sequences ``[T, H, 128]`` with ``cu_seqlens`` (then the log-sum-exp is
    ``[sequences, Hq, padded max length]``).  ``kv_ready`` (int32 ``[B, chunks]``): chunks of ``kv_chunk_rows`` key /
    value rows are still arriving; the kernel waits for ``kv_seq`` in a chunk's word before it loads from it."""
    packed = cu_seqlens is not None
    if packed:
        cu = cu_seqlens.to(torch.int32).contiguous()
        if max_seqlen is None:
            max_seqlen = int((cu[1:] - cu[:-1]).max())
        q, k, v = _packed_view(q), _packed_view(k), _packed_view(v)
        T, Hq, D = q.shape[1:]
        B, Sq, Skv, Hkv = cu.numel() - 1, int(max_seqlen), int(max_seqlen), k.size(2)
        out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.zeros((B, Hq, _padded(Sq)), dtype=torch.float32, device=q.device) if return_lse else None
    else:
        cu, T = None, 0
        q, k, v = _token_major(q), _token_major(k), _token_major(v)
        B, Sq, Hq, D = q.shape
        Skv, Hkv = k.size(1), k.size(2)
        out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    _lib.check(_lib.cuda_lib().lme_attention_fwd(q.data_ptr(), q.stride(1), k.data_ptr(), k.stride(1), v.data_ptr(),
                                                 v.stride(1), out.data_ptr(), Hq * D, _lib.ptr(lse), B, Sq, Skv, Hq,
                                                 Hkv, int(causal), int(sliding_window or 0), float(softmax_scale),
                                                 _lib.ptr(cu), T, _lib.ptr(kv_ready), int(kv_chunk_rows),
                                                 int(kv_seq), _lib.stream_ptr()),
               f"lme_attention_fwd B={B} Sq={Sq} Skv={Skv} Hq={Hq} Hkv={Hkv} packed={packed}")
    _lib.count_launch()
    return (out, lse) if return_lse else out


def flash_attention_backward(dout, q, k, v, out, lse, *, causal: bool, softmax_scale: float,
                             sliding_window: int | None = None, cu_seqlens: torch.Tensor | None = None,
                             max_seqlen: int | None = None):
    """Returns contiguous ``(dq, dk, dv)`` for operands laid out as in the forward call."""
    packed = cu_seqlens is not None
    if packed:
        cu = cu_seqlens.to(torch.int32).contiguous()
        q, k, v, dout, out = (_packed_view(t) for t in (q, k, v, dout, out))
        T, Hq, D = q.shape[1:]
        B, Sq, Skv, Hkv = cu.numel() - 1, int(max_seqlen), int(max_seqlen), k.size(2)
        dq, dk, dv = q.new_empty((T, Hq, D)), k.new_empty((T, Hkv, D)), k.new_empty((T, Hkv, D))
    else:
        cu, T = None, 0
        q, k, v, dout, out = (_token_major(t) for t in (q, k, v, dout, out))
        B, Sq, Hq, D = q.shape
        Skv, Hkv = k.size(1), k.size(2)
        dq, dk, dv = q.new_empty((B, Sq, Hq, D)), k.new_empty((B, Skv, Hkv, D)), k.new_empty((B, Skv, Hkv, D))
    delta = torch.empty((B, Hq, _padded(Sq)), dtype=torch.float32, device=q.device)    # rowsum(dout * out), filled by the call
    _lib.check(_lib.cuda_lib().lme_attention_bwd(
        q.data_ptr(), q.stride(1), k.data_ptr(), k.stride(1), v.data_ptr(), v.stride(1), dout.data_ptr(),
        dout.stride(1), out.data_ptr(), out.stride(1), lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), Hq * D, dk.data_ptr(), Hkv * D,
        dv.data_ptr(), Hkv * D, B, Sq, Skv, Hq, Hkv, int(causal), int(sliding_window or 0), float(softmax_scale),
        _lib.ptr(cu), T, _lib.stream_ptr()),
        f"lme_attention_bwd B={B} Sq={Sq} Skv={Skv} Hq={Hq} Hkv={Hkv}")
    _lib.count_launch(3)
    return dq, dk, dv


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal: bool, scale: float, window: int | None = None, cu_seqlens=None,
                max_seqlen: int | None = None):
        if cu_seqlens is not None and max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        out, lse = flash_attention_forward(q, k, v, causal=causal, softmax_scale=scale, return_lse=True,
                                           sliding_window=window, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        ctx.save_for_backward(q, k, v, out, lse, *([cu_seqlens] if cu_seqlens is not None else []))
        ctx.cfg = (causal, scale, window, max_seqlen)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, *rest = ctx.saved_tensors
        causal, scale, window, max_seqlen = ctx.cfg
        dq, dk, dv = flash_attention_backward(dout, q, k, v, out, lse, causal=causal, softmax_scale=scale,
                                              sliding_window=window, cu_seqlens=rest[0] if rest else None,
                                              max_seqlen=max_seqlen)
        return dq, dk, dv, None, None, None, None, None


def flash_attention(q, k, v, *, causal, softmax_scale, sliding_window=None, cu_seqlens=None, max_seqlen=None):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _FlashAttention.apply(q, k, v, bool(causal), float(softmax_scale), sliding_window, cu_seqlens,
                                     max_seqlen)
    return flash_attention_forward(q, k, v, causal=causal, softmax_scale=softmax_scale, sliding_window=sliding_window,
                                   cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
