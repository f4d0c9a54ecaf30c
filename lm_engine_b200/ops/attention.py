"""Softmax attention with GQA, causal / sliding-window masking, packed (varlen) batches and LSE output.

``attention()`` dispatches to the hand-written sm_100a kernel when it covers the case and to PyTorch SDPA otherwise;
``attention_reference()`` is the explicit-mask fp32 statement used as CPU path and oracle.  Covers what the
reference reaches through flash-attn / SDPA
(lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/flash_attention.py:37-225,
softmax_attention/module.py:248-259).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _band_mask(q_len: int, k_len: int, causal: bool, window: int | None, device) -> torch.Tensor | None:
    """Boolean [q_len, k_len] mask (True = attend); queries are aligned to the end of the keys."""
    if not causal and window is None:
        return None
    qi = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
    kj = torch.arange(k_len, device=device)[None, :]
    m = torch.ones(q_len, k_len, dtype=torch.bool, device=device)
    if causal:
        m &= kj <= qi
    if window is not None:
        m &= kj > qi - window if causal else (kj - qi).abs() < window
    return m


def attention_reference(q, k, v, *, causal=True, softmax_scale=None, sliding_window=None, attention_mask=None,
                        cu_seqlens=None, dropout_p=0.0, return_lse=False):
    """q ``[B, Sq, Hq, D]``, k/v ``[B, Sk, Hkv, D]`` (or packed ``[T, H, D]`` with ``cu_seqlens``).
    ``attention_mask``: ``[B, Sk]`` 1 = real token (left or right padding)."""
    if cu_seqlens is not None:
        outs, lses = [], []
        bounds = cu_seqlens.tolist()
        for a, b in zip(bounds[:-1], bounds[1:]):
            o = attention_reference(q[None, a:b], k[None, a:b], v[None, a:b], causal=causal,
                                    softmax_scale=softmax_scale, sliding_window=sliding_window,
                                    dropout_p=dropout_p, return_lse=return_lse)
            if return_lse:
                outs.append(o[0][0]); lses.append(o[1][0])
            else:
                outs.append(o[0])
        out = torch.cat(outs, 0)
        return (out, torch.cat(lses, 0)) if return_lse else out
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.size(1), k.size(2)
    scale = softmax_scale if softmax_scale is not None else 1 / math.sqrt(D)
    G = Hq // Hkv
    qf = q.float().transpose(1, 2)                                   # [B, Hq, Sq, D]
    kf = k.float().transpose(1, 2).repeat_interleave(G, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(G, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale               # [B, Hq, Sq, Sk]
    band = _band_mask(Sq, Sk, causal, sliding_window, q.device)
    if band is not None:
        s = s.masked_fill(~band, float("-inf"))
    if attention_mask is not None:
        s = s.masked_fill(~attention_mask.bool()[:, None, None, :], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                 # [B, Hq, Sq]
    p = torch.exp(s - lse.masked_fill(lse == float("-inf"), 0)[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0:
        p = F.dropout(p, dropout_p)
    out = torch.matmul(p, vf).transpose(1, 2).to(q.dtype)           # [B, Sq, Hq, D]
    return (out, lse.transpose(1, 2)) if return_lse else out


def _sdpa(q, k, v, causal, scale, dropout_p):
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         dropout_p=dropout_p, is_causal=causal, scale=scale,
                                         enable_gqa=q.size(2) != k.size(2))
    return out.transpose(1, 2)


def _flash_attn_varlen_usable(q: torch.Tensor) -> bool:
    if q.dtype not in (torch.bfloat16, torch.float16) or q.size(-1) > 256:
        return False
    try:
        import flash_attn  # noqa: F401
    except Exception:  # noqa: BLE001
        return False
    return True


def _flash_attn_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale, sliding_window, dropout_p):
    """Packed sequences on the GPU through the flash-attn library kernel (what the reference calls for its
    padding-free path, lm_engine/modeling_utils/sequence_mixer_blocks/softmax_attention/utils.py); the PyTorch
    statement would loop over the sequences and materialise their score matrices."""
    from flash_attn import flash_attn_varlen_func

    cu = cu_seqlens.to(torch.int32)
    if max_seqlen is None:
        max_seqlen = int((cu[1:] - cu[:-1]).max())
    window = (-1, -1) if sliding_window is None else ((sliding_window - 1, 0) if causal
                                                      else (sliding_window - 1, sliding_window - 1))
    return flash_attn_varlen_func(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, max_seqlen, max_seqlen,
                                  dropout_p=dropout_p, softmax_scale=scale, causal=causal, window_size=window)


def attention(q, k, v, *, causal=True, softmax_scale=None, sliding_window=None, attention_mask=None,
              cu_seqlens=None, max_seqlen=None, dropout_p=0.0):
    """Returns ``[B, Sq, Hq, D]`` (or packed ``[T, Hq, D]``)."""
    from . import attention_cuda

    D = q.size(-1)
    scale = softmax_scale if softmax_scale is not None else 1 / math.sqrt(D)
    if q.is_cuda and attention_cuda.supports(q, k, v, causal=causal, sliding_window=sliding_window,
                                             attention_mask=attention_mask, cu_seqlens=cu_seqlens,
                                             dropout_p=dropout_p):
        return attention_cuda.flash_attention(q, k, v, causal=causal, softmax_scale=scale,
                                              sliding_window=sliding_window, cu_seqlens=cu_seqlens,
                                              max_seqlen=max_seqlen)
    if q.is_cuda:
        from ..logging_utils.logger import warn_once

        why = attention_cuda.why_unsupported(q, k, v, causal=causal, sliding_window=sliding_window,
                                             attention_mask=attention_mask, cu_seqlens=cu_seqlens,
                                             dropout_p=dropout_p)
        warn_once(f"attention-fallback-{why}", f"attention: the tcgen05 kernels do not take this case ({why}); "
                  "it runs on a library kernel or on the PyTorch statement")
    if cu_seqlens is not None and q.is_cuda and attention_mask is None and _flash_attn_varlen_usable(q):
        return _flash_attn_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale, sliding_window, dropout_p)
    if (sliding_window is not None and q.is_cuda and attention_mask is None and cu_seqlens is None
            and (q.size(1) == k.size(1) or not causal) and _flash_attn_varlen_usable(q)):
        # windows the tcgen05 kernels do not take (head dim != 128, ragged lengths): the library's windowed kernel
        from flash_attn import flash_attn_func

        window = (sliding_window - 1, 0) if causal else (sliding_window - 1, sliding_window - 1)
        return flash_attn_func(q, k, v, dropout_p=dropout_p, softmax_scale=scale, causal=causal, window_size=window)
    plain = sliding_window is None and attention_mask is None and cu_seqlens is None
    if plain and (q.size(1) == k.size(1) or not causal):
        return _sdpa(q, k, v, causal, scale, dropout_p)
    return attention_reference(q, k, v, causal=causal, softmax_scale=scale, sliding_window=sliding_window,
                               attention_mask=attention_mask, cu_seqlens=cu_seqlens, dropout_p=dropout_p)
