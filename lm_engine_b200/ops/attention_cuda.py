"""Binding of the sm_100a flash-attention kernels (forward / backward, GQA, causal, LSE output)."""

from __future__ import annotations

import torch

from . import _lib

_ENABLED = False  # switched on once the kernels are built into liblme_cuda.so


def supports(q, k, v, *, causal, sliding_window, attention_mask, cu_seqlens, dropout_p) -> bool:
    if not _ENABLED:
        return False
    return (q.dtype == torch.bfloat16 and q.size(-1) in (64, 128) and attention_mask is None and dropout_p == 0
            and sliding_window is None and cu_seqlens is None and q.dim() == 4 and q.size(1) == k.size(1))


def flash_attention(q, k, v, *, causal, softmax_scale, sliding_window=None, cu_seqlens=None, max_seqlen=None):
    raise NotImplementedError
