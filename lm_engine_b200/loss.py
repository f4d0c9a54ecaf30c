"""Autoregressive language-modelling loss (lm_engine/loss.py:24-101) on top of the fused cross-entropy kernels.

``get_autoregressive_language_modeling_loss`` accepts either logits or (hidden states, vocabulary weight); the second
form computes the LM head in token chunks so the full ``[T, V]`` logits never exist at once (what the reference's
fused-linear-CE kernels provide).  Under tensor parallelism the logits are vocabulary slices and the loss runs
vocab-parallel.
"""

from __future__ import annotations

import torch

from . import ops
from .models.layers.embedding import get_tensor_parallel_vocab_info
from .parallel.manager import ProcessGroupManager

IGNORE_INDEX = -100


def _shift(logits_or_hidden: torch.Tensor, labels: torch.Tensor, cu_seqlens: torch.Tensor | None,
           padding_free: bool) -> tuple[torch.Tensor, torch.Tensor]:
    if padding_free:
        # packed: drop the first label of every document by masking the last position of the previous document
        x = logits_or_hidden[:-1]
        y = labels[1:].clone()
        if cu_seqlens is not None:
            ends = cu_seqlens[1:-1].long() - 1
            y[ends] = IGNORE_INDEX
        return x, y
    return logits_or_hidden[..., :-1, :], labels[..., 1:]


def get_autoregressive_language_modeling_loss(
    lm_logits: torch.Tensor | None,
    labels: torch.Tensor,
    hidden_states: torch.Tensor | None = None,
    vocab_weight: torch.Tensor | None = None,
    cu_seqlens: torch.Tensor | None = None,
    use_padding_free_transformer: bool = False,
    reduction: str = "sum",
    shift_logits_and_labels: bool = True,
    tensor_parallel_enabled: bool = False,
    vocab_size: int | None = None,
    logit_scale: float | None = None,
    chunk_tokens: int = 8192,
) -> torch.Tensor:
    assert reduction in ("sum", "mean")
    x = lm_logits if lm_logits is not None else hidden_states
    if shift_logits_and_labels:
        x, labels = _shift(x, labels, cu_seqlens, use_padding_free_transformer)
    labels = labels.reshape(-1)
    group, v0 = None, 0
    if tensor_parallel_enabled:
        group = ProcessGroupManager.get_tensor_parallel_group()
        v0 = get_tensor_parallel_vocab_info(vocab_size)[0] if vocab_size is not None else 0
    if lm_logits is not None:
        x = x.reshape(-1, x.size(-1))
        loss = ops.cross_entropy_sum(x, labels, IGNORE_INDEX, v0, group)
    else:
        h = x.reshape(-1, x.size(-1))
        loss = 0
        for a in range(0, h.size(0), chunk_tokens):
            logits = ops.linear(h[a:a + chunk_tokens], vocab_weight)
            if logit_scale is not None:
                logits = logits * logit_scale
            loss = loss + ops.cross_entropy_sum(logits, labels[a:a + chunk_tokens], IGNORE_INDEX, v0, group)
    if reduction == "mean":
        loss = loss / (labels != IGNORE_INDEX).sum().clamp(min=1)
    return loss


def is_aux_loss_zero(aux_loss) -> bool:
    return isinstance(aux_loss, (int, float)) and aux_loss == 0
