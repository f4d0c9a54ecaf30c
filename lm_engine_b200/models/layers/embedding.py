"""Token embedding (optionally vocab-parallel) and the LM head that shares its weight layout.

Under tensor parallelism the vocabulary is padded up to a multiple of 64 and split over ranks; out-of-range ids
contribute zeros and the partial results are summed (reduce-scatter to the sequence-parallel layout or all-reduce),
as in lm_engine/modeling_utils/embedding.py:22-92 and lm_engine/modeling_utils/lm_head.py:15-84.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...parallel import tp_comm
from ...parallel.manager import ProcessGroupManager
from ...parameter import mark_parameter_as_initialized, mark_tp_shard
from ...utils import ceil_divide


def get_tensor_parallel_vocab_info(vocab_size: int, make_vocab_size_divisible_by: int = 64) -> tuple[int, int, int]:
    """(first id, one-past-last id, padded per-rank size) of this TP rank's vocabulary slice."""
    tp = ProcessGroupManager.get_tensor_parallel_world_size()
    rank = ProcessGroupManager.get_tensor_parallel_rank()
    multiple = make_vocab_size_divisible_by * tp
    padded = ceil_divide(vocab_size, multiple) * multiple
    per_rank = padded // tp
    start = rank * per_rank
    return start, min(start + per_rank, vocab_size), per_rank


class ParameterizedEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, std: float | None = None,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.std = num_embeddings, embedding_dim, std
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.tp_world_size = ProcessGroupManager.get_tensor_parallel_world_size()
        if self.tp_world_size > 1:
            self.vocab_start, self.vocab_end, rows = get_tensor_parallel_vocab_info(num_embeddings)
        else:
            self.vocab_start, self.vocab_end, rows = 0, num_embeddings, num_embeddings
        self.weight = nn.Parameter(torch.empty(rows, embedding_dim))
        if self.tp_world_size > 1:
            mark_tp_shard(self.weight, 0, (rows * self.tp_world_size, embedding_dim))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.weight.is_meta:
            return
        nn.init.normal_(self.weight, mean=0, std=1 if self.std is None else self.std)
        mark_parameter_as_initialized(self.weight)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        from ...ops.embedding import embedding

        if self.tp_world_size == 1:
            return embedding(input_ids, self.weight) if self.weight.is_cuda else F.embedding(input_ids, self.weight)
        x = embedding(input_ids, self.weight, self.vocab_start, self.vocab_end)
        if self.sequence_parallel:
            return tp_comm.scatter_to_sequence_parallel(x, tp_comm.seq_dim(x, self.use_padding_free_transformer))
        return tp_comm.reduce_from_tensor_parallel(x)

    # ---- use of the matrix as an output projection (LM head, or tied embeddings)
    def _tp_input(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_world_size > 1:
            if self.sequence_parallel:
                return tp_comm.gather_from_sequence_parallel(x, tp_comm.seq_dim(x, self.use_padding_free_transformer))
            return tp_comm.copy_to_tensor_parallel(x)
        return x

    def compute_with_weight(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return ops.linear(self._tp_input(x), weight)

    def loss_with_weight(self, x: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, **kw) -> torch.Tensor:
        from ...loss import get_autoregressive_language_modeling_loss

        return get_autoregressive_language_modeling_loss(
            lm_logits=None, labels=labels, hidden_states=self._tp_input(x), vocab_weight=weight,
            tensor_parallel_enabled=self.tp_world_size > 1, vocab_size=self.num_embeddings, **kw)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}"


class LMHead(ParameterizedEmbedding):
    """Projects hidden states onto the (local slice of the) vocabulary; logits stay vocab-sharded under TP."""

    def forward(self, x: torch.Tensor, labels: torch.Tensor | None = None,
                loss_kwargs: dict | None = None) -> torch.Tensor:
        """Logits, or - when ``labels`` are given - the summed cross entropy computed chunk by chunk so that the
        full logits never exist (the weight is only guaranteed to be materialised inside this call)."""
        if labels is None:
            return self.compute_with_weight(x, self.weight)
        return self.loss_with_weight(x, self.weight, labels, **(loss_kwargs or {}))

