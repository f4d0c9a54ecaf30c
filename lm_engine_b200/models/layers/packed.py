"""Packed-token (padding-free) inputs for the batch-shaped mixers.

The convolution and scan code of the recurrent mixers works on ``[B, S, ...]`` batches.  With packed tokens ``[T, ...]``
and ``cu_seqlens`` the token-wise projections stay on the packed rows and only the tensors that enter the convolution /
scan are moved into a left-padded batch ``[num_sequences, max_seqlen, ...]`` and back (row-copy kernels on CUDA).
Padded steps carry zero inputs and start from a zero state, which every recurrence here maps to a zero state again, so
one batched scan gives each sequence exactly what a scan of that sequence alone gives.
Role of pack_sequence / unpack_sequence around the varlen kernels in the reference
(lm_engine/modeling_utils/sequence_mixer_blocks/rnn/module.py:150-205, m2rnn/module.py:213-306).
"""

from __future__ import annotations

import torch

from ...ops.packing import pack_sequence, unpack_sequence


class PackedBatch:
    def __init__(self, cu_seqlens: torch.Tensor, max_seqlen: int | None, total_tokens: int) -> None:
        assert cu_seqlens is not None, "padding-free mixers need cu_seqlens"
        self.cu_seqlens = cu_seqlens
        self.num_sequences = cu_seqlens.numel() - 1
        lengths = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
        self.max_seqlen = int(max_seqlen) if max_seqlen is not None else int(lengths.max())
        self.total_tokens = total_tokens
        assert self.total_tokens <= self.num_sequences * self.max_seqlen, "max_seqlen is smaller than a sequence"
        # every sequence as long as the longest one: the packed rows already are the batch, nothing is padded
        self.dense = total_tokens == self.num_sequences * self.max_seqlen
        if self.dense:
            self.mask = None
        else:
            steps = torch.arange(self.max_seqlen, device=cu_seqlens.device)
            self.mask = (steps[None, :] >= (self.max_seqlen - lengths)[:, None]).to(torch.int64)   # left-padded

    @classmethod
    def of(cls, enabled: bool, info, x: torch.Tensor, cache_params) -> "PackedBatch | None":
        """The layout of packed input ``x [T, H]`` when the mixer runs padding-free, else None."""
        if not enabled:
            return None
        assert cache_params is None, "packed inputs are a training layout: no generation cache"
        assert x.dim() == 2, "padding-free mixers take packed tokens [T, H]"
        cached = getattr(info, "_packed_batch", None)      # one layout per forward pass, shared by the layers
        if cached is None or cached.total_tokens != x.size(0) or cached.cu_seqlens is not info.cu_seqlens:
            cached = cls(info.cu_seqlens, info.max_seqlen, x.size(0))
            info._packed_batch = cached
        return cached

    def unpack(self, t: torch.Tensor) -> torch.Tensor:
        """[T, ...] -> [num_sequences, max_seqlen, ...], zeros in front of the shorter sequences."""
        shape = (self.num_sequences, self.max_seqlen, *t.shape[1:])
        return t.reshape(shape) if self.dense else unpack_sequence(t, self.cu_seqlens, shape)

    def pack(self, t: torch.Tensor) -> torch.Tensor:
        if self.dense:
            return t.reshape(self.total_tokens, *t.shape[2:])
        return pack_sequence(t, self.cu_seqlens, self.total_tokens)
