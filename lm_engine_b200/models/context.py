"""Per-forward shared state handed to every block: attention-mask info, position info, generation cache.

``AttentionMaskInfo`` / ``PositionInfo`` keep the reference's names and fields
(lm_engine/modeling_utils/attention_mask_info.py:13-124, lm_engine/modeling_utils/position_embedding/info.py:13-52);
the cache is a per-layer dictionary of named states with two update rules: *append* along the sequence (attention
K/V) and *replace* (convolution windows, recurrent states) - the roles of ``LinearCache`` / ``ConstantCache`` in
lm_engine/generation_cache/*.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class AttentionMaskInfo:
    attention_mask: torch.Tensor | None = None     # [B, S_total] 1 = token, 0 = padding
    cu_seqlens: torch.Tensor | None = None         # int32 [num_docs + 1] for packed batches
    max_seqlen: int | None = None
    _sdpa_mask: torch.Tensor | None = field(default=None, repr=False)

    def get_causal_mask(self, query_length: int, key_length: int, dtype: torch.dtype) -> torch.Tensor | None:
        """Additive ``[B, 1, q, k]`` mask combining causality with padding (None when there is no padding).  Rows
        that would be fully masked are zeroed so softmax stays finite."""
        if self.attention_mask is None:
            return None
        B = self.attention_mask.size(0)
        m = self._sdpa_mask
        if m is not None and m.shape == (B, 1, query_length, key_length) and m.dtype == dtype:
            return m
        dev = self.attention_mask.device
        past = key_length - query_length
        qi = torch.arange(query_length, device=dev)[:, None] + past
        kj = torch.arange(key_length, device=dev)[None, :]
        allowed = (kj <= qi)[None] & self.attention_mask.bool()[:, None, :key_length]
        neg = torch.finfo(dtype).min
        add = torch.zeros(B, query_length, key_length, dtype=dtype, device=dev).masked_fill(~allowed, neg)
        add = add * allowed.any(-1, keepdim=True)
        self._sdpa_mask = add[:, None]
        return self._sdpa_mask

    def recurrent_mask(self, cache: "GenerationCache | None") -> torch.Tensor | None:
        """Padding mask for recurrent / convolutional mixers: only needed while prefilling a padded batch."""
        if self.attention_mask is None or cache is None or cache.get_seq_length() > 0:
            return None
        if bool(torch.all(self.attention_mask == 1)):
            return None
        return self.attention_mask


@dataclass
class PositionInfo:
    position_ids: torch.Tensor | None = None
    rope_cos_sin: tuple[torch.Tensor, torch.Tensor] | None = None     # gathered [.., rope_dim] (reference path)
    rope_tables: tuple[torch.Tensor, torch.Tensor] | None = None      # full fp32 tables (kernel path)
    sequence_length: int | None = None                                # global key length

    def fill(self, attention_mask: torch.Tensor | None, past_length: int, query_length: int, key_length: int,
             device: torch.device) -> None:
        from ..parallel.context_parallel import shard_sequence

        self.sequence_length = key_length
        if self.position_ids is not None:
            return
        if attention_mask is not None and attention_mask.dim() == 2:
            pos = attention_mask.long().cumsum(-1) - 1
            pos.masked_fill_(attention_mask == 0, 0)
            if past_length > 0:
                pos = pos[:, past_length:key_length]
        else:
            pos = torch.arange(past_length, key_length, dtype=torch.long, device=device).view(-1, query_length)
        self.position_ids = shard_sequence((pos,), seq_dim=1)[0]


def resolve_attention_and_position_info(a: AttentionMaskInfo | None, p: PositionInfo | None):
    return (a if a is not None else AttentionMaskInfo()), (p if p is not None else PositionInfo())


class GenerationCache:
    APPEND, REPLACE = "append", "replace"

    def __init__(self) -> None:
        self.layers: dict[int, dict[str, torch.Tensor]] = {}
        self._seen: dict[int, int] = {}

    def update(self, layer_idx: int, name: str, state: torch.Tensor | None, rule: str = APPEND, seq_dim: int = 1,
               num_tokens_added: int | None = None) -> torch.Tensor | None:
        slot = self.layers.setdefault(layer_idx, {})
        if rule == self.APPEND:
            slot[name] = state if name not in slot else torch.cat((slot[name], state), dim=seq_dim)
            if name in ("key", "k"):
                self._seen[layer_idx] = slot[name].size(seq_dim)
        else:
            if state is not None:
                slot[name] = state
            if num_tokens_added:
                self._seen[layer_idx] = self._seen.get(layer_idx, 0) + num_tokens_added
        return slot.get(name)

    def get(self, layer_idx: int, name: str) -> torch.Tensor | None:
        return self.layers.get(layer_idx, {}).get(name)

    def get_seq_length(self, layer_idx: int | None = None) -> int:
        if not self._seen:
            return 0
        if layer_idx is None:
            layer_idx = min(self._seen)
        return self._seen.get(layer_idx, 0)

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        for slot in self.layers.values():
            for k, v in slot.items():
                slot[k] = v.index_select(0, beam_idx.to(v.device))

    def __len__(self) -> int:
        return len(self.layers)
