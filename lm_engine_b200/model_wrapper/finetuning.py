"""Finetuning wrapper: a batch is ``input_ids`` / ``labels`` (+ ``attention_mask`` for padded batches, or
``cu_seqlens`` / ``max_seqlen`` / ``position_ids`` for packed ones); the loss shifts logits against labels and masks
label ``-100`` (lm_engine/model_wrapper/finetuning.py:19-105).

Only the first rank of a tensor-parallel group reads data; the others receive the batch by broadcast.  Shapes travel
first as one small int64 tensor so that the receiving ranks can allocate, then every field is broadcast in place.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..kernels import is_fused_linear_cross_entropy_enabled
from ..models import AttentionMaskInfo, PositionInfo
from ..parallel.manager import ProcessGroupManager
from .base import ModelWrapper

_PACKED_KEYS = ("input_ids", "position_ids", "labels", "cu_seqlens", "max_seqlen")
_PADDED_KEYS = ("input_ids", "attention_mask", "labels")


class ModelWrapperForFinetuning(ModelWrapper):
    def forward(self, batch: dict, lm_loss_multiplier: float = 1) -> dict:
        assert not ProcessGroupManager.is_context_parallel_enabled(), "finetuning does not shard the sequence"
        batch = dict(self._broadcast_inputs_for_tensor_parallel(batch))
        labels = batch.pop("labels")
        cu_seqlens = batch.pop("cu_seqlens", None)
        max_seqlen = batch.pop("max_seqlen", None)
        if isinstance(max_seqlen, torch.Tensor):
            max_seqlen = int(max_seqlen)
        mask_info = AttentionMaskInfo(attention_mask=batch.pop("attention_mask", None), cu_seqlens=cu_seqlens,
                                      max_seqlen=max_seqlen)
        pos_info = PositionInfo(position_ids=batch.pop("position_ids", None))
        extra = {"output_parallel_lm_logits": True} if ProcessGroupManager.is_tensor_parallel_enabled() else {}
        out = self.model(input_ids=batch["input_ids"], attention_mask_info=mask_info, position_info=pos_info,
                         skip_logits=self.skip_logits(), **extra)
        return self.get_loss(out, labels, shift_logits_and_labels=True, cu_seqlens=cu_seqlens,
                             lm_loss_multiplier=lm_loss_multiplier)

    def skip_logits(self) -> bool:
        return is_fused_linear_cross_entropy_enabled() and not ProcessGroupManager.is_tensor_parallel_enabled()

    def _broadcast_inputs_for_tensor_parallel(self, batch: dict | None) -> dict:
        if not ProcessGroupManager.is_tensor_parallel_enabled():
            return batch
        group = ProcessGroupManager.get_tensor_parallel_group()
        src = ProcessGroupManager.get_tensor_parallel_first_rank()
        first = ProcessGroupManager.is_tensor_parallel_first_rank()
        device = self.engine.device if self.engine is not None else next(self.model.parameters()).device
        keys = _PACKED_KEYS if self.use_padding_free_transformer else _PADDED_KEYS
        # header: per key (ndim, d0, d1) -- every field is at most 2-D
        header = torch.zeros(len(keys) * 3, dtype=torch.long, device=device)
        if first:
            batch = {k: torch.as_tensor(batch[k]).to(device) for k in keys}
            for i, k in enumerate(keys):
                shp = list(batch[k].shape)
                header[3 * i] = len(shp)
                for j, s in enumerate(shp):
                    header[3 * i + 1 + j] = s
        dist.broadcast(header, src=src, group=group)
        if not first:
            h = header.tolist()
            batch = {}
            for i, k in enumerate(keys):
                shape = tuple(h[3 * i + 1:3 * i + 1 + h[3 * i]])
                dtype = torch.int32 if k == "cu_seqlens" else torch.long
                batch[k] = torch.empty(shape, dtype=dtype, device=device)
        for k in keys:
            t = batch[k]
            if k == "cu_seqlens" and t.dtype != torch.int32:
                t = batch[k] = t.to(torch.int32)
            dist.broadcast(t, src=src, group=group)
        return batch
