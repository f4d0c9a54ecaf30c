"""Pretraining wrapper: a batch is ``[micro_batch, sequence_length + 1]`` token ids; inputs are ``t[:, :-1]``, labels
``t[:, 1:]`` (no shift inside the loss), both context-parallel sharded.  Padding-free mode flattens the batch and
can restart attention / positions at EOS (lm_engine/model_wrapper/pretraining.py:26-285).
"""

from __future__ import annotations

import torch

from ..models import AttentionMaskInfo, PipelineParallelInput, PositionInfo
from ..models.base import CausalLMOutputWithPast
from ..loss import is_aux_loss_zero
from ..parallel.context_parallel import shard_sequence
from ..parallel.manager import ProcessGroupManager
from ..parallel.tensor_parallel import broadcast_tensor_parallel_input
from .base import ModelWrapper


class ModelWrapperForPretraining(ModelWrapper):
    def __init__(self, *args, micro_batch_size: int, sequence_length: int, reset_attention_mask: bool = False,
                 reset_position_ids: bool = False, **kwargs) -> None:
        self.micro_batch_size, self.sequence_length = micro_batch_size, sequence_length
        self.reset_attention_mask, self.reset_position_ids = reset_attention_mask, reset_position_ids
        super().__init__(*args, **kwargs)
        if not self.use_padding_free_transformer:
            assert not reset_attention_mask, "reset_attention_mask is only implemented for padding free transformer"
            assert not reset_position_ids, "reset_position_ids is only implemented for padding free transformer"
        elif reset_position_ids:
            assert reset_attention_mask, "reset_attention_mask should be specified with reset_position_ids"
        self._static: dict[str, torch.Tensor] = {}

    def forward(self, batch: dict | torch.Tensor, aux_loss_from_pipeline_parallel: torch.Tensor | float = 0,
                lm_loss_multiplier: float = 1):
        if isinstance(batch, torch.Tensor):
            batch = {"text": batch}
        if self.is_pipeline_parallel_enabled:
            return self._forward_pipeline_stage(batch["text"], aux_loss_from_pipeline_parallel)
        assert is_aux_loss_zero(aux_loss_from_pipeline_parallel)
        inputs, labels = self._prepare_model_inputs(batch)
        out = self.model(**inputs, skip_logits=self.skip_logits())
        return self.get_loss(out, labels, shift_logits_and_labels=False, lm_loss_multiplier=lm_loss_multiplier)

    # ------------------------------------------------------------------ pipeline stages exchange raw tensors
    def forward_pipeline_stage(self, tokens: torch.Tensor | None, hidden_in: torch.Tensor | None, aux_in=0):
        """One micro-batch through this stage.  The first stage embeds ``tokens[:, :-1]``; later stages continue from
        ``hidden_in`` (and the auxiliary loss accumulated so far).  Returns ``(hidden, aux_loss)``, or the loss dict on
        the last stage, whose labels are ``tokens[:, 1:]``."""
        device = next(self.model.parameters()).device if self.engine is None else self.engine.device
        tp = ProcessGroupManager.is_tensor_parallel_enabled()
        if self.is_first_stage:
            (ids,) = shard_sequence((tokens[:, :-1].to(device),), seq_dim=1)
            kw = dict(input_ids=ids)
        else:
            kw = dict(pipeline_parallel_input=PipelineParallelInput(hidden_states=hidden_in, aux_loss=aux_in))
        if not self.is_last_stage:
            out = self.model(**kw)
            return out.hidden_states, out.aux_loss
        out = self.model(**kw, output_parallel_lm_logits=tp, skip_logits=self.skip_logits())
        (labels,) = shard_sequence((tokens[:, 1:].to(device),), seq_dim=1)
        cp = ProcessGroupManager.get_context_parallel_world_size()
        return self.get_loss(out, labels, shift_logits_and_labels=False,
                             lm_loss_multiplier=1 / (self.micro_batch_size * self.sequence_length / cp))

    def _forward_pipeline_stage(self, tokens: torch.Tensor, aux_in):
        """Reference-shaped entry: a stage called with the raw tensor of its predecessor returns raw tensors."""
        if self.is_first_stage:
            hidden, aux = self.forward_pipeline_stage(tokens, None)
        else:
            out = self.model(pipeline_parallel_input=PipelineParallelInput(hidden_states=tokens, aux_loss=aux_in),
                             output_parallel_lm_logits=ProcessGroupManager.is_tensor_parallel_enabled())
            aux = out.aux_loss
            hidden = out.logits if isinstance(out, CausalLMOutputWithPast) else out.hidden_states
        if is_aux_loss_zero(aux):
            return hidden
        return hidden, (aux.unsqueeze(0) if aux.dim() == 0 else aux)

    # ------------------------------------------------------------------ inputs
    def _prepare_model_inputs(self, batch: dict) -> tuple[dict, torch.Tensor]:
        tokens = None if batch is None else batch["text"]
        tokens = broadcast_tensor_parallel_input(tokens, (self.micro_batch_size, self.sequence_length + 1))
        ids, labels = tokens[:, :-1], tokens[:, 1:]
        ids, labels = shard_sequence((ids, labels), seq_dim=1)
        inputs: dict = {}
        if self.use_padding_free_transformer:
            assert not ProcessGroupManager.is_context_parallel_enabled()
            B, S = ids.shape
            ids = ids.reshape(-1)
            dev = ids.device
            if self.reset_attention_mask:
                ends = ids == self.eos_token_id
                ends[S - 1::S] = True
                cu = torch.cat((torch.zeros(1, dtype=torch.long, device=dev), ends.nonzero(as_tuple=True)[0] + 1))
                lens = cu[1:] - cu[:-1]
                max_seqlen = int(lens.max())
                if self.reset_position_ids:
                    pos = torch.arange(B * S, device=dev) - torch.repeat_interleave(cu[:-1], lens)
                else:
                    pos = self._cached("pos", lambda: torch.arange(S, device=dev).repeat(B))
                cu = cu.to(torch.int32)
            else:
                cu = self._cached("cu", lambda: torch.arange(0, B * S + 1, S, dtype=torch.int32, device=dev))
                pos = self._cached("pos", lambda: torch.arange(S, device=dev).repeat(B))
                max_seqlen = S
            inputs["attention_mask_info"] = AttentionMaskInfo(cu_seqlens=cu, max_seqlen=max_seqlen)
            inputs["position_info"] = PositionInfo(position_ids=pos)
        inputs["input_ids"] = ids
        if ProcessGroupManager.is_tensor_parallel_enabled():
            inputs["output_parallel_lm_logits"] = True
        return inputs, labels

    def _cached(self, key: str, make):
        if key not in self._static:
            self._static[key] = make()
        return self._static[key]
