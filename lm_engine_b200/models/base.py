"""Model skeleton shared by all families: embeddings -> blocks of this pipeline stage -> final norm (-> LM head).

Module and parameter names are the checkpoint format of the reference (``transformer.wte``, ``transformer.h.{i}.*``,
``transformer.ln_f``, ``lm_head``; lm_engine/mixins/dense/base.py:29-275, lm_engine/mixins/dense/main.py:34-255).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..parallel import tp_comm
from ..parallel.manager import ProcessGroupManager
from ..utils import SafeTensorsWeightsManager, divide_if_divisible, is_generation_cache_enabled
from .aux_loss import add_aux_loss, clear_aux_loss, get_aux_loss
from .blocks import Block, LadderBlock, PaLMBlock
from .config import CommonConfig
from .context import AttentionMaskInfo, GenerationCache, PositionInfo, resolve_attention_and_position_info
from .layers.dropout import Dropout
from .layers.embedding import LMHead, ParameterizedEmbedding
from .layers.init_utils import std_for_embedding
from .layers.norm import get_normalization_function
from .layers.rope import RoPE, YaRNScaledRoPE


@dataclass
class BaseModelOutputWithPast:
    last_hidden_state: torch.Tensor | None = None
    cache_params: GenerationCache | None = None


@dataclass
class CausalLMOutputWithPast:
    loss: torch.Tensor | None = None
    aux_loss: torch.Tensor | float = 0
    logits: torch.Tensor | None = None
    cache_params: GenerationCache | None = None
    last_hidden_state: torch.Tensor | None = None


@dataclass
class PipelineParallelInput:
    hidden_states: torch.Tensor | None = None
    aux_loss: torch.Tensor | float = 0


@dataclass
class PipelineParallelOutput:
    hidden_states: torch.Tensor | None = None
    aux_loss: torch.Tensor | float = 0


class TransformerModel(nn.Module):
    """``transformer`` sub-module: embeddings, the blocks of one pipeline stage, final norm."""

    layer_class = Block

    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool = False,
                 sequence_parallel: bool = False, num_pipeline_stages: int = 1, pipeline_stage_id: int = 0) -> None:
        super().__init__()
        self.config = config
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.num_pipeline_stages, self.pipeline_stage_id = num_pipeline_stages, pipeline_stage_id
        self.is_first_stage = pipeline_stage_id == 0
        self.is_last_stage = pipeline_stage_id == num_pipeline_stages - 1
        if num_pipeline_stages > 1 and config.tie_word_embeddings:
            raise NotImplementedError("tied embeddings are not supported with pipeline parallel")
        H = config.hidden_size
        self.embed_dim, self.m_emb = H, config.m_emb
        per_stage = divide_if_divisible(config.num_layers, num_pipeline_stages,
                                        "layers should be divisible by num_pipeline_stages")
        self.layer_start_id = per_stage * pipeline_stage_id
        self.layer_end_id = per_stage * (pipeline_stage_id + 1)
        kw = dict(use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel)
        if self.is_first_stage:
            self.wte = ParameterizedEmbedding(
                config.vocab_size, H,
                std=std_for_embedding(config.initializer_range, config.embedding_init_method, H), **kw)
            self.embedding_dropout = Dropout(config.embedding_dropout)
        self.h = nn.ModuleDict({
            str(i): self.layer_class(config, use_padding_free_transformer=use_padding_free_transformer,
                                     layer_idx=i, sequence_parallel=sequence_parallel)
            for i in range(self.layer_start_id, self.layer_end_id)})
        if self.is_last_stage:
            self.ln_f = get_normalization_function(config.normalization_function, H, eps=config.layer_norm_epsilon,
                                                   sequence_parallel=sequence_parallel)
        self.position_embedding_type = config.position_embedding_type
        if self.position_embedding_type == "learned_absolute":
            if self.is_first_stage:
                self.wpe = ParameterizedEmbedding(config.max_position_embeddings, H, std=config.initializer_range,
                                                  **kw)
        elif self.position_embedding_type == "rope":
            if config.rope_scaling is None:
                self.rope = RoPE(config.rope_dim, config.max_position_embeddings, base=config.rope_theta)
            else:
                self.rope = YaRNScaledRoPE(
                    config.rope_dim, config.max_position_embeddings, base=config.rope_theta,
                    scale=config.rope_scaling["factor"],
                    original_max_position_embeddings=config.rope_scaling["original_max_position_embeddings"])
        elif self.position_embedding_type != "nope":
            raise NotImplementedError(self.position_embedding_type)

    # ------------------------------------------------------------------ helpers
    def _sequence_multiplier(self) -> int:
        m = ProcessGroupManager.get_context_parallel_world_size()
        if self.sequence_parallel:
            m *= ProcessGroupManager.get_tensor_parallel_world_size()
        return m

    def _setup_positions(self, position_info: PositionInfo, attention_mask, past_length, query_length, key_length,
                         device) -> None:
        position_info.fill(attention_mask, past_length, query_length, key_length, device)
        if self.position_embedding_type == "rope":
            cos, sin = self.rope.tables(key_length)
            position_info.rope_tables = (cos, sin)
            pid = position_info.position_ids
            position_info.rope_cos_sin = (cos[pid], sin[pid])

    def embed(self, input_ids, cache_params, attention_mask_info: AttentionMaskInfo, position_info: PositionInfo):
        if self.use_padding_free_transformer:
            assert position_info.position_ids is not None, "packed inputs need position_ids"
            ms = attention_mask_info.max_seqlen
            key_length = int(ms.item()) if isinstance(ms, torch.Tensor) else ms
            past_length, query_length = 0, key_length
        else:
            past_length = 0 if cache_params is None else cache_params.get_seq_length()
            query_length = input_ids.size(-1) * ProcessGroupManager.get_context_parallel_world_size()
            key_length = past_length + query_length
        x = self.wte(input_ids)
        if self.position_embedding_type in ("rope", "learned_absolute"):
            self._setup_positions(position_info, attention_mask_info.attention_mask, past_length, query_length,
                                  key_length, input_ids.device)
        if self.position_embedding_type == "learned_absolute":
            pos = self.wpe(position_info.position_ids)
            if self.sequence_parallel and ProcessGroupManager.is_tensor_parallel_enabled():
                pass  # wpe output is already reduce-scattered like wte's
            x = x + pos
        x = self.embedding_dropout(x)
        if self.m_emb is not None:
            x = x * self.m_emb
        return x

    def run_blocks(self, x, cache_params, attention_mask_info, position_info):
        for i in range(self.layer_start_id, self.layer_end_id):
            x = self.h[str(i)](x, cache_params=cache_params, attention_mask_info=attention_mask_info,
                               position_info=position_info)
        return x

    def forward(self, input_ids: torch.Tensor | None = None, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None,
                position_info: PositionInfo | None = None) -> BaseModelOutputWithPast:
        attention_mask_info, position_info = resolve_attention_and_position_info(attention_mask_info, position_info)
        if self.is_first_stage:
            x = self.embed(input_ids, cache_params, attention_mask_info, position_info)
        else:
            # later pipeline stages receive hidden states in place of token ids
            x = input_ids
            assert cache_params is None and attention_mask_info.attention_mask is None
            if self.use_padding_free_transformer:
                key_length = attention_mask_info.max_seqlen
            else:
                key_length = x.size(1) * self._sequence_multiplier()
            if self.position_embedding_type in ("rope", "learned_absolute"):
                self._setup_positions(position_info, None, 0, key_length, key_length, x.device)
        # a K/V cache is only ever useful for inference; under training it would also break activation
        # recomputation (the recomputed block would append its keys to the ones cached by the first forward)
        training_pass = self.training and torch.is_grad_enabled()
        if (not self.use_padding_free_transformer and is_generation_cache_enabled() and cache_params is None
                and not training_pass):
            cache_params = GenerationCache()
        x = self.run_blocks(x, cache_params, attention_mask_info, position_info)
        if self.is_last_stage:
            x = self.ln_f(x)
        return BaseModelOutputWithPast(last_hidden_state=x, cache_params=cache_params)


class PaLMModel(TransformerModel):
    layer_class = PaLMBlock


class LadderResidualModel(TransformerModel):
    layer_class = LadderBlock

    def run_blocks(self, x, cache_params, attention_mask_info, position_info):
        state = (x, None, None)
        for i in range(self.layer_start_id, self.layer_end_id):
            state = self.h[str(i)](state, cache_params=cache_params, attention_mask_info=attention_mask_info,
                                   position_info=position_info)
        residual, a, m = state
        return residual + a + m


class CausalLM(nn.Module):
    """``transformer`` + untied ``lm_head`` (or the tied embedding matrix) with muP logit scaling."""

    base_model_class = TransformerModel
    model_type = "gpt_base"

    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool = False,
                 sequence_parallel: bool = False, num_pipeline_stages: int = 1, pipeline_stage_id: int = 0,
                 **_unused) -> None:
        super().__init__()
        self.config = config
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.num_pipeline_stages, self.pipeline_stage_id = num_pipeline_stages, pipeline_stage_id
        self.is_first_stage = pipeline_stage_id == 0
        self.is_last_stage = pipeline_stage_id == num_pipeline_stages - 1
        self.is_pipeline_parallel_enabled = num_pipeline_stages > 1
        self._tied_word_embeddings = config.tie_word_embeddings
        self.router_aux_loss_coef = config.router_aux_loss_coef or 0
        self.vocab_size = config.vocab_size
        self.bos_token_id, self.eos_token_id, self.pad_token_id = (config.bos_token_id, config.eos_token_id,
                                                                  config.pad_token_id)
        self.transformer = self.base_model_class(
            config, use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel,
            num_pipeline_stages=num_pipeline_stages, pipeline_stage_id=pipeline_stage_id)
        if self.is_last_stage:
            if not self._tied_word_embeddings:
                self.lm_head = LMHead(config.vocab_size, config.hidden_size, std=config.initializer_range,
                                      use_padding_free_transformer=use_padding_free_transformer,
                                      sequence_parallel=sequence_parallel)
            self.m_width = config.m_width

    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.transformer.wte if self._tied_word_embeddings else self.lm_head

    def compute_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self._tied_word_embeddings:
            wte = self.transformer.wte
            logits = LMHead.compute_with_weight(wte, hidden_states, wte.weight)
        else:
            logits = self.lm_head(hidden_states)
        if self.m_width is not None:
            logits = logits * (1 / self.m_width)
        return logits

    def compute_lm_loss(self, hidden_states: torch.Tensor, labels: torch.Tensor, **loss_kwargs) -> torch.Tensor:
        """Summed cross entropy straight from the final hidden states (LM head evaluated in token chunks)."""
        if self._tied_word_embeddings:
            wte = self.transformer.wte
            return LMHead.loss_with_weight(wte, hidden_states, wte.weight, labels, **loss_kwargs)
        return self.lm_head(hidden_states, labels=labels, loss_kwargs=loss_kwargs)

    def forward(self, input_ids: torch.Tensor | None = None, cache_params: GenerationCache | None = None,
                attention_mask_info: AttentionMaskInfo | None = None, position_info: PositionInfo | None = None,
                output_parallel_lm_logits: bool = False, pipeline_parallel_input: PipelineParallelInput | None = None,
                skip_logits: bool = False):
        attention_mask_info, position_info = resolve_attention_and_position_info(attention_mask_info, position_info)
        clear_aux_loss()
        if self.is_first_stage:
            assert pipeline_parallel_input is None, "first stage should not get pipeline_parallel_input"
            if self.use_padding_free_transformer:
                assert attention_mask_info.cu_seqlens is not None and attention_mask_info.max_seqlen is not None
                assert attention_mask_info.attention_mask is None and cache_params is None
        else:
            assert input_ids is None
            add_aux_loss(pipeline_parallel_input.aux_loss)
        out = self.transformer(
            input_ids=input_ids if pipeline_parallel_input is None else pipeline_parallel_input.hidden_states,
            cache_params=cache_params, attention_mask_info=attention_mask_info, position_info=position_info)
        hidden, aux = out.last_hidden_state, get_aux_loss()
        if not self.is_last_stage:
            return PipelineParallelOutput(hidden_states=hidden, aux_loss=aux)
        logits = None
        if skip_logits:
            if self.m_width is not None:
                hidden = hidden * (1 / self.m_width)
        else:
            logits = self.compute_logits(hidden)
            if ProcessGroupManager.is_tensor_parallel_enabled() and not output_parallel_lm_logits:
                logits = tp_comm.gather_last_dim_from_tensor_parallel(logits)[..., : self.vocab_size]
        return CausalLMOutputWithPast(aux_loss=aux, logits=logits, cache_params=out.cache_params,
                                      last_hidden_state=hidden)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_from_safetensors_weights_manager(self, manager: SafeTensorsWeightsManager) -> None:
        """Loads (the tensor-parallel shard of) every parameter present in the checkpoint."""
        tp_rank = ProcessGroupManager.get_tensor_parallel_rank()
        for name, p in list(self.named_parameters()) + list(self.named_buffers()):
            if not manager.has_tensor(name):
                continue
            dim = getattr(p, "tp_shard_dim", None)
            ep_dim = getattr(p, "ep_shard_dim", None)
            if ep_dim is not None and ProcessGroupManager.get_expert_parallel_world_size() > 1:
                # experts are split over the expert-parallel ranks (never combined with a tensor-parallel split)
                sl = manager.get_slice(name)
                n = p.size(ep_dim)
                lo = ProcessGroupManager.get_expert_parallel_rank() * n
                idx = [slice(None)] * len(sl.get_shape())
                idx[ep_dim] = slice(lo, lo + n)
                t = sl[tuple(idx)]
            elif dim is None or ProcessGroupManager.get_tensor_parallel_world_size() == 1:
                t = manager.get_tensor(name)
            else:
                sl = manager.get_slice(name)
                n = p.size(dim)
                full = sl.get_shape()[dim]
                lo, hi = tp_rank * n, min((tp_rank + 1) * n, full)
                idx = [slice(None)] * len(sl.get_shape())
                idx[dim] = slice(lo, hi)
                t = sl[tuple(idx)]
                if hi - lo < n:  # vocabulary padding
                    pad_shape = list(t.shape)
                    pad_shape[dim] = n - (hi - lo)
                    t = torch.cat((t, torch.zeros(pad_shape, dtype=t.dtype)), dim=dim)
            p.copy_(t.to(device=p.device, dtype=p.dtype))

    def get_dummy_intermediate_tensor(self, micro_batch_size: int, sequence_length: int, dtype: torch.dtype,
                                      device) -> torch.Tensor:
        s = sequence_length // ProcessGroupManager.get_context_parallel_world_size()
        if self.sequence_parallel:
            s = divide_if_divisible(s, ProcessGroupManager.get_tensor_parallel_world_size())
        H = self.config.hidden_size
        shape = (micro_batch_size * s, H) if self.use_padding_free_transformer else (micro_batch_size, s, H)
        return torch.empty(shape, dtype=dtype, device=device)


class PaLMForCausalLM(CausalLM):
    base_model_class = PaLMModel
    model_type = "palm"


class LadderResidualForCausalLM(CausalLM):
    base_model_class = LadderResidualModel
    model_type = "ladder_residual"
