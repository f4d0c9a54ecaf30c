"""Checkpoint interchange with Hugging Face layouts: ``llama``, ``granite`` and ``granitemoehybrid``, both directions
(role of tools/model_conversion/{__init__,llama,granite,granitemoehybrid}.py and tools/{import_from,export_to}_hf.py).

The conversion is table driven.  For a given config, :func:`tensor_rules` lists, per native parameter, the Hugging
Face tensors it is built from and the pair of packing functions between them:

* fused ``c_attn``  <->  ``q_proj`` / ``k_proj`` / ``v_proj``  (per KV group: its query heads, then key, then value)
* packed ``c_fc``   <->  ``up_proj`` / ``gate_proj`` (rows interleaved gate, up, gate, up, ...), and the same for the
  MoE ``input_linear`` ``[E, 2I, H]`` and the shared expert, which Hugging Face stores as the two halves stacked
* Mamba-2 parameters are renamed only.

Configs travel as plain ``config.json`` dictionaries, so neither direction needs the ``transformers`` classes.

Command line::

    python -m lm_engine_b200.model_conversion import --path <hf dir> --save <dir>
    python -m lm_engine_b200.model_conversion export --path <native dir> --model-type llama --save <dir>
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
from dataclasses import dataclass
from typing import Callable

import torch

from ..models import CommonConfig, config_from_dict
from ..models.layers.attention import (
    interleave_query_key_value_tensor_for_attention as _pack_qkv,
    split_query_key_value_tensor_for_attention as _split_qkv,
)
from ..models.layers.mlp import interleave_up_gate, split_up_gate
from ..utils import SafeTensorsWeightsManager, divide_if_divisible

_ARCHITECTURES = {"llama": "LlamaForCausalLM", "granite": "GraniteForCausalLM",
                  "granitemoehybrid": "GraniteMoeHybridForCausalLM"}
_TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "tokenizer.model",
                    "vocab.json", "merges.txt", "added_tokens.json")


@dataclass
class Rule:
    native: str
    hf: tuple[str, ...]
    to_native: Callable[..., torch.Tensor]           # (*hf tensors) -> native tensor
    to_hf: Callable[[torch.Tensor], tuple]           # native tensor -> hf tensors
    optional: bool = False                           # skipped when absent from the source checkpoint


def _same(native: str, hf: str, optional: bool = False) -> Rule:
    return Rule(native, (hf,), lambda t: t, lambda t: (t,), optional)


def _all_equal(config: CommonConfig, blocks: str, key: str, only_type: str | None = None, default=None):
    vals = []
    for b in getattr(config, blocks):
        if only_type is not None and getattr(b, "sequence_mixer_type", getattr(b, "mlp_type", None)) != only_type:
            continue
        vals.append(getattr(b, key))
    if not vals:
        return default
    assert all(v == vals[0] for v in vals), f"{blocks}.{key} differs between layers: {vals}"
    return vals[0]


def _mixer_type(b) -> str:
    return b.sequence_mixer_type


# ---------------------------------------------------------------------------------------------------- tensors
def tensor_rules(config: CommonConfig, model_type: str) -> list[Rule]:
    rules = [_same("transformer.wte.weight", "model.embed_tokens.weight"),
             _same("transformer.ln_f.weight", "model.norm.weight"),
             _same("lm_head.weight", "lm_head.weight", optional=True)]
    for i in range(config.num_layers):
        n, h = f"transformer.h.{i}.", f"model.layers.{i}."
        rules += [_same(n + "ln_1.weight", h + "input_layernorm.weight"),
                  _same(n + "ln_2.weight", h + "post_attention_layernorm.weight")]
        mixer, mlp = config.sequence_mixer_blocks[i], config.mlp_blocks[i]
        if _mixer_type(mixer) == "softmax_attention":
            Hq, Hkv = mixer.num_attention_heads, mixer.num_key_value_heads
            D = mixer.head_dim or divide_if_divisible(config.hidden_size, Hq, "")
            for suffix, opt in (("weight", False), ("bias", True)):
                rules.append(Rule(n + f"sequence_mixer.c_attn.{suffix}",
                                  tuple(h + f"self_attn.{p}_proj.{suffix}" for p in "qkv"),
                                  lambda q, k, v, Hq=Hq, Hkv=Hkv, D=D: _pack_qkv(q, k, v, Hq, Hkv, D),
                                  lambda t, Hq=Hq, Hkv=Hkv, D=D: _split_qkv(t, Hq, Hkv, D), opt))
                rules.append(_same(n + f"sequence_mixer.c_proj.{suffix}", h + f"self_attn.o_proj.{suffix}", opt))
        elif _mixer_type(mixer) == "mamba2":
            assert model_type == "granitemoehybrid", "only granitemoehybrid has Mamba-2 layers"
            for a, b, opt in (("conv1d.weight", "conv1d.weight", False), ("conv1d.bias", "conv1d.bias", True),
                              ("in_proj.weight", "in_proj.weight", False), ("in_proj.bias", "in_proj.bias", True),
                              ("decay_gate.dt_bias", "dt_bias", False), ("decay_gate.A_log", "A_log", False),
                              ("D", "D", False), ("out_proj.weight", "out_proj.weight", False),
                              ("out_proj.bias", "out_proj.bias", True), ("norm.weight", "norm.weight", False)):
                rules.append(_same(n + "sequence_mixer." + a, h + "mamba." + b, opt))
        else:
            raise NotImplementedError(f"{_mixer_type(mixer)} layers have no Hugging Face counterpart")

        def halves_to_packed(t, dim=0):          # HF: [gate ; up] stacked  ->  rows interleaved gate, up, ...
            g, u = t.chunk(2, dim=dim)
            if dim == 0:
                return interleave_up_gate(u, g)
            return torch.stack([interleave_up_gate(u[e], g[e]) for e in range(t.size(0))])

        def packed_to_halves(t, dim=0):
            if dim == 0:
                u, g = split_up_gate(t)
                return (torch.cat((g, u), dim=0),)
            parts = [split_up_gate(t[e]) for e in range(t.size(0))]
            return (torch.stack([torch.cat((g, u), dim=0) for u, g in parts]),)

        if model_type == "granitemoehybrid":
            if mlp.mlp_type == "MoE":
                rules += [_same(n + "mlp_block.gate.weight", h + "block_sparse_moe.router.layer.weight"),
                          Rule(n + "mlp_block.c_fc.weight", (h + "block_sparse_moe.input_linear.weight",),
                               lambda t: halves_to_packed(t, 1), lambda t: packed_to_halves(t, 1)),
                          _same(n + "mlp_block.c_proj.weight", h + "block_sparse_moe.output_linear.weight")]
                if mlp.shared_intermediate_size is not None:
                    rules += [Rule(n + "mlp_block.c_fc_shared.weight", (h + "shared_mlp.input_linear.weight",),
                                   halves_to_packed, packed_to_halves),
                              _same(n + "mlp_block.c_proj_shared.weight", h + "shared_mlp.output_linear.weight")]
            else:
                rules += [Rule(n + "mlp_block.c_fc.weight", (h + "shared_mlp.input_linear.weight",),
                               halves_to_packed, packed_to_halves),
                          _same(n + "mlp_block.c_proj.weight", h + "shared_mlp.output_linear.weight")]
        else:
            assert mlp.mlp_type == "MLP", f"{model_type} has dense MLPs only"
            for suffix, opt in (("weight", False), ("bias", True)):
                rules.append(Rule(n + f"mlp_block.c_fc.{suffix}",
                                  (h + f"mlp.up_proj.{suffix}", h + f"mlp.gate_proj.{suffix}"),
                                  lambda u, g: interleave_up_gate(u, g), lambda t: split_up_gate(t), opt))
                rules.append(_same(n + f"mlp_block.c_proj.{suffix}", h + f"mlp.down_proj.{suffix}", opt))
    return rules


def import_state_dict(config: CommonConfig, model_type: str, weights: SafeTensorsWeightsManager) -> dict:
    out = {}
    for r in tensor_rules(config, model_type):
        if not all(weights.has_tensor(k) for k in r.hf):
            assert r.optional, f"checkpoint lacks {r.hf}"
            continue
        out[r.native] = r.to_native(*[weights.get_tensor(k) for k in r.hf]).contiguous()
    return out


def export_state_dict(config: CommonConfig, model_type: str, weights: SafeTensorsWeightsManager) -> dict:
    out = {}
    for r in tensor_rules(config, model_type):
        if not weights.has_tensor(r.native):
            assert r.optional, f"checkpoint lacks {r.native}"
            continue
        for k, t in zip(r.hf, r.to_hf(weights.get_tensor(r.native))):
            out[k] = t.contiguous()
    return out


# ---------------------------------------------------------------------------------------------------- configs
def _attention_block(hf: dict, multiplier) -> dict:
    return {"sequence_mixer_type": "softmax_attention", "add_bias": hf.get("attention_bias", False),
            "num_attention_heads": hf["num_attention_heads"],
            "num_key_value_heads": hf.get("num_key_value_heads", hf["num_attention_heads"]),
            "head_dim": None, "softmax_dropout": hf.get("attention_dropout", 0), "dropout": 0,
            "attention_multiplier": multiplier,
            "attention_multiplier_method": "1 / sqrt(head_dim)" if multiplier is None else None,
            "sliding_window": None}


def _one_or_none(v):
    return None if v in (None, 1, 1.0) else v


def import_config(hf: dict) -> CommonConfig:
    mt = hf["model_type"]
    assert mt in _ARCHITECTURES, f"model_type {mt} is not supported"
    assert hf.get("hidden_act", "silu") == "silu"
    L = hf["num_hidden_layers"]
    common = dict(vocab_size=hf["vocab_size"], max_position_embeddings=hf["max_position_embeddings"],
                  hidden_size=hf["hidden_size"], num_layers=L, normalization_function="rmsnorm",
                  layer_norm_epsilon=hf["rms_norm_eps"], embedding_dropout=0,
                  tie_word_embeddings=hf.get("tie_word_embeddings", False),
                  initializer_range=hf.get("initializer_range", 0.02), rope_theta=_rope_theta(hf),
                  rope_scaling=hf.get("rope_scaling"), init_method="normal", embedding_init_method="normal",
                  use_depth_scaled_init=True, rope_dim=None, bos_token_id=hf.get("bos_token_id"),
                  eos_token_id=hf.get("eos_token_id"), pad_token_id=hf.get("pad_token_id"))
    if mt == "llama":
        assert hf.get("mlp_bias", False) == hf.get("attention_bias", False)
        mixers = [_attention_block(hf, None) for _ in range(L)]
        mlps = [{"mlp_type": "MLP", "add_bias": hf.get("mlp_bias", False), "activation_function": "swiglu",
                 "intermediate_size": hf["intermediate_size"], "dropout": 0} for _ in range(L)]
        extra = dict(position_embedding_type="rope", router_aux_loss_coef=0.001, m_emb=None, m_width=None,
                     m_residual=None)
    else:
        extra = dict(m_emb=_one_or_none(hf.get("embedding_multiplier", 1)),
                     m_residual=_one_or_none(hf.get("residual_multiplier", 1)),
                     m_width=_one_or_none(hf.get("logits_scaling", 1)))
        mult = hf.get("attention_multiplier")
        if mt == "granite":
            assert hf.get("mlp_bias", False) == hf.get("attention_bias", False)
            mixers = [_attention_block(hf, mult) for _ in range(L)]
            mlps = [{"mlp_type": "MLP", "add_bias": hf.get("mlp_bias", False), "activation_function": "swiglu",
                     "intermediate_size": hf["intermediate_size"], "dropout": 0} for _ in range(L)]
            extra.update(position_embedding_type="rope", router_aux_loss_coef=0.001)
        else:
            assert not hf.get("attention_bias", False)
            mixers = []
            for kind in hf["layer_types"]:
                if kind == "attention":
                    mixers.append(_attention_block(hf, mult))
                elif kind == "mamba":
                    mixers.append({"sequence_mixer_type": "mamba2", "state_size": hf["mamba_d_state"],
                                   "intermediate_size": hf["mamba_expand"] * hf["hidden_size"],
                                   "num_heads": hf["mamba_n_heads"], "conv_kernel_size": hf["mamba_d_conv"],
                                   "add_bias": hf.get("mamba_proj_bias", False),
                                   "use_conv_bias": hf.get("mamba_conv_bias", True),
                                   "num_groups": hf["mamba_n_groups"], "chunk_size": hf["mamba_chunk_size"],
                                   "activation_function": "silu", "normalization_function": "rmsnorm"})
                else:
                    raise ValueError(f"unexpected layer type {kind}")
            if hf.get("num_local_experts", 0) == 0:
                mlps = [{"mlp_type": "MLP", "intermediate_size": hf["shared_intermediate_size"],
                         "activation_function": "swiglu", "add_bias": False, "dropout": 0} for _ in range(L)]
            else:
                shared = hf.get("shared_intermediate_size", 0)
                mlps = [{"mlp_type": "MoE", "intermediate_size": hf["intermediate_size"],
                         "shared_intermediate_size": None if shared == 0 else shared,
                         "num_experts": hf["num_local_experts"], "num_experts_per_tok": hf["num_experts_per_tok"],
                         "activation_function": "swiglu", "add_bias": False, "dropout": 0,
                         "shared_expert_gating": False, "normalized_topk": True} for _ in range(L)]
            extra.update(position_embedding_type=hf.get("position_embedding_type", "nope"),
                         router_aux_loss_coef=hf.get("router_aux_loss_coef", 0.001))
    return config_from_dict(dict(model_type="gpt_base", sequence_mixer_blocks=mixers, mlp_blocks=mlps,
                                 **common, **extra))


def _rope_theta(hf: dict):
    if "rope_theta" in hf:
        return hf["rope_theta"]
    rp = hf.get("rope_parameters") or {}
    return rp.get("rope_theta", 10000)


def export_config(config: CommonConfig, model_type: str) -> dict:
    assert model_type in _ARCHITECTURES
    assert config.normalization_function == "rmsnorm"
    _all_equal(config, "mlp_blocks", "activation_function")
    att = "softmax_attention"
    out = dict(model_type=model_type, architectures=[_ARCHITECTURES[model_type]], vocab_size=config.vocab_size,
               max_position_embeddings=config.max_position_embeddings, hidden_size=config.hidden_size,
               num_hidden_layers=config.num_layers,
               num_attention_heads=_all_equal(config, "sequence_mixer_blocks", "num_attention_heads", att),
               num_key_value_heads=_all_equal(config, "sequence_mixer_blocks", "num_key_value_heads", att),
               hidden_act="silu", rms_norm_eps=config.layer_norm_epsilon, use_cache=True,
               attention_bias=_all_equal(config, "sequence_mixer_blocks", "add_bias", att, False),
               tie_word_embeddings=config.tie_word_embeddings, initializer_range=config.initializer_range,
               rope_theta=config.rope_theta, rope_scaling=config.rope_scaling,
               attention_dropout=_all_equal(config, "sequence_mixer_blocks", "softmax_dropout", att, 0),
               bos_token_id=config.bos_token_id, eos_token_id=config.eos_token_id, pad_token_id=config.pad_token_id)
    mult = _all_equal(config, "sequence_mixer_blocks", "attention_multiplier", att)
    if model_type == "llama":
        assert config.position_embedding_type == "rope"
        assert config.m_emb is None and config.m_residual is None and config.m_width is None and mult is None
    else:
        out.update(embedding_multiplier=1 if config.m_emb is None else config.m_emb,
                   residual_multiplier=1 if config.m_residual is None else config.m_residual,
                   logits_scaling=1 if config.m_width is None else config.m_width, attention_multiplier=mult)
    if model_type in ("llama", "granite"):
        assert config.position_embedding_type == "rope"
        assert _all_equal(config, "mlp_blocks", "mlp_type") == "MLP"
        out.update(intermediate_size=_all_equal(config, "mlp_blocks", "intermediate_size"),
                   mlp_bias=_all_equal(config, "mlp_blocks", "add_bias"))
        return out
    assert config.position_embedding_type == "nope"
    assert _all_equal(config, "mlp_blocks", "add_bias") is False
    if all(b.mlp_type == "MLP" for b in config.mlp_blocks):
        experts = topk = 0
        shared = _all_equal(config, "mlp_blocks", "intermediate_size")
        inter = shared
    else:
        experts = _all_equal(config, "mlp_blocks", "num_experts")
        topk = _all_equal(config, "mlp_blocks", "num_experts_per_tok")
        shared = _all_equal(config, "mlp_blocks", "shared_intermediate_size")
        inter = _all_equal(config, "mlp_blocks", "intermediate_size")
    m2 = "mamba2"
    mamba_inter = _all_equal(config, "sequence_mixer_blocks", "intermediate_size", m2)
    out.update(intermediate_size=inter, shared_intermediate_size=0 if shared is None else shared,
               num_local_experts=experts, num_experts_per_tok=topk, router_aux_loss_coef=config.router_aux_loss_coef,
               layer_types=["mamba" if b.sequence_mixer_type == m2 else "attention"
                            for b in config.sequence_mixer_blocks],
               position_embedding_type="nope", normalization_function=config.normalization_function,
               init_method=config.init_method)
    if mamba_inter is not None:
        out.update(mamba_expand=divide_if_divisible(mamba_inter, config.hidden_size, ""),
                   mamba_n_groups=_all_equal(config, "sequence_mixer_blocks", "num_groups", m2),
                   mamba_n_heads=_all_equal(config, "sequence_mixer_blocks", "num_heads", m2),
                   mamba_d_state=_all_equal(config, "sequence_mixer_blocks", "state_size", m2),
                   mamba_d_conv=_all_equal(config, "sequence_mixer_blocks", "conv_kernel_size", m2),
                   mamba_chunk_size=_all_equal(config, "sequence_mixer_blocks", "chunk_size", m2),
                   mamba_conv_bias=_all_equal(config, "sequence_mixer_blocks", "use_conv_bias", m2),
                   mamba_proj_bias=_all_equal(config, "sequence_mixer_blocks", "add_bias", m2))
    return out


# ---------------------------------------------------------------------------------------------------- entry points
def _copy_tokenizer(src: str, dst: str) -> None:
    for f in _TOKENIZER_FILES:
        if os.path.isfile(os.path.join(src, f)):
            shutil.copy(os.path.join(src, f), os.path.join(dst, f))


def _generation_config(cfg: dict) -> dict:
    return {k: cfg.get(k) for k in ("bos_token_id", "eos_token_id", "pad_token_id") if cfg.get(k) is not None}


def import_from_huggingface(pretrained_model_name_or_path: str, save_path: str | None = None):
    """Hugging Face directory -> ``(config, state_dict)`` of this package (written to ``save_path`` when given)."""
    path = pretrained_model_name_or_path
    assert os.path.isdir(path), "there is no hub access: pass a local directory"
    with open(os.path.join(path, "config.json")) as f:
        hf = json.load(f)
    config = import_config(hf)
    sd = import_state_dict(config, hf["model_type"], SafeTensorsWeightsManager(path))
    if save_path is not None:
        os.makedirs(save_path, exist_ok=True)
        config.save_pretrained(save_path)
        with open(os.path.join(save_path, "generation_config.json"), "w") as f:
            json.dump(_generation_config(config.to_dict()), f, indent=2)
        SafeTensorsWeightsManager.save_state_dict(sd, save_path)
        _copy_tokenizer(path, save_path)
    return config, sd


def export_to_huggingface(pretrained_model_name_or_path: str, model_type: str, save_path: str | None = None):
    """Directory of this package -> ``(Hugging Face config dict, state_dict)``."""
    path = pretrained_model_name_or_path
    config = CommonConfig.from_pretrained(path)
    sd = export_state_dict(config, model_type, SafeTensorsWeightsManager(path))
    hf = export_config(config, model_type)
    if save_path is not None:
        os.makedirs(save_path, exist_ok=True)
        with open(os.path.join(save_path, "config.json"), "w") as f:
            json.dump(hf, f, indent=2)
        with open(os.path.join(save_path, "generation_config.json"), "w") as f:
            json.dump(_generation_config(hf), f, indent=2)
        SafeTensorsWeightsManager.save_state_dict(sd, save_path)
        _copy_tokenizer(path, save_path)
    return hf, sd


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(prog="python -m lm_engine_b200.model_conversion")
    ap.add_argument("direction", choices=["import", "export"])
    ap.add_argument("--path", required=True)
    ap.add_argument("--save", required=True)
    ap.add_argument("--model-type", choices=sorted(_ARCHITECTURES), default=None)
    a = ap.parse_args(argv)
    if a.direction == "import":
        import_from_huggingface(a.path, a.save)
    else:
        assert a.model_type is not None, "--model-type is required for export"
        export_to_huggingface(a.path, a.model_type, a.save)
