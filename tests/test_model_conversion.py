"""Hugging Face interchange: export -> import round trip is byte exact, and the exported checkpoint loaded into the
``transformers`` implementation of the architecture produces the same logits as the native model."""

import json
import os

import pytest
import torch

from lm_engine_b200.model_conversion import export_to_huggingface, import_from_huggingface
from lm_engine_b200.models import build_model, config_from_dict, dense_config
from lm_engine_b200.utils import SafeTensorsWeightsManager

VOCAB = 128


def _native(kind: str):
    d = dense_config(vocab_size=VOCAB, hidden_size=64, num_layers=3, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=96, max_position_embeddings=128).to_dict()
    d.update(bos_token_id=0, eos_token_id=1, pad_token_id=2)
    if kind == "granite":
        d.update(m_emb=2.0, m_residual=0.5, m_width=4.0)
        for b in d["sequence_mixer_blocks"]:
            b.update(attention_multiplier=0.2, attention_multiplier_method=None)
    if kind == "granitemoehybrid":
        d.update(position_embedding_type="nope", m_emb=2.0, m_residual=0.5, m_width=4.0)
        for b in d["sequence_mixer_blocks"]:
            b.update(attention_multiplier=0.2, attention_multiplier_method=None)
        d["sequence_mixer_blocks"][0] = {
            "sequence_mixer_type": "mamba2", "state_size": 16, "intermediate_size": 128, "num_heads": 8,
            "conv_kernel_size": 4, "add_bias": False, "use_conv_bias": True, "num_groups": 1, "chunk_size": 8,
            "activation_function": "silu", "normalization_function": "rmsnorm"}
        d["mlp_blocks"] = [{"mlp_type": "MoE", "intermediate_size": 32, "num_experts": 4, "num_experts_per_tok": 2,
                            "activation_function": "swiglu", "shared_intermediate_size": 48, "add_bias": False}
                           for _ in range(3)]
    torch.manual_seed(0)
    cfg = config_from_dict(d)
    return cfg, build_model(cfg).eval()


@pytest.mark.parametrize("kind", ["llama", "granite", "granitemoehybrid"])
def test_export_import_roundtrip_is_exact(kind, tmp_path):
    cfg, model = _native(kind)
    a, b, c = (str(tmp_path / n) for n in "abc")
    cfg.save_pretrained(a)
    SafeTensorsWeightsManager.save_state_dict(model.state_dict(), a)
    export_to_huggingface(a, kind, b)
    cfg2, sd2 = import_from_huggingface(b, c)
    assert json.load(open(os.path.join(b, "config.json")))["architectures"]
    sd = model.state_dict()
    assert set(sd2) == set(sd)
    for k in sd:
        assert torch.equal(sd[k], sd2[k]), k
    d1, d2 = cfg.to_dict(), cfg2.to_dict()
    for key in ("vocab_size", "hidden_size", "num_layers", "m_emb", "m_width", "m_residual", "rope_theta",
                "position_embedding_type", "tie_word_embeddings", "layer_norm_epsilon"):
        assert d1[key] == d2[key], key
    for b1, b2 in zip(d1["sequence_mixer_blocks"] + d1["mlp_blocks"], d2["sequence_mixer_blocks"] + d2["mlp_blocks"]):
        for k in b2:
            if k in b1 and k not in ("dropout", "softmax_dropout"):
                assert b1[k] == b2[k], k


@pytest.mark.parametrize("kind", ["llama", "granite", "granitemoehybrid"])
def test_exported_checkpoint_matches_transformers_logits(kind, tmp_path):
    transformers = pytest.importorskip("transformers")
    cfg, model = _native(kind)
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    cfg.save_pretrained(a)
    SafeTensorsWeightsManager.save_state_dict(model.state_dict(), a)
    export_to_huggingface(a, kind, b)
    try:
        hf = transformers.AutoModelForCausalLM.from_pretrained(b, dtype=torch.float32).eval()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build {kind} here: {type(e).__name__}: {e}")
    ids = torch.randint(3, VOCAB, (2, 24))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = model(input_ids=ids).logits
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-4, atol=2e-4)
