"""HF-style adapter: generation with the cache equals full recomputation, left padding does not change a row's
continuation, save / load round-trips, sampling filters."""

import pytest
import torch

VOCAB = 96


def _adapter(kind="dense", seed=0):
    from lm_engine_b200.hf_adapter import LLMAdapter_HF
    from lm_engine_b200.models import config_from_dict, dense_config

    torch.manual_seed(seed)
    if kind == "dense":
        cfg = dense_config(vocab_size=VOCAB, hidden_size=32, num_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=64, max_position_embeddings=64)
    else:
        d = dense_config(vocab_size=VOCAB, hidden_size=32, num_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, max_position_embeddings=64).to_dict()
        d["mlp_blocks"] = [{"mlp_type": "MoE", "intermediate_size": 32, "num_experts": 4, "num_experts_per_tok": 2,
                            "activation_function": "swiglu", "shared_intermediate_size": None} for _ in range(2)]
        cfg = config_from_dict(d)
    return LLMAdapter_HF._from_config(cfg).eval()


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_cached_generation_equals_recompute(kind):
    m = _adapter(kind)
    ids = torch.randint(3, VOCAB, (2, 7))
    a = m.generate_simple(ids, max_new_tokens=6, use_cache=True, eos_token_id=-1)
    b = m.generate_simple(ids, max_new_tokens=6, use_cache=False, eos_token_id=-1)
    assert a.shape == (2, 13) and torch.equal(a, b)


def test_left_padding_does_not_change_the_continuation():
    m = _adapter()
    short, long = torch.randint(3, VOCAB, (1, 4)), torch.randint(3, VOCAB, (1, 9))
    alone = m.generate_simple(short, max_new_tokens=5, eos_token_id=-1)[0, 4:]
    batch = torch.cat((torch.cat((torch.full((1, 5), 2), short), 1), long))
    mask = torch.ones_like(batch)
    mask[0, :5] = 0
    both = m.generate_simple(batch, attention_mask=mask, max_new_tokens=5, eos_token_id=-1)
    assert torch.equal(both[0, 9:], alone)


def test_eos_stops_rows_and_pads():
    m = _adapter()
    ids = torch.randint(3, VOCAB, (2, 5))
    first = m.generate_simple(ids, max_new_tokens=1, eos_token_id=-1)[:, -1]
    out = m.generate_simple(ids, max_new_tokens=4, eos_token_id=int(first[0]), pad_token_id=0)
    assert out[0, 5] == first[0] and (out[0, 6:] == 0).all()


def test_save_and_load_roundtrip(tmp_path):
    from lm_engine_b200.hf_adapter import LLMAdapter_HF

    m = _adapter()
    m.save_pretrained(str(tmp_path))
    m2 = LLMAdapter_HF.from_pretrained(str(tmp_path))
    ids = torch.randint(3, VOCAB, (1, 6))
    torch.testing.assert_close(m(ids).logits, m2(ids).logits)
    out = m2(ids, labels=ids)
    assert out.loss.dim() == 0 and torch.isfinite(out.loss)


def test_sampling_filters():
    from lm_engine_b200.hf_adapter import _sample

    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0, 10.0]]).repeat(64, 1)
    g = torch.Generator().manual_seed(0)
    assert (_sample(logits, 1.0, 1, None, g) == 4).all()
    assert (_sample(logits, 1.0, None, 0.5, g) == 4).all()
    flat = torch.zeros(256, 5)
    s = _sample(flat, 1.0, 2, None, g)
    assert s.max() <= 4 and len(s.unique()) <= 5


def test_hugging_face_generate_matches_the_simple_loop():
    """The adapter is a transformers ``PreTrainedModel`` + ``GenerationMixin``: its inherited ``generate`` (greedy, with
    the package's own cache, left-padded batch) produces the tokens of the dependency-free loop, and beam search
    runs through the same forward."""
    transformers = pytest.importorskip("transformers")
    m = _adapter()
    assert isinstance(m, transformers.PreTrainedModel) and isinstance(m, transformers.GenerationMixin)
    torch.manual_seed(1)
    ids = torch.randint(3, VOCAB, (2, 7))
    mask = torch.ones_like(ids)
    mask[1, :3] = 0                                    # second row is left-padded
    want = m.generate_simple(ids, attention_mask=mask, max_new_tokens=6, eos_token_id=-1)
    got = m.generate(input_ids=ids, attention_mask=mask, max_new_tokens=6, do_sample=False, eos_token_id=None,
                     pad_token_id=0)
    assert torch.equal(got, want)
    no_cache = m.generate(input_ids=ids, attention_mask=mask, max_new_tokens=6, do_sample=False, eos_token_id=None,
                          pad_token_id=0, use_cache=False)
    assert torch.equal(no_cache, want)
    beams = m.generate(input_ids=ids[:1], max_new_tokens=4, num_beams=3, do_sample=False, eos_token_id=None,
                       pad_token_id=0)
    assert beams.shape == (1, 11)
