"""MoE model (router, experts, aux loss) against the unmodified reference on CPU fp32."""

import torch

from lm_engine_b200.models import build_model, config_from_dict

from .refutil import build_reference_model


def _moe_cfg(normalized_topk=True, shared=None):
    L = 3
    return dict(
        model_type="gpt_base", vocab_size=512, max_position_embeddings=128, hidden_size=64, num_layers=L,
        normalization_function="rmsnorm", layer_norm_epsilon=1e-5, initializer_range=0.02, bos_token_id=0,
        eos_token_id=1, pad_token_id=2, position_embedding_type="rope", rope_theta=10000, rope_scaling=None,
        m_emb=None, m_width=None, m_residual=None, init_method="normal", embedding_init_method="normal",
        use_depth_scaled_init=False, tie_word_embeddings=False, router_aux_loss_coef=0.01,
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=4,
                                    num_key_value_heads=2) for _ in range(L)],
        mlp_blocks=[dict(mlp_type="MoE", intermediate_size=48, activation_function="swiglu", num_experts=8,
                         num_experts_per_tok=2, shared_intermediate_size=shared, normalized_topk=normalized_topk,
                         shared_expert_gating=shared is not None) for _ in range(L)])


def _check(cfg):
    ref = build_reference_model(cfg)
    ours = build_model(config_from_dict(cfg))
    ours.load_state_dict(ref.state_dict(), strict=True)
    ref.train(); ours.train()
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 512, (2, 33), generator=g)
    o, r = ours(x), ref(input_ids=x)
    assert torch.allclose(o.logits, r.logits, atol=2e-5, rtol=1e-5)
    assert torch.allclose(o.aux_loss, r.aux_loss, atol=1e-5)
    (o.logits.float().pow(2).mean() + 0.01 * o.aux_loss).backward()
    (r.logits.float().pow(2).mean() + 0.01 * r.aux_loss).backward()
    for (n, po), (_, pr) in zip(ours.named_parameters(), ref.named_parameters()):
        assert torch.allclose(po.grad, pr.grad, atol=2e-5, rtol=1e-4), n


def test_moe_topk_then_softmax():
    _check(_moe_cfg(True))


def test_moe_softmax_then_topk_with_shared_expert():
    _check(_moe_cfg(False, shared=32))


def test_expert_exchange_capacity_defaults_to_the_worst_case(monkeypatch):
    """Rows an owner can receive: every assignment of every rank by default (nothing can overflow); the switch lowers it
    but never below the rank's own assignments, and the result is whole 128-row tiles plus one tile per local expert."""
    from lm_engine_b200.parallel import expert_exchange as xx

    monkeypatch.delenv("LME_EP_CAPACITY_FACTOR", raising=False)
    assert xx.capacity_rows(1000, 4, 8) == 8 * 1000 // 128 * 128 + 128 + 4 * 128
    monkeypatch.setenv("LME_EP_CAPACITY_FACTOR", "2")
    assert xx.capacity_rows(1000, 4, 8) == 2048 + 4 * 128
    monkeypatch.setenv("LME_EP_CAPACITY_FACTOR", "0.1")
    assert xx.capacity_rows(1024, 2, 4) == 1024 + 2 * 128
    monkeypatch.setenv("LME_EP_CAPACITY_FACTOR", "100")
    assert xx.capacity_rows(1024, 2, 4) == 4096 + 2 * 128
