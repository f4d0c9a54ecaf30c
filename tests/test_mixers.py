"""Sequence mixers on CPU: chunked SSD == token recurrence; hybrid / recurrent models against the reference."""

import pytest
import torch

from lm_engine_b200.models import build_model, config_from_dict
from lm_engine_b200.ops.ssd import ssd_chunk_scan, ssd_recurrent_step

from .refutil import build_reference_model


@pytest.mark.parametrize("S,L,G", [(37, 8, 1), (64, 16, 2), (5, 8, 1)])
def test_ssd_chunked_equals_recurrence(S, L, G):
    torch.manual_seed(0)
    b, N, P, Sd = 2, 4, 8, 6
    x = torch.randn(b, S, N, P)
    dt = torch.rand(b, S, N) * 0.5 + 0.01
    A = -torch.rand(N) * 2 - 0.1
    B, C = torch.randn(b, S, G, Sd), torch.randn(b, S, G, Sd)
    D = torch.randn(N)
    h0 = torch.randn(b, N, P, Sd)
    y, hf = ssd_chunk_scan(x, dt, A, B, C, D, L, initial_state=h0)
    h = h0.clone()
    ys = []
    for t in range(S):
        yt, h = ssd_recurrent_step(x[:, t], dt[:, t], A, B[:, t], C[:, t], D, h)
        ys.append(yt)
    assert torch.allclose(y, torch.stack(ys, 1), atol=1e-4, rtol=1e-4)
    assert torch.allclose(hf, h, atol=1e-4, rtol=1e-4)


def _base(L, mixers, **extra):
    d = dict(model_type="gpt_base", vocab_size=256, max_position_embeddings=64, hidden_size=32, num_layers=L,
             normalization_function="rmsnorm", layer_norm_epsilon=1e-5, initializer_range=0.02, bos_token_id=0,
             eos_token_id=1, pad_token_id=2, position_embedding_type="nope", rope_theta=10000, rope_scaling=None,
             m_emb=None, m_width=None, m_residual=None, init_method="normal", embedding_init_method="normal",
             use_depth_scaled_init=False, tie_word_embeddings=False, sequence_mixer_blocks=mixers,
             mlp_blocks=[dict(mlp_type="MLP", intermediate_size=64, activation_function="swiglu") for _ in range(L)])
    d.update(extra)
    return d


def _parity(cfg, atol=3e-5):
    ref = build_reference_model(cfg)
    ours = build_model(config_from_dict(cfg))
    ours.load_state_dict(ref.state_dict(), strict=True)
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 256, (2, 24), generator=g)
    o, r = ours(x).logits, ref(input_ids=x).logits
    assert torch.allclose(o, r, atol=atol, rtol=1e-4), (o - r).abs().max()
    o.float().pow(2).mean().backward()
    r.float().pow(2).mean().backward()
    for (n, po), (_, pr) in zip(ours.named_parameters(), ref.named_parameters()):
        assert torch.allclose(po.grad, pr.grad, atol=atol, rtol=1e-3), n


MAMBA = dict(sequence_mixer_type="mamba2", state_size=8, intermediate_size=64, num_heads=4, conv_kernel_size=4,
             activation_function="silu", num_groups=1, chunk_size=8, normalization_function="rmsnorm")
ATTN = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2)


def test_hybrid_mamba2_attention_matches_reference():
    _parity(_base(3, [MAMBA, dict(ATTN), MAMBA], position_embedding_type="rope", rope_dim=8))


RNN_ = dict(sequence_mixer_type="rnn", state_head_dim=8, num_input_heads=2, num_weight_heads=4, add_bias=False,
            normalization_function="rmsnorm", gradient_clipping=None, kernel_size=None, activation_function="tanh")
GRU_ = dict(sequence_mixer_type="gru", state_head_dim=8, num_input_heads=4, num_forget_input_heads=2,
            num_reset_input_heads=1, num_weight_heads=2, num_forget_weight_heads=4, num_reset_weight_heads=1,
            add_bias=True, normalization_function="rmsnorm", gradient_clipping=None, kernel_size=4,
            activation_function="silu")
M2RNN_ = dict(sequence_mixer_type="m2rnn", k_head_dim=4, v_head_dim=8, num_q_heads=2, num_k_heads=2, num_v_heads=4,
              num_f_heads=4, num_g_heads=4, num_weight_heads=4, use_residual=True, kernel_size=4,
              activation_function="silu", add_bias=False, gradient_clipping=None, normalization_function="rmsnorm")


def test_rnn_gru_match_reference():
    _parity(_base(2, [RNN_, GRU_]))


def test_m2rnn_matches_reference():
    _parity(_base(2, [M2RNN_, dict(ATTN)]))


def test_gated_delta_rule_properties():
    """No CPU reference exists in lm-engine for the delta rule; check the recurrence against its definition on a
    case with a closed form (beta = 1, no decay, orthonormal keys: the state stores v_t under k_t)."""
    from lm_engine_b200.ops.recurrence import gated_delta_rule_scan

    B, S, N, K, V = 1, 4, 1, 4, 3
    k = torch.eye(K)[None, :, None, :].expand(B, S, N, K).contiguous()
    v = torch.randn(B, S, N, V)
    g = torch.zeros(B, S, N)
    beta = torch.ones(B, S, N)
    y, h = gated_delta_rule_scan(k, k, v, g, beta, scale=1.0)
    assert torch.allclose(y, v, atol=1e-5)
    assert torch.allclose(h[0, 0], v[0, :, 0], atol=1e-5)
    cfg = _base(2, [dict(sequence_mixer_type="gated_deltanet", k_head_dim=4, v_head_dim=8, num_k_heads=2,
                         num_v_heads=4, use_gate=True, attention_multiplier=None, allow_neg_eigval=True,
                         kernel_size=4), dict(ATTN)])
    m = build_model(config_from_dict(cfg))
    out = m(torch.randint(0, 256, (2, 16))).logits
    out.float().pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())


def test_other_model_families_run_and_share_kv():
    x = torch.randint(0, 256, (2, 12))
    for mt in ("palm", "ladder_residual"):
        cfg = _base(2, [dict(ATTN), dict(ATTN)], model_type=mt, position_embedding_type="rope", rope_dim=8)
        ours = build_model(config_from_dict(cfg))
        ours(x).logits.float().pow(2).mean().backward()
        assert all(p.grad is not None for p in ours.parameters())
        try:
            # in this snapshot of the reference these two families fail inside their own constructors / forward
            # (TypeError); compare only when they run
            ref = build_reference_model(cfg)
            want = ref(input_ids=x).logits
        except TypeError:
            continue
        ours.load_state_dict(ref.state_dict(), strict=True)
        assert torch.allclose(ours(x).logits, want, atol=3e-5), mt
    cfg = _base(4, [dict(ATTN) for _ in range(4)], model_type="gpt_crosslayer", sharing_pattern=[0, 0, 2, 2],
                position_embedding_type="rope", rope_dim=8)
    m = build_model(config_from_dict(cfg))
    names = [n for n, _ in m.named_parameters()]
    assert any("h.0.kv_proj" in n for n in names) and not any("h.1.kv_proj" in n for n in names)
    m(x).logits.float().pow(2).mean().backward()
    assert all(p.grad is not None for p in m.parameters())


@pytest.mark.parametrize("S", [1, 63, 64, 150])
def test_chunk_parallel_forms_equal_the_token_recurrences(S):
    from lm_engine_b200.ops.recurrence import (gated_delta_rule_chunked, gated_delta_rule_scan,
                                               linear_attention_chunked, linear_attention_scan)

    torch.manual_seed(S)
    B, N, K, V = 2, 3, 8, 5
    q, k = torch.randn(B, S, N, K, dtype=torch.float64), torch.randn(B, S, N, K, dtype=torch.float64)
    v = torch.randn(B, S, N, V, dtype=torch.float64)
    h0 = torch.randn(B, N, K, V)
    y0, s0 = linear_attention_scan(q.float(), k.float(), v.float(), h0, 0.7)
    y1, s1 = linear_attention_chunked(q.float(), k.float(), v.float(), h0, 0.7, chunk=64)
    torch.testing.assert_close(y1, y0, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(s1, s0, rtol=2e-4, atol=2e-4)
    g = -torch.rand(B, S, N) * 0.2
    beta = torch.rand(B, S, N)
    a = [t.float().requires_grad_(True) for t in (q, k, v)]
    b = [t.float().requires_grad_(True) for t in (q, k, v)]
    y2, s2 = gated_delta_rule_scan(*a, g, beta, h0=h0)
    y3, s3 = gated_delta_rule_chunked(*b, g, beta, h0=h0, chunk=64)
    torch.testing.assert_close(y3, y2, rtol=3e-4, atol=3e-4)
    torch.testing.assert_close(s3, s2, rtol=3e-4, atol=3e-4)
    w = torch.randn_like(y2)
    (y2 * w).sum().backward()
    (y3 * w).sum().backward()
    for x, y in zip(a, b):
        torch.testing.assert_close(y.grad, x.grad, rtol=2e-3, atol=2e-3)


def test_gated_delta_rule_large_blocks_equal_the_token_recurrence():
    """Long sequences run the chunk-parallel form with 256-step blocks (fewer sequential block steps)."""
    from lm_engine_b200.ops import recurrence as rec

    torch.manual_seed(7)
    B, S, N, K, V = 1, 4 * rec.LONG_CHUNK + 37, 2, 8, 6
    q, k = torch.randn(B, S, N, K), torch.randn(B, S, N, K)
    v = torch.randn(B, S, N, V)
    g = -torch.rand(B, S, N) * 0.05
    beta = torch.rand(B, S, N)
    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v)]
    y2, s2 = rec.gated_delta_rule_scan(*a, g, beta)
    y3, s3 = rec.gated_delta_rule(*b, g, beta)          # dispatcher: S >= 4 * LONG_CHUNK takes the large blocks
    torch.testing.assert_close(y3, y2, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(s3, s2, rtol=1e-3, atol=1e-3)
    w = torch.randn_like(y2)
    (y2 * w).sum().backward()
    (y3 * w).sum().backward()
    for x, y in zip(a, b):
        torch.testing.assert_close(y.grad, x.grad, rtol=5e-3, atol=5e-3)


GDN_ = dict(sequence_mixer_type="gated_deltanet", k_head_dim=8, v_head_dim=8, num_k_heads=2, num_v_heads=4,
            use_gate=True, attention_multiplier=None, allow_neg_eigval=True, kernel_size=4,
            A_init_min=0, A_init_max=16, dt_init_min=0.001, dt_init_max=0.1, dt_init_floor=1e-4)
LINATT_ = dict(sequence_mixer_type="linear_attention", k_head_dim=4, v_head_dim=8, num_q_heads=2, num_k_heads=2,
               num_v_heads=4, num_g_heads=4, kernel_size=4, activation_function="silu", add_bias=False,
               attention_multiplier=None, normalization_function="rmsnorm")


@pytest.mark.parametrize("mixer", [RNN_, GRU_, M2RNN_, MAMBA, GDN_, LINATT_], ids=lambda m: m["sequence_mixer_type"])
def test_packed_tokens_equal_each_sequence_alone(mixer):
    """Padding-free input [T] with cu_seqlens through every recurrent mixer: logits and weight gradients equal those
    of the sequences run one at a time."""
    from lm_engine_b200.models.context import AttentionMaskInfo, PositionInfo

    torch.manual_seed(0)
    cfg = config_from_dict(_base(2, [dict(mixer), dict(mixer)]))
    packed = build_model(cfg, use_padding_free_transformer=True)
    plain = build_model(cfg)
    plain.load_state_dict(packed.state_dict())
    lens = [7, 12, 3]
    ids = torch.randint(0, 256, (sum(lens),))
    cu = torch.tensor([0, 7, 19, 22], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    out = packed(ids, attention_mask_info=AttentionMaskInfo(cu_seqlens=cu, max_seqlen=max(lens)),
                 position_info=PositionInfo(position_ids=pos)).logits
    assert out.shape[0] == sum(lens)
    alone = torch.cat([plain(ids[a:b][None]).logits[0] for a, b in zip(cu[:-1].tolist(), cu[1:].tolist())])
    torch.testing.assert_close(out, alone, atol=3e-5, rtol=1e-4)
    out.float().pow(2).mean().backward()
    alone.float().pow(2).mean().backward()
    for (n, a), (_, b) in zip(packed.named_parameters(), plain.named_parameters()):
        torch.testing.assert_close(a.grad, b.grad, atol=3e-5, rtol=1e-3, msg=n)


def test_left_padded_batch_runs_as_one_scan():
    """A padded batch without a state is one batched scan on masked inputs and equals the per-sample result."""
    from lm_engine_b200.models.layers.recurrent import run_per_sample
    from lm_engine_b200.ops.recurrence import rnn

    torch.manual_seed(0)
    x = torch.randn(3, 9, 2, 8)
    W = torch.randn(2, 8, 8) * 0.3
    mask = torch.ones(3, 9, dtype=torch.int64)
    mask[0, :4] = 0
    mask[2, :8] = 0
    calls = []

    def fn(t, st):
        calls.append(t[0].shape[0])
        return rnn(t[0], W, st, None)

    y, h = run_per_sample(fn, mask, [x], None)
    assert calls == [3]
    for b, n in enumerate((5, 9, 1)):
        yb, hb = rnn(x[b:b + 1, 9 - n:], W, None, None)
        torch.testing.assert_close(y[b:b + 1, 9 - n:], yb)
        torch.testing.assert_close(h[b:b + 1], hb)
        assert y[b, :9 - n].abs().max().item() == 0 if n < 9 else True


def test_sliding_window_counts_keys_like_the_reference():
    """``sliding_window = w`` lets a causal query see itself and the w keys before it (the reference passes
    (w, w) to flash-attn): moving a token w + 1 positions back must not change the last position's output, moving
    one w positions back must."""
    torch.manual_seed(0)
    w = 3
    cfg = config_from_dict(_base(1, [dict(sequence_mixer_type="softmax_attention", num_attention_heads=4,
                                          num_key_value_heads=2, sliding_window=w)]))
    model = build_model(cfg).eval()
    ids = torch.randint(3, 256, (1, 12))
    with torch.no_grad():
        base = model(input_ids=ids).logits[0, -1]
        far = ids.clone()
        far[0, 11 - (w + 1)] = (far[0, 11 - (w + 1)] + 7) % 256         # outside the window of position 11
        near = ids.clone()
        near[0, 11 - w] = (near[0, 11 - w] + 7) % 256                   # the oldest key inside it
        assert torch.allclose(model(input_ids=far).logits[0, -1], base, atol=1e-6)
        assert not torch.allclose(model(input_ids=near).logits[0, -1], base, atol=1e-4)


def test_mixers_without_a_context_parallel_form_refuse_it(monkeypatch):
    """RNN, GRU, linear attention and the gated delta net would treat a rank's shard as the whole sequence: they
    fail at construction under context parallelism instead (Mamba-2, M2RNN and softmax attention have a form)."""
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    monkeypatch.setattr(ProcessGroupManager, "is_context_parallel_enabled", staticmethod(lambda: True))
    for mixer in (RNN_, GRU_, LINATT_, GDN_):
        with pytest.raises(NotImplementedError, match="context parallelism"):
            build_model(config_from_dict(_base(1, [dict(mixer)])))
