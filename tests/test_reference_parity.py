"""Loss / gradient parity of the dense model with the unmodified reference on CPU fp32 (same weights copied over)."""

import torch

from lm_engine_b200.models import build_model, dense_config

from .refutil import build_reference_model


def _cfg():
    return dense_config(vocab_size=2048, hidden_size=256, num_layers=4, num_attention_heads=4, num_key_value_heads=2,
                        intermediate_size=1024, head_dim=64, max_position_embeddings=512)


def test_forward_backward_matches_reference():
    cfg = _cfg()
    ref = build_reference_model(cfg.to_dict())
    torch.manual_seed(0)
    ours = build_model(cfg)
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    g = torch.Generator().manual_seed(1234)
    tokens = torch.randint(0, 2048, (2, 129), generator=g)
    x, y = tokens[:, :-1], tokens[:, 1:]
    lo = ours(x).logits
    lr = ref(input_ids=x).logits
    assert torch.allclose(lo, lr, atol=2e-5, rtol=1e-5)
    loss_o = torch.nn.functional.cross_entropy(lo.float().reshape(-1, 2048), y.reshape(-1))
    loss_r = torch.nn.functional.cross_entropy(lr.float().reshape(-1, 2048), y.reshape(-1))
    loss_o.backward()
    loss_r.backward()
    for (n, po), (_, pr) in zip(ours.named_parameters(), ref.named_parameters()):
        assert torch.allclose(po.grad, pr.grad, atol=1e-5, rtol=1e-4), n
