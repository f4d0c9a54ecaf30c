"""Gated-delta-rule chain kernels (forward, backward) against the fp32 block loop on the same operands, and the whole
recurrence through the dispatcher against the token-by-token fp32 scan."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _operands(B, N, nc, K, V, seed=0):
    L = 64
    g = torch.Generator(device="cuda").manual_seed(seed)

    def r(*s, scale):
        return (torch.randn(*s, generator=g, device="cuda") * scale).to(torch.bfloat16).float()

    Wk = r(B, N, nc, L, K, scale=K ** -0.5)
    Wv = r(B, N, nc, L, V, scale=1.0)
    qe = r(B, N, nc, L, K, scale=K ** -0.5)
    qk = torch.tril(r(B, N, nc, L, L, scale=0.2))
    ke = r(B, N, nc, L, K, scale=K ** -0.5)
    a = torch.rand(B, N, nc, generator=g, device="cuda") * 0.5 + 0.5
    h = r(B, N, K, V, scale=0.5)
    return [Wk, Wv, qe, qk, ke, a, h]


@pytest.mark.parametrize("B,N,nc,K,V", [(1, 2, 1, 128, 64), (2, 3, 5, 256, 128), (1, 1, 16, 256, 512),
                                        (2, 2, 3, 128, 192),
                                        # enough (batch, head, 64-column slice) triples for the 64-column kernels
                                        (4, 4, 2, 128, 512), (4, 8, 3, 256, 256)])
def test_chain_kernels_match_block_loop(B, N, nc, K, V):
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.recurrence import _DeltaChain, delta_chain_kernel_usable, delta_chain_reference

    _lib.read_status(clear=True)
    ops = _operands(B, N, nc, K, V)
    assert delta_chain_kernel_usable(ops[0], ops[1])
    a_ops = [t.clone().requires_grad_(True) for t in ops]
    b_ops = [t.clone().requires_grad_(True) for t in ops]
    y, hf = _DeltaChain.apply(*a_ops)
    y2, hf2 = delta_chain_reference(*b_ops)
    assert _rel(y, y2) < 1e-2 and _rel(hf, hf2) < 1e-2, (_rel(y, y2), _rel(hf, hf2))
    g = torch.Generator(device="cuda").manual_seed(5)
    gy = torch.randn(y.shape, generator=g, device="cuda").to(torch.bfloat16).float()
    gh = torch.randn(hf.shape, generator=g, device="cuda") * 0.1
    ((y * gy).sum() + (hf * gh).sum()).backward()
    ((y2 * gy).sum() + (hf2 * gh).sum()).backward()
    for name, u, v in zip(("Wk", "Wv", "qe", "qk", "ke", "a", "h0"), a_ops, b_ops):
        assert _rel(u.grad, v.grad) < 2e-2, (name, _rel(u.grad, v.grad))
    torch.cuda.synchronize()
    assert _lib.read_status(clear=True)[0] == 0


def test_chain_without_state_gradient_and_without_initial_state():
    from lm_engine_b200.ops.recurrence import _DeltaChain, delta_chain_reference

    ops = _operands(1, 2, 4, 128, 64, seed=3)
    ops[-1] = torch.zeros_like(ops[-1])
    a_ops = [t.clone().requires_grad_(True) for t in ops]
    b_ops = [t.clone().requires_grad_(True) for t in ops]
    y, _ = _DeltaChain.apply(*a_ops)
    y2, _ = delta_chain_reference(*b_ops)
    y.square().sum().backward()
    y2.square().sum().backward()
    assert _rel(y, y2) < 1e-2
    for u, v in zip(a_ops[:5], b_ops[:5]):
        assert _rel(u.grad, v.grad) < 3e-2


@pytest.mark.parametrize("S,K,V", [(200, 128, 64), (512, 256, 128)])
def test_gated_delta_rule_on_kernels_matches_token_scan(S, K, V):
    from lm_engine_b200.ops import recurrence as rec

    torch.manual_seed(S)
    B, N = 2, 2
    q, k = (torch.randn(B, S, N, K, device="cuda") for _ in range(2))
    v = torch.randn(B, S, N, V, device="cuda")
    gl = -torch.rand(B, S, N, device="cuda") * 0.2
    beta = torch.rand(B, S, N, device="cuda")
    h0 = torch.randn(B, N, K, V, device="cuda") * 0.1
    a = [t.clone().requires_grad_(True) for t in (q, k, v, gl, beta)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v, gl, beta)]
    y, h = rec.gated_delta_rule(*a, h0=h0)                  # dispatcher: chain kernels
    y2, h2 = rec.gated_delta_rule_scan(*b, h0=h0)
    assert _rel(y, y2) < 2e-2 and _rel(h, h2) < 2e-2, (_rel(y, y2), _rel(h, h2))
    w = torch.randn_like(y2)
    (y * w).sum().backward()
    (y2 * w).sum().backward()
    for name, u, t in zip("qkvgb", a, b):
        assert _rel(u.grad, t.grad) < 5e-2, (name, _rel(u.grad, t.grad))


@pytest.mark.parametrize("S,K,V", [(300, 64, 64), (128, 16, 16), (520, 128, 96)])
def test_linear_attention_on_chain_kernels_matches_token_scan(S, K, V):
    from lm_engine_b200.ops import recurrence as rec

    torch.manual_seed(S + K)
    B, N = 2, 3
    q, k = (torch.randn(B, S, N, K, device="cuda") * K ** -0.5 for _ in range(2))
    v = torch.randn(B, S, N, V, device="cuda")
    h0 = torch.randn(B, N, K, V, device="cuda") * 0.1
    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v)]
    y, h = rec.linear_attention_on_chain(*a, h0=h0, attention_multiplier=0.5)
    y2, h2 = rec.linear_attention_scan(*b, h0=h0, attention_multiplier=0.5)
    assert y.shape == y2.shape and h.shape == h2.shape
    assert _rel(y, y2) < 2e-2 and _rel(h, h2) < 2e-2, (_rel(y, y2), _rel(h, h2))
    w = torch.randn_like(y2)
    (y * w).sum().backward()
    (y2 * w).sum().backward()
    for name, u, t in zip("qkv", a, b):
        assert _rel(u.grad, t.grad) < 4e-2, (name, _rel(u.grad, t.grad))
