"""The recurrences that the gated-delta-rule chain kernels implement (forward chain, reverse chain for the state
gradient, operand gradients as products over the state columns), written out in PyTorch and checked against autograd
through the block loop in float64."""

import torch


def _operands(B=2, N=2, nc=3, L=8, K=16, V=12, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64) * 0.3   # noqa: E731
    return (r(B, N, nc, L, K), r(B, N, nc, L, V), r(B, N, nc, L, K), r(B, N, nc, L, L), r(B, N, nc, L, K),
            torch.rand(B, N, nc, generator=g, dtype=torch.float64) * 0.5 + 0.5, r(B, N, K, V))


def test_reverse_chain_and_operand_gradients_match_autograd():
    from lm_engine_b200.ops.recurrence import delta_chain_reference

    ops = [t.clone().requires_grad_(True) for t in _operands()]
    y, hf = delta_chain_reference(*ops)
    gy, gh = torch.randn_like(y), torch.randn_like(hf)
    (y * gy).sum().backward(retain_graph=True)
    (hf * gh).sum().backward()
    want = [t.grad for t in ops]

    Wk, Wv, qe, qk, ke, a, h = [t.detach() for t in ops]
    nc = Wk.size(2)
    # forward chain: what the forward kernel leaves behind
    U, H = [], []
    for c in range(nc):
        H.append(h)
        U.append(Wv[:, :, c] - Wk[:, :, c] @ h)
        h = a[:, :, c, None, None] * h + ke[:, :, c].transpose(-1, -2) @ U[-1]
    # reverse chain: what the backward kernel computes
    dh = gh
    dU, dH = [None] * nc, [None] * nc
    for c in reversed(range(nc)):
        dH[c] = dh
        dU[c] = qk[:, :, c].transpose(-1, -2) @ gy[:, :, c] + ke[:, :, c] @ dh
        dh = (a[:, :, c, None, None] * dh + qe[:, :, c].transpose(-1, -2) @ gy[:, :, c]
              - Wk[:, :, c].transpose(-1, -2) @ dU[c])
    U, H, dU, dH = (torch.stack(t, dim=2) for t in (U, H, dU, dH))
    got = [-dU @ H.transpose(-1, -2), dU, gy @ H.transpose(-1, -2), gy @ U.transpose(-1, -2),
           U @ dH.transpose(-1, -2), (dH * H).sum((-1, -2)), dh]
    for name, u, v in zip(("Wk", "Wv", "qe", "qk", "ke", "a", "h0"), got, want):
        torch.testing.assert_close(u, v, rtol=1e-9, atol=1e-9, msg=lambda m, name=name: f"{name}: {m}")


def test_dispatcher_uses_the_block_loop_on_cpu():
    from lm_engine_b200.ops import recurrence as rec

    ops = _operands(K=128, V=64, L=64, nc=2)
    assert not rec.delta_chain_kernel_usable(ops[0], ops[1])
    y, h = rec.delta_chain(*ops)
    y2, h2 = rec.delta_chain_reference(*ops)
    assert torch.equal(y, y2) and torch.equal(h, h2)


def test_linear_attention_is_the_chain_without_correction():
    """``W_k = 0``, ``a = 1`` turns the delta-rule chain into linear attention: checked against the token recurrence
    (values, final state and gradients) with the PyTorch block loop standing in for the kernels."""
    from lm_engine_b200.ops import recurrence as rec

    torch.manual_seed(0)
    B, S, N, K, V = 2, 150, 2, 24, 40
    q, k, v = torch.randn(B, S, N, K) * 0.3, torch.randn(B, S, N, K) * 0.3, torch.randn(B, S, N, V)
    h0 = torch.randn(B, N, K, V) * 0.1
    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v)]
    y, h = rec.linear_attention_on_chain(*a, h0=h0, attention_multiplier=0.7, chain=rec.delta_chain_reference)
    y2, h2 = rec.linear_attention_scan(*b, h0=h0, attention_multiplier=0.7)
    torch.testing.assert_close(y, y2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(h, h2, rtol=1e-4, atol=1e-4)
    w = torch.randn_like(y2)
    (y * w).sum().backward()
    (y2 * w).sum().backward()
    for u, t in zip(a, b):
        torch.testing.assert_close(u.grad, t.grad, rtol=1e-3, atol=1e-4)
