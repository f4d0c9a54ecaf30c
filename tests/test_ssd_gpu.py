"""SSD chunk scan with the fused intra-chunk kernels against the plain PyTorch path (same op, fp32 math) on bf16
inputs: outputs, final state and every gradient."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,L,N,G", [(256, 64, 8, 1), (200, 128, 4, 2), (512, 256, 8, 8)])
def test_fused_intra_chunk_matches_reference_path(S, L, N, G):
    import sys

    from lm_engine_b200.ops.ssd import ssd_chunk_scan

    mod = sys.modules["lm_engine_b200.ops.ssd"]
    torch.manual_seed(0)
    b, P, Sd = 2, 32, 16
    bf = torch.bfloat16

    def inputs():
        g = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn(b, S, N, P, device="cuda", generator=g).to(bf).requires_grad_(True)
        dt = (torch.rand(b, S, N, device="cuda", generator=g) * 0.3 + 0.01).to(bf).requires_grad_(True)
        A = (-torch.rand(N, device="cuda", generator=g) - 0.1).requires_grad_(True)
        B = (torch.randn(b, S, G, Sd, device="cuda", generator=g) * 0.5).to(bf).requires_grad_(True)
        C = (torch.randn(b, S, G, Sd, device="cuda", generator=g) * 0.5).to(bf).requires_grad_(True)
        D = torch.randn(N, device="cuda", generator=g).requires_grad_(True)
        return x, dt, A, B, C, D

    outs = []
    for fused in (True, False):
        mod.FUSED_INTRA_CHUNK = fused
        ins = inputs()
        y, h = ssd_chunk_scan(*ins, L)
        g = torch.Generator(device="cuda").manual_seed(2)
        dy = torch.randn(y.shape, device="cuda", generator=g).to(bf)
        (y.float() * dy.float()).sum().backward()
        outs.append((y, h, [t.grad for t in ins]))
    mod.FUSED_INTRA_CHUNK = True

    def rel(a, r):
        return float((a.float() - r.float()).norm() / (r.float().norm() + 1e-6))

    (y1, h1, g1), (y0, h0, g0) = outs
    assert rel(y1, y0) < 2e-2 and rel(h1, h0) < 1e-3
    for name, a, r in zip("x dt A B C D".split(), g1, g0):
        # A's gradient is one strongly cancelling sum per head over every token: looser bound
        assert rel(a, r) < (1e-1 if name == "A" else 4e-2), (name, rel(a, r))


def test_scan_kernels_with_an_initial_state_and_wider_heads():
    """P = 64, grouped B / C, a carried-in state (the generation / context-parallel entry) and a ragged length."""
    import sys

    from lm_engine_b200.ops.ssd import ssd_chunk_scan

    mod = sys.modules["lm_engine_b200.ops.ssd"]
    b, S, L, N, G, P, Sd = 2, 300, 64, 8, 2, 64, 32
    bf = torch.bfloat16

    def inputs():
        g = torch.Generator(device="cuda").manual_seed(3)
        x = torch.randn(b, S, N, P, device="cuda", generator=g).to(bf).requires_grad_(True)
        dt = (torch.rand(b, S, N, device="cuda", generator=g) * 0.3 + 0.01).to(bf).requires_grad_(True)
        A = (-torch.rand(N, device="cuda", generator=g) - 0.1).requires_grad_(True)
        B = (torch.randn(b, S, G, Sd, device="cuda", generator=g) * 0.5).to(bf).requires_grad_(True)
        C = (torch.randn(b, S, G, Sd, device="cuda", generator=g) * 0.5).to(bf).requires_grad_(True)
        D = torch.randn(N, device="cuda", generator=g).requires_grad_(True)
        h0 = (torch.randn(b, N, P, Sd, device="cuda", generator=g) * 0.5).requires_grad_(True)
        return x, dt, A, B, C, D, h0

    outs = []
    for fused in (True, False):
        mod.FUSED_INTRA_CHUNK = fused
        *ins, h0 = inputs()
        y, h = ssd_chunk_scan(*ins, L, initial_state=h0)
        g = torch.Generator(device="cuda").manual_seed(4)
        dy = torch.randn(y.shape, device="cuda", generator=g).to(bf)
        dh = torch.randn(h.shape, device="cuda", generator=g) * 0.1
        ((y.float() * dy.float()).sum() + (h * dh).sum()).backward()
        outs.append((y, h, [t.grad for t in (*ins, h0)]))
    mod.FUSED_INTRA_CHUNK = True

    def rel(a, r):
        return float((a.detach().float() - r.detach().float()).norm() / (r.detach().float().norm() + 1e-6))

    (y1, h1, g1), (y0, h0_, g0) = outs
    assert rel(y1, y0) < 2e-2 and rel(h1, h0_) < 5e-3
    for name, a, r in zip("x dt A B C D h0".split(), g1, g0):
        assert rel(a, r) < (1e-1 if name == "A" else 4e-2), (name, rel(a, r))
