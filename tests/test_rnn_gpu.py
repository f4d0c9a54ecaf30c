"""Vector-state RNN / GRU scan kernels against the PyTorch recurrences in fp32: outputs, final state and every
gradient, with shared heads, an initial state, gradient clipping, more than 16 batch rows and ragged lengths."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, r):
    return float((a.detach().float() - r.detach().float()).norm() / (r.detach().float().norm() + 1e-6))


@pytest.mark.parametrize("B,S,H,Nx,Nw,with_h0,clip", [
    (2, 37, 16, 6, 6, False, None),
    (3, 64, 16, 2, 4, True, 1.0),
    (19, 21, 32, 4, 2, True, None),
    (2, 30, 64, 3, 3, False, 0.5),
])
def test_rnn_kernel_matches_scan(B, S, H, Nx, Nw, with_h0, clip):
    from lm_engine_b200.ops.recurrence import rnn_scan
    from lm_engine_b200.ops.rnn import rnn_cuda

    torch.manual_seed(2)
    bf, dev = torch.bfloat16, "cuda"
    N = max(Nx, Nw)
    # x as a slice of a wider projection output, like the layer
    proj = torch.randn(B, S, Nx * H + 32, device=dev).to(bf).requires_grad_(True)
    W = (torch.randn(Nw, H, H, device=dev) / H ** 0.5).to(bf).requires_grad_(True)
    h0 = (torch.randn(B, N, H, device=dev) * 0.5).to(bf).requires_grad_(True) if with_h0 else None
    y, hS = rnn_cuda(proj[..., :Nx * H].view(B, S, Nx, H), W, h0, clip)
    dy, dhS = torch.randn_like(y), torch.randn_like(hS)
    torch.autograd.backward([y, hS], [dy, dhS])
    ref = [t.detach().float().requires_grad_(True) if t is not None else None for t in (proj, W, h0)]
    yr, hr = rnn_scan(ref[0][..., :Nx * H].view(B, S, Nx, H), ref[1], ref[2], clip)
    torch.autograd.backward([yr, hr], [dy.float(), dhS.float()])
    assert _rel(y, yr) < 2e-2 and _rel(hS, hr) < 2e-2
    assert _rel(proj.grad, ref[0].grad) < 4e-2
    assert _rel(W.grad, ref[1].grad) < 4e-2
    if with_h0:
        assert _rel(h0.grad, ref[2].grad) < 4e-2


@pytest.mark.parametrize("B,S,H,heads,wheads,with_h0,clip", [
    (2, 37, 16, (4, 4, 4), (4, 4, 4), False, None),
    (3, 40, 16, (1, 4, 2), (4, 2, 1), True, 1.0),
    (18, 19, 32, (2, 2, 2), (2, 1, 2), True, None),
])
def test_gru_kernel_matches_scan(B, S, H, heads, wheads, with_h0, clip):
    from lm_engine_b200.ops.recurrence import gru_scan
    from lm_engine_b200.ops.rnn import gru_cuda

    torch.manual_seed(3)
    bf, dev = torch.bfloat16, "cuda"
    N = max(*heads, *wheads)
    widths = [n * H for n in heads]
    proj = torch.randn(B, S, sum(widths), device=dev).to(bf).requires_grad_(True)
    Ws = [(torch.randn(n, H, H, device=dev) / H ** 0.5).to(bf).requires_grad_(True) for n in wheads]
    h0 = (torch.randn(B, N, H, device=dev) * 0.5).to(bf).requires_grad_(True) if with_h0 else None

    def split(t):
        return [p.view(B, S, n, H) for p, n in zip(t.split(widths, dim=-1), heads)]

    y, hS = gru_cuda(*split(proj), *Ws, h0, clip)
    dy, dhS = torch.randn_like(y), torch.randn_like(hS)
    torch.autograd.backward([y, hS], [dy, dhS])
    ref = [t.detach().float().requires_grad_(True) if t is not None else None for t in (proj, *Ws, h0)]
    yr, hr = gru_scan(*split(ref[0]), ref[1], ref[2], ref[3], ref[4], clip)
    torch.autograd.backward([yr, hr], [dy.float(), dhS.float()])
    assert _rel(y, yr) < 2e-2 and _rel(hS, hr) < 2e-2
    assert _rel(proj.grad, ref[0].grad) < 4e-2
    for w, r in zip(Ws, ref[1:4]):
        assert _rel(w.grad, r.grad) < 4e-2
    if with_h0:
        assert _rel(h0.grad, ref[4].grad) < 4e-2
