"""Matrix-state RNN scan kernels against the PyTorch recurrence in fp32: output, final state and every gradient,
with shared heads, an initial state, gradient clipping, ragged lengths and several replay segments."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, r):
    return float((a.float() - r.float()).norm() / (r.float().norm() + 1e-6))


CASES = [
    # B, S, K, V, Nq, Nk, Nv, Nf, Nw, h0, clip
    (2, 37, 64, 16, 1, 1, 6, 6, 6, False, None),      # the published layout: one q/k head shared by all v heads
    (2, 64, 64, 16, 1, 1, 4, 4, 2, True, 1.0),
    (1, 50, 32, 32, 2, 2, 2, 2, 2, True, None),
    (2, 41, 64, 64, 2, 4, 4, 2, 4, False, 0.5),
    (1, 24, 16, 64, 3, 3, 3, 3, 1, True, None),
]


@pytest.mark.parametrize("B,S,K,V,Nq,Nk,Nv,Nf,Nw,with_h0,clip", CASES)
@pytest.mark.parametrize("segments", [1, 3])
def test_m2rnn_kernel_matches_scan(B, S, K, V, Nq, Nk, Nv, Nf, Nw, with_h0, clip, segments, monkeypatch):
    from lm_engine_b200.ops import m2rnn as op
    from lm_engine_b200.ops.recurrence import m2rnn_scan

    N = max(Nq, Nk, Nv, Nf, Nw)
    if segments > 1:   # force several replay segments of 16 steps
        monkeypatch.setattr(op, "RECORD_BYTES", 16 * B * N * K * V * 2)
    torch.manual_seed(1)
    bf, dev = torch.bfloat16, "cuda"
    # q / k / v as slices of one projection output (token stride larger than the head block), like the layer
    width = Nq * K + Nk * K + Nv * V
    xc = (torch.randn(B, S, width, device=dev) * 0.7).to(bf).requires_grad_(True)
    f = torch.sigmoid(torch.randn(B, S, Nf, device=dev) + 1).requires_grad_(True)
    W = (torch.eye(V, device=dev) + 0.2 * torch.randn(Nw, V, V, device=dev)).to(bf).requires_grad_(True)
    h0 = (torch.randn(B, N, K, V, device=dev) * 0.5).to(bf).requires_grad_(True) if with_h0 else None

    def split(t):
        q, k, v = t.split((Nq * K, Nk * K, Nv * V), dim=-1)
        return q.view(B, S, Nq, K), k.view(B, S, Nk, K), v.view(B, S, Nv, V)

    y, hS = op.m2rnn_cuda(*split(xc), f, W, h0, clip)
    dy = torch.randn_like(y)
    dhS = torch.randn_like(hS) * 0.3
    torch.autograd.backward([y, hS], [dy, dhS])

    ref_in = [t.detach().float().requires_grad_(True) if t is not None else None for t in (xc, f, W, h0)]
    yr, hr = m2rnn_scan(*split(ref_in[0]), ref_in[1], ref_in[2], ref_in[3], clip)
    torch.autograd.backward([yr, hr], [dy.float(), dhS.float()])

    assert _rel(y, yr) < 2e-2
    assert _rel(hS, hr) < 2e-2
    assert _rel(xc.grad, ref_in[0].grad) < 4e-2
    assert _rel(f.grad, ref_in[1].grad) < 4e-2
    assert _rel(W.grad, ref_in[2].grad) < 4e-2
    if with_h0:
        assert _rel(h0.grad, ref_in[3].grad) < 4e-2
