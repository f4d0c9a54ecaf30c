"""Depthwise causal conv1d kernels against the PyTorch statement (fp32), forward and all gradients."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S,C,K", [(2, 200, 64, 4), (1, 64, 1032, 4), (3, 70, 32, 2), (2, 130, 48, 7), (2, 5, 16, 4)])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("with_state", [False, True])
def test_causal_conv1d_matches_reference(B, S, C, K, act, with_state):
    from lm_engine_b200.ops.conv1d import causal_conv1d, causal_conv1d_reference

    torch.manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn(B, S, C, device="cuda").to(bf).requires_grad_(True)
    w = (torch.randn(C, K, device="cuda") * 0.5).to(bf).requires_grad_(True)
    b = torch.randn(C, device="cuda").to(bf).requires_grad_(True)
    st = torch.randn(B, C, K - 1, device="cuda").to(bf).requires_grad_(True) if with_state else None
    y = causal_conv1d(x, w, b, st, act)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref_in = [t.detach().float().requires_grad_(True) if t is not None else None for t in (x, w, b, st)]
    ref = causal_conv1d_reference(*ref_in, act)
    ref.backward(dy.float())

    def close(a, r, tol):
        assert float((a.float() - r).norm() / (r.norm() + 1e-6)) < tol

    close(y, ref, 1e-2)
    close(x.grad, ref_in[0].grad, 1.5e-2)
    close(w.grad, ref_in[1].grad, 1.5e-2)
    close(b.grad, ref_in[2].grad, 1.5e-2)
    if with_state:
        close(st.grad, ref_in[3].grad, 1.5e-2)
