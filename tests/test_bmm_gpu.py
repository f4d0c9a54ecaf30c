"""Batched tcgen05 GEMM (3-D tensor maps) and the SSD chunk-boundary scan kernels against fp32 PyTorch statements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, r):
    return float((a.float() - r.float()).norm() / (r.float().norm() + 1e-9))


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("batch,M,N,K", [(5, 256, 64, 256), (3, 200, 40, 72), (7, 64, 256, 16), (2, 384, 512, 128),
                                         (300, 128, 128, 64)])
def test_bmm_matches_fp32_statement(a_mn, b_mn, batch, M, N, K):
    from lm_engine_b200.ops import _lib, bmm

    g = torch.Generator(device="cuda").manual_seed(batch * 1000 + M + N + K)
    a = torch.randn((batch, K, M) if a_mn else (batch, M, K), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((batch, K, N) if b_mn else (batch, N, K), device="cuda", generator=g).to(torch.bfloat16)
    a.requires_grad_(True)
    b.requires_grad_(True)
    out = bmm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert out.dtype == torch.float32 and out.shape == (batch, M, N)
    dy = torch.randn(out.shape, device="cuda", generator=g)
    out.backward(dy)
    A = (a.detach().float().transpose(1, 2) if a_mn else a.detach().float()).requires_grad_()
    B = (b.detach().float() if b_mn else b.detach().float().transpose(1, 2)).requires_grad_()
    ref = torch.bmm(A, B)
    ref.backward(dy.to(torch.bfloat16).float())            # the backward rounds the incoming gradient to bf16
    assert _rel(out, ref) < 2e-3
    assert _rel(a.grad, A.grad.transpose(1, 2) if a_mn else A.grad) < 1e-2
    assert _rel(b.grad, B.grad if b_mn else B.grad.transpose(1, 2)) < 1e-2
    assert _lib.read_status()[0] == 0


def test_bmm_bf16_output_and_strided_batches():
    from lm_engine_b200.ops import bmm

    g = torch.Generator(device="cuda").manual_seed(3)
    big = torch.randn(4, 2, 128, 64, device="cuda", generator=g).to(torch.bfloat16)
    a = big[:, 0]                                            # batch pitch 2 * 128 * 64: a view, not a copy
    b = torch.randn(4, 96, 64, device="cuda", generator=g).to(torch.bfloat16)
    out = bmm(a, b, out_dtype=torch.bfloat16)
    ref = torch.bmm(a.float(), b.float().transpose(1, 2))
    assert out.dtype == torch.bfloat16 and _rel(out, ref) < 1e-2


@pytest.mark.parametrize("with_init", [False, True])
def test_boundary_scan_matches_loop(with_init):
    from lm_engine_b200.ops.ssd import _BoundaryScan

    b, nc, N, P, Sd = 2, 9, 5, 32, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    states = torch.randn(b, nc, N, P, Sd, device="cuda", generator=g, requires_grad=True)
    decay = (torch.rand(b, nc, N, device="cuda", generator=g) * 0.9 + 0.05).requires_grad_(True)
    init = torch.randn(b, N, P, Sd, device="cuda", generator=g, requires_grad=True) if with_init else None
    h0, hf = _BoundaryScan.apply(states, decay, init)
    # h0 is a bf16 output, so autograd hands its gradient over in bf16: use weights that bf16 represents exactly
    w0 = torch.randn(h0.shape, device="cuda", generator=g).to(torch.bfloat16).float()
    wf = torch.randn(hf.shape, device="cuda", generator=g)
    ((h0.float() * w0).sum() + (hf * wf).sum()).backward()
    got = [states.grad.clone(), decay.grad.clone(), None if init is None else init.grad.clone()]
    s2, d2 = states.detach().clone().requires_grad_(), decay.detach().clone().requires_grad_()
    i2 = None if init is None else init.detach().clone().requires_grad_()
    h = torch.zeros(b, N, P, Sd, device="cuda") if i2 is None else i2
    starts = []
    for c in range(nc):
        starts.append(h)
        h = h * d2[:, c, :, None, None] + s2[:, c]
    r0 = torch.stack(starts, 1)
    ((r0 * w0).sum() + (h * wf).sum()).backward()
    assert _rel(h0, r0) < 5e-3 and _rel(hf, h) < 1e-5
    # the kernel's h0 output is bf16, so its gradient path sees w0 exactly; only rounding of the sums differs
    assert _rel(got[0], s2.grad) < 1e-4 and _rel(got[1], d2.grad) < 1e-4
    if with_init:
        assert _rel(got[2], i2.grad) < 1e-4
