"""Layout algebra of the batched product's backward pass, checked on CPU: the kernel launch is replaced by its
PyTorch statement, so what is tested is which operands and layout flags the two gradient products use."""

import pytest
import torch

import importlib

G = importlib.import_module("lm_engine_b200.ops.gemm")   # the package re-exports a function of the same name


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
def test_bmm_gradients_for_every_layout(monkeypatch, a_mn, b_mn):
    monkeypatch.setattr(G, "_bmm_kernel", lambda a, b, am, bm, dt: G.bmm_reference(a, b, a_mn=am, b_mn=bm,
                                                                                   out_dtype=torch.float64))
    torch.manual_seed(0)
    batch, M, N, K = 3, 5, 7, 4
    a = torch.randn((batch, K, M) if a_mn else (batch, M, K), dtype=torch.float64, requires_grad=True)
    b = torch.randn((batch, K, N) if b_mn else (batch, N, K), dtype=torch.float64, requires_grad=True)
    g = torch.randn(batch, M, N, dtype=torch.float64)

    class _F64(G._Bmm):
        @staticmethod
        def backward(ctx, grad):   # keep fp64: the production backward rounds the incoming gradient to bf16
            a_, b_ = ctx.saved_tensors
            am, bm = ctx.cfg
            da = G._bmm_kernel(b_, grad, not bm, False, None) if am else G._bmm_kernel(grad, b_, False, not bm, None)
            db = G._bmm_kernel(a_, grad, not am, True, None) if bm else G._bmm_kernel(grad, a_, True, not am, None)
            return da, db, None, None, None

    out = _F64.apply(a, b, a_mn, b_mn, torch.float64)
    out.backward(g)
    A = a.detach().transpose(1, 2) if a_mn else a.detach()
    B = b.detach() if b_mn else b.detach().transpose(1, 2)          # [batch, K, N]
    A, B = A.clone().requires_grad_(), B.clone().requires_grad_()
    ref = torch.bmm(A, B)
    ref.backward(g)
    assert torch.allclose(out, ref)
    assert torch.allclose(a.grad, A.grad.transpose(1, 2) if a_mn else A.grad)
    assert torch.allclose(b.grad, B.grad if b_mn else B.grad.transpose(1, 2))


def test_production_backward_uses_the_same_products():
    """The fp64 copy of the backward above must stay in step with the real one: same branches, same flags."""
    import inspect

    src = inspect.getsource(G._Bmm.backward)
    assert "_bmm_kernel(b, g, not b_mn, False" in src and "_bmm_kernel(g, b, False, not b_mn" in src
    assert "_bmm_kernel(a, g, not a_mn, True" in src and "_bmm_kernel(g, a, True, not a_mn" in src
