"""Every CUDA kernel against a plain PyTorch fp32 statement of the same op (B200 only)."""

import pytest
import torch

from lm_engine_b200 import ops
from lm_engine_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _status_ok():
    st = _lib.read_status()
    assert st[0] == 0, f"device status {st}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (384, 768, 192), (200, 264, 136), (1024, 128, 256),
                                   (64, 64, 64), (4096, 4096, 1024), (8192, 1024, 4096)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    # plain fp32 statement of the product (no reduced-precision library path: TF32 is off by default)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_err(out, ref) < 5e-3


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 512, 1024, 384
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    assert _rel_err(ops.gemm(a, b, bias=bias), ref + bias.float()) < 5e-3
    assert _rel_err(ops.gemm(a, b, residual=res), ref + res.float()) < 5e-3
    acc32 = torch.randn(M, N, device=DEV, dtype=torch.float32)
    want = acc32 + ref
    ops.gemm(a, b, out=acc32, accumulate=True)
    assert _rel_err(acc32, want) < 1e-3
    acc16 = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    want = acc16.float() + ref
    ops.gemm(a, b, out=acc16, accumulate=True)
    assert _rel_err(acc16, want) < 5e-3
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    y = ops.gemm(a, b, swiglu=True, preact=pre)
    assert _rel_err(pre, ref) < 5e-3
    assert _rel_err(y, ops.swiglu_packed_reference(ref.to(torch.bfloat16))) < 1e-2
    _status_ok()


def test_linear_autograd_matches_torch():
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    b = torch.randn(512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 5e-3
    assert _rel_err(w.grad, wr.grad) < 5e-3
    assert _rel_err(b.grad, br.grad) < 5e-3
    # main_grad accumulation path
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(512, 256, device=DEV, dtype=torch.float32)
    for _ in range(2):
        ops.linear(x.detach(), w2, None).backward(g)
    assert w2.grad is None
    assert _rel_err(w2.main_grad, 2 * wr.grad) < 5e-3
    _status_ok()


@pytest.mark.parametrize("T,H", [(64, 128), (333, 4096), (17, 1024), (9, 8192), (5, 16384)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(T, H, with_res):
    torch.manual_seed(3)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device=DEV, dtype=torch.bfloat16)).requires_grad_()
    y, h = ops.rmsnorm(x, w, 1e-5, residual=r)
    gy, gh = torch.randn_like(y), torch.randn_like(y)
    loss_terms = [(y, gy)] + ([(h, gh)] if with_res else [])
    torch.autograd.backward([t for t, _ in loss_terms], [g for _, g in loss_terms])
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    hr = xr + rr if with_res else xr
    if with_res:
        hr = hr.detach().to(torch.bfloat16).float() + (hr - hr.detach())  # straight-through the bf16 rounding of the sum
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    torch.autograd.backward([yr] + ([hr] if with_res else []), [gy.float()] + ([gh.float()] if with_res else []))
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    if with_res:
        assert _rel_err(r.grad, rr.grad) < 1e-2


def test_swiglu():
    torch.manual_seed(4)
    x = torch.randn(37, 2 * 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.swiglu_packed(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = xr[..., 1::2] * torch.nn.functional.silu(xr[..., ::2])
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2


@pytest.mark.parametrize("D,rd", [(128, 128), (64, 64), (128, 64)])
def test_qkv_rope(D, rd):
    from lm_engine_b200.ops.rope import qkv_split_rope_reference

    torch.manual_seed(5)
    B, S, Hkv, G = 2, 48, 2, 4
    qkv = torch.randn(B, S, Hkv * (G + 2) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    inv = 1.0 / (10000 ** (torch.arange(0, rd, 2, device=DEV).float() / rd))
    ang = torch.outer(torch.arange(S, device=DEV).float(), inv)
    ang = torch.cat((ang, ang), -1)
    cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
    q, k, v = ops.qkv_split_rope(qkv, Hkv, G, D, cos_t, sin_t, None, S)
    gs = [torch.randn_like(t) for t in (q, k, v)]
    torch.autograd.backward([q, k, v], gs)
    xr = qkv.detach().float().requires_grad_()
    pos = torch.arange(S, device=DEV).expand(B, S)
    qr, kr, vr = qkv_split_rope_reference(xr, Hkv, G, D, cos_t[pos], sin_t[pos])
    torch.autograd.backward([qr, kr, vr], [g.float() for g in gs])
    for a, b in ((q, qr), (k, kr), (v, vr), (qkv.grad, xr.grad)):
        assert _rel_err(a, b) < 1e-2


@pytest.mark.parametrize("T,V", [(64, 2048), (33, 50304), (16, 128256)])
def test_cross_entropy(T, V):
    torch.manual_seed(6)
    logits = (torch.randn(T, V, device=DEV) * 2).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    ref_in = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, labels, reduction="sum", ignore_index=-100)
    (ref * 0.37).backward()
    x = logits.detach().clone().requires_grad_()
    loss = ops.cross_entropy_sum(x, labels)
    (loss * 0.37).backward()
    assert abs(loss.item() - ref.item()) / abs(ref.item()) < 1e-3
    assert _rel_err(x.grad, ref_in.grad) < 1e-2


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_and_norm(gdtype):
    torch.manual_seed(7)
    n = 1_000_003
    p = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    plp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pr = p.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=3e-4, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(gdtype)
        ss = torch.zeros(1, device=DEV)
        ops.sumsq_(g, ss)
        norm, coef = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
        ops.clip_coef_(ss, 1.0, norm, coef)
        assert abs(norm.item() - g.float().norm().item()) / norm.item() < 1e-4
        ops.adamw_step(p, m, v, g, plp, lr=3e-4, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1, step=step,
                       gscale=coef)
        pr.grad = g.float() * coef
        opt.step()
    assert _rel_err(p, pr.detach()) < 1e-5
    assert _rel_err(plp, pr.detach()) < 5e-3
