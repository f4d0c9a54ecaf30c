"""Grouped (per-expert) GEMM kernels: forward, input gradient and weight gradient against a per-expert fp32 loop, with
empty experts, counts that are not multiples of the tile, and the fused SwiGLU epilogue; then the whole MoE layer."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(E, counts, K, N, seed=0):
    torch.manual_seed(seed)
    total = sum(counts)
    freq = torch.tensor(counts, device="cuda")
    ids = torch.repeat_interleave(torch.arange(E, device="cuda"), freq)
    x = torch.randn(total, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    return freq, ids, x, w


@pytest.mark.parametrize("counts", [[300, 0, 129, 1, 128, 77, 0, 512], [5, 3], [0, 0, 640, 0]])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_linear_matches_loop(counts, swiglu):
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.activation import swiglu_packed
    from lm_engine_b200.ops.moe import GroupLayout, grouped_linear_padded

    E, K, N = len(counts), 256, 384
    freq, ids, x, w = _case(E, counts, K, N)
    x.requires_grad_(True)
    w.requires_grad_(True)
    layout = GroupLayout(ids, freq)
    y = layout.gather(grouped_linear_padded(layout.scatter(x), w, layout, swiglu=swiglu))
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    outs, start = [], 0
    for e, n in enumerate(counts):
        o = xr[start:start + n] @ wr[e].t()
        outs.append(swiglu_packed(o) if swiglu else o)
        start += n
    ref = torch.cat(outs)
    ref.backward(dy.float())

    def rel(a, b):
        return float((a.float() - b).norm() / (b.norm() + 1e-6))

    assert rel(y, ref) < 1e-2
    assert rel(x.grad, xr.grad) < 1.5e-2
    assert rel(w.grad, wr.grad) < 1.5e-2
    for e, n in enumerate(counts):
        if n == 0:
            assert float(w.grad[e].abs().max()) == 0.0
    assert _lib.read_status()[0] == 0


def test_grouped_wgrad_accumulates_into_main_grad():
    from lm_engine_b200.ops.moe import GroupLayout, grouped_linear_padded

    counts = [130, 0, 64]
    freq, ids, x, w = _case(3, counts, 128, 192, seed=1)
    w.requires_grad_(True)
    w.main_grad = torch.full_like(w, 3.0)
    w.main_grad_stale = True
    layout = GroupLayout(ids, freq)
    for _ in range(2):
        y = layout.gather(grouped_linear_padded(layout.scatter(x), w, layout))
        y.backward(torch.ones_like(y))
    start, ref = 0, torch.zeros_like(w, dtype=torch.float32)
    for e, n in enumerate(counts):
        ref[e] = torch.ones(n, 192, device="cuda").t() @ x[start:start + n].float()
        start += n
    torch.testing.assert_close(w.main_grad.float(), 2 * ref, rtol=3e-2, atol=3e-2)


def test_moe_layer_grouped_path_matches_loop_path():
    from lm_engine_b200.models import config_from_dict, dense_config
    from lm_engine_b200.models.layers.moe import MoE
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=0)
    d = dense_config(vocab_size=64, hidden_size=256, num_layers=1, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=128, max_position_embeddings=64).to_dict()
    d["mlp_blocks"] = [{"mlp_type": "MoE", "intermediate_size": 128, "num_experts": 8, "num_experts_per_tok": 2,
                        "activation_function": "swiglu", "shared_intermediate_size": None, "add_bias": False}]
    cfg = config_from_dict(d)
    torch.manual_seed(0)
    moe = MoE(256, cfg.mlp_blocks[0], "normal", 0.02, None, 1, True).cuda().to(torch.bfloat16)
    x = torch.randn(4, 96, 256, device="cuda").to(torch.bfloat16)

    def run(grouped):
        moe.zero_grad()
        moe._grouped_kernels = (lambda xs: False) if not grouped else MoE._grouped_kernels.__get__(moe)
        xi = x.clone().requires_grad_(True)
        y = moe(xi)
        y.float().pow(2).sum().backward()
        return y, xi.grad, moe.c_fc.weight.grad.clone(), moe.c_proj.weight.grad.clone()

    a, b = run(True), run(False)
    for u, v in zip(a, b):
        assert float((u.float() - v.float()).norm() / (v.float().norm() + 1e-6)) < 2e-2


def test_dispatch_combine_kernels_match_index_ops():
    from lm_engine_b200.ops.moe import GroupLayout, combine_tokens, dispatch_tokens

    torch.manual_seed(3)
    T, K, E, H = 300, 2, 8, 64
    sel = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)])
    gates = torch.rand(T, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    se, order = sel.flatten().sort()
    freq = torch.bincount(se, minlength=E)
    layout = GroupLayout(se, freq, order=order, top_k=K)
    xp = dispatch_tokens(x, layout)
    token = order // K
    assert torch.equal(xp[layout.dest], x.detach()[token])
    assert float(xp.float().abs().sum()) == pytest.approx(float(x.detach()[token].float().abs().sum()), rel=1e-6)
    yp = (torch.randn_like(xp) * (xp.abs().sum(-1, keepdim=True) > 0)).requires_grad_(True)
    out = combine_tokens(yp, gates, layout)
    ref_g = gates.detach().float().requires_grad_(True)
    ref_y = yp.detach().float().requires_grad_(True)
    ref = torch.zeros(T, H, device="cuda").index_add(0, token, ref_y[layout.dest] * ref_g.flatten()[order][:, None])
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    do = torch.randn_like(out)
    (out.float() * do.float()).sum().backward()
    (ref * do.float()).sum().backward()
    torch.testing.assert_close(yp.grad.float(), ref_y.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(gates.grad.float(), ref_g.grad, rtol=3e-2, atol=3e-2)
    xp.backward(torch.ones_like(xp))
    torch.testing.assert_close(x.grad.float(), torch.full_like(x, float(K)).float())


@pytest.mark.parametrize("T,K,E", [(300, 2, 8), (5000, 8, 64), (7, 1, 3), (4096, 4, 1000)])
def test_route_layout_kernels_match_sort_based_layout(T, K, E):
    """The counting-sort layout equals the one derived from a stable sort, entry by entry."""
    from lm_engine_b200.ops.moe import GroupLayout

    torch.manual_seed(T + K)
    sel = torch.randint(0, E, (T, K), device="cuda")
    if E > 4:
        sel[sel == 2] = 3                       # an empty expert
    se, order = sel.flatten().sort(stable=True)
    freq = torch.bincount(se, minlength=E)
    ref = GroupLayout(se, freq, order=order, top_k=K)
    got = GroupLayout.from_selection(sel, E)
    assert got.capacity == ref.capacity
    assert torch.equal(got.freq, freq)
    assert torch.equal(got.k0, ref.k0) and torch.equal(got.kb, ref.kb)
    assert torch.equal(got.tile_group, ref.tile_group)
    assert torch.equal(got.slot, ref.slot)


@pytest.mark.parametrize("normalized", [True, False])
@pytest.mark.parametrize("T,E,K", [(1000, 64, 8), (33, 8, 2), (257, 500, 1), (64, 40, 32)])
def test_topk_softmax_kernel_matches_fp32_reference(normalized, T, E, K):
    from lm_engine_b200.ops.moe import topk_softmax

    torch.manual_seed(E + K)
    # distinct bf16 values in a row, so that the selection has no ties
    base = torch.stack([torch.randperm(E, device="cuda") for _ in range(T)]).float()
    logits = ((base - E / 2) * (8.0 / E)).to(torch.bfloat16)
    if E > 256:
        logits = (base - E / 2).to(torch.bfloat16)                 # integers below 256 are exact in bf16
    lg = logits.clone().requires_grad_(True)
    w, sel = topk_softmax(lg, K, normalized)
    ref_l = logits.float().requires_grad_(True)
    if normalized:
        rv, rs = ref_l.topk(K, dim=-1)
        rw = torch.softmax(rv, dim=-1)
    else:
        rw, rs = torch.softmax(ref_l, dim=-1).topk(K, dim=-1)
    assert torch.equal(sel, rs)
    torch.testing.assert_close(w.float(), rw, rtol=1e-2, atol=1e-3)
    dw = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w.backward(dw)
    rw.backward(dw.float())
    torch.testing.assert_close(lg.grad.float(), ref_l.grad, rtol=2e-2, atol=2e-3)
