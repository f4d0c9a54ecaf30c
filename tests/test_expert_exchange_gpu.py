"""Expert-parallel exchange kernels with all ranks of the group emulated on ONE GPU: every phase runs for all ranks
before the next phase starts, so each wait finds its flag already set (kernels of different ranks never wait on one
another here).  The layout, the landed rows, the zeroed tile tails, both pull modes and the overflow report are
checked against plain PyTorch indexing."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, E, K, T, H, cap, seed=0):
    from lm_engine_b200.ops.moe import GroupLayout
    from lm_engine_b200.parallel.expert_exchange import RankBuffers

    g = torch.Generator(device="cuda").manual_seed(seed)
    ranks = RankBuffers.emulated(world, E, cap, H, T, K, "cuda")
    sel = [torch.randint(0, E, (T, K), device="cuda", generator=g) for _ in range(world)]
    if E > 4:
        for s in sel:
            s[s == 1] = 2                                    # an expert nobody selects
    x = [torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16) for _ in range(world)]
    layouts = [GroupLayout.from_selection(sel[r], E) for r in range(world)]
    seqs = [ranks[r].publish_counts(layouts[r]) for r in range(world)]
    plans = [ranks[r].make_plan(sel[r], layouts[r], seqs[r]) for r in range(world)]
    return ranks, sel, x, plans, seqs


@pytest.mark.parametrize("world,E,K,T,H", [(2, 4, 2, 300, 64), (4, 16, 2, 257, 128), (8, 64, 8, 512, 256),
                                           (1, 8, 2, 100, 64)])
def test_exchange_round_trip_emulated_ranks(world, E, K, T, H):
    from lm_engine_b200.ops import _lib

    _lib.read_status(clear=True)
    Le = E // world
    cap = (world * T * K + 127) // 128 * 128 + Le * 128        # worst case: nothing can overflow
    ranks, sel, x, plans, seqs = _setup(world, E, K, T, H, cap)
    for r in range(world):
        ranks[r].offer(x[r], plans[r], True, seqs[r])
    x_pads = [ranks[r].land(plans[r], True, seqs[r]) for r in range(world)]

    # reference layout of owner r: experts in order, inside an expert the sources in rank order, inside a source the
    # assignments in (token, k) order
    for r in range(world):
        own = plans[r].owner_layout
        k0, kb, tg = own.k0.tolist(), own.kb.tolist(), own.tile_group.tolist()
        row = 0
        for le in range(Le):
            e = r * Le + le
            want = torch.cat([x[s][(sel[s] == e).flatten().nonzero().flatten() // K] for s in range(world)])
            n = want.size(0)
            pad = (n + 127) // 128 * 128
            assert k0[le] == row and kb[le] == pad // 64
            assert torch.equal(x_pads[r][row:row + n], want)
            assert float(x_pads[r][row + n:row + pad].float().abs().sum()) == 0.0
            assert all(t == le for t in tg[row // 128:(row + pad) // 128])
            row += pad
        assert all(t == -1 for t in tg[row // 128:])
        assert int(plans[r].rows_own.sum()) == sum(int((sel[s] // Le == r).sum()) for s in range(world))

    # forward pull: each assignment gets its own row back (the "experts" double the rows)
    for r in range(world):
        ranks[r].publish_output(x_pads[r] * 2, True, seqs[r])
    for r in range(world):
        rows = ranks[r].pull(plans[r], False, True, seqs[r])
        assert torch.equal(rows.view(T, K, H), (x[r] * 2)[:, None, :].expand(T, K, H))

    # backward direction: push one gradient row per assignment, pull the sum over k
    g = torch.Generator(device="cuda").manual_seed(7)
    dy = [torch.randn(T * K, H, device="cuda", generator=g).to(torch.bfloat16) for _ in range(world)]
    for r in range(world):
        ranks[r].seq_b += 1
        plans[r].seq_b = ranks[r].seq_b
        ranks[r].offer(dy[r], plans[r], False, plans[r].seq_b)
    dy_pads = [ranks[r].land(plans[r], False, plans[r].seq_b) for r in range(world)]
    for r in range(world):
        d = plans[r].dest.long()
        for owner in range(world):
            mine = (d[:, 0] == owner).nonzero().flatten()
            assert torch.equal(dy_pads[owner][d[mine, 1]], dy[r][mine])
    for r in range(world):
        ranks[r].publish_output(dy_pads[r], False, plans[r].seq_b)
    for r in range(world):
        dx = ranks[r].pull(plans[r], True, False, plans[r].seq_b)
        want = dy[r].view(T, K, H).float().sum(1)
        torch.testing.assert_close(dx.float(), want, rtol=1e-2, atol=1e-2)
    # a second forward round with another routing: table entries of the first round must not leak into it
    from lm_engine_b200.ops.moe import GroupLayout

    sel2 = [torch.randint(0, E, (T, K), device="cuda", generator=g) for _ in range(world)]
    lay2 = [GroupLayout.from_selection(sel2[r], E) for r in range(world)]
    seq2 = [ranks[r].publish_counts(lay2[r]) for r in range(world)]
    plan2 = [ranks[r].make_plan(sel2[r], lay2[r], seq2[r]) for r in range(world)]
    for r in range(world):
        ranks[r].offer(x[r], plan2[r], True, seq2[r])
    for r in range(world):
        pad2 = ranks[r].land(plan2[r], True, seq2[r])
        own = plan2[r].owner_layout
        for le, (k0, kb) in enumerate(zip(own.k0.tolist(), own.kb.tolist())):
            e = r * Le + le
            want = torch.cat([x[s][(sel2[s] == e).flatten().nonzero().flatten() // K] for s in range(world)])
            assert torch.equal(pad2[k0:k0 + want.size(0)], want)
            assert float(pad2[k0 + want.size(0):k0 + 64 * kb].float().abs().sum()) == 0.0
    torch.cuda.synchronize()
    assert _lib.read_status(clear=True)[0] == 0


def test_exchange_overflow_is_reported_not_written():
    """A slab too small for the routed rows: the status word reports it, rows past the capacity are dropped (their
    destination is -1), nothing is written outside the slab."""
    from lm_engine_b200.ops import _lib

    _lib.read_status(clear=True)
    world, E, K, T, H = 2, 4, 2, 400, 64
    cap = 512                                                   # 1600 assignments over 2 owners cannot fit
    ranks, sel, x, plans, seqs = _setup(world, E, K, T, H, cap)
    guard = [ranks[r].tensors["y_out"][r] for r in range(world)]      # never written in this test
    for r in range(world):
        ranks[r].offer(x[r], plans[r], True, seqs[r])
    pads = [ranks[r].land(plans[r], True, seqs[r]) for r in range(world)]
    torch.cuda.synchronize()
    status = _lib.read_status(clear=True)
    assert status[0] == 3, status                               # bounds
    for r in range(world):
        d = plans[r].dest
        assert int(d[:, 1].max()) < cap and int((d[:, 1] < 0).sum()) > 0
        own = plans[r].owner_layout
        assert int((own.k0 + 64 * own.kb).max()) <= cap
        assert float(guard[r].float().abs().sum()) == 0.0
        assert pads[r].shape == (cap, H)


def test_moe_layer_on_emulated_exchange_matches_local_experts():
    """The whole forward / backward of the expert-parallel path (dispatch, grouped GEMMs, collect, combine) for one
    rank of a 1-rank group against the path without expert parallelism: same kernels around a different row layout."""
    from lm_engine_b200.models import config_from_dict, dense_config
    from lm_engine_b200.models.layers.moe import MoE
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.moe import GroupLayout, combine_tokens
    from lm_engine_b200.parallel import expert_exchange as xx
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
    x = torch.randn(384, 256, device="cuda").to(torch.bfloat16)
    T, K, E = 384, 2, 8
    rk = xx.RankBuffers.emulated(1, E, xx.capacity_rows(T * K, E, 1), 256, T, K, "cuda")[0]

    def run(exchange):
        moe.zero_grad()
        xi = x.clone().requires_grad_(True)
        logits, w, sel = moe._route(xi)
        if exchange:
            layout = GroupLayout.from_selection(sel, E)
            plan = rk.make_plan(sel.contiguous(), layout, rk.publish_counts(layout))
            y_pad = moe._grouped_mlp_padded(xx._Dispatch.apply(xi, rk, plan), plan.owner_layout)
            y = combine_tokens(xx._Collect.apply(y_pad, rk, plan), w, rk.identity_layout(T, K))
        else:
            y, _ = moe._experts(xi, w, sel)
        y.float().pow(2).sum().backward()
        return y, xi.grad, moe.c_fc.weight.grad.clone(), moe.c_proj.weight.grad.clone(), moe.gate.weight.grad.clone()

    _lib.read_status(clear=True)
    a, b = run(True), run(False)
    for u, v in zip(a, b):
        assert float((u.float() - v.float()).norm() / (v.float().norm() + 1e-6)) < 2e-2
    torch.cuda.synchronize()
    assert _lib.read_status(clear=True)[0] == 0
