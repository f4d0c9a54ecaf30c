"""tcgen05 flash-attention forward against the fp32 PyTorch statement: output and log-sum-exp, causal and full,
grouped K/V heads, operands that are strided slices of one projection output."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [
    (1, 128, 1, 1, False),
    (1, 128, 1, 1, True),
    (2, 256, 4, 2, True),
    (1, 512, 8, 8, False),
    (2, 640, 6, 2, True),
])
@pytest.mark.parametrize("fused_qkv", [False, True])
def test_attention_forward_matches_reference(B, S, Hq, Hkv, causal, fused_qkv):
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention_reference
    from lm_engine_b200.ops.attention_cuda import flash_attention_forward

    torch.manual_seed(0)
    D = 128
    if fused_qkv:
        qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q, k, v = (t.view(B, S, -1, D) for t in qkv.split((Hq * D, Hkv * D, Hkv * D), dim=-1))
    else:
        q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
    scale = D ** -0.5
    out, lse = flash_attention_forward(q, k, v, causal=causal, softmax_scale=scale, return_lse=True)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), causal=causal, softmax_scale=scale,
                                       return_lse=True)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, ref_lse.transpose(1, 2), rtol=1e-3, atol=1e-3)    # ours is [B, Hq, Sq]


@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [
    (1, 128, 1, 1, True),
    (1, 256, 2, 2, False),
    (2, 384, 4, 2, True),
    (1, 640, 8, 2, True),
])
def test_attention_backward_matches_reference(B, S, Hq, Hkv, causal):
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention_reference
    from lm_engine_b200.ops.attention_cuda import _FlashAttention

    torch.manual_seed(1)
    D = 128
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    ref_in = qkv.detach().float().requires_grad_(True)

    def split(t):
        return [x.view(B, S, -1, D) for x in t.split((Hq * D, Hkv * D, Hkv * D), dim=-1)]

    scale = D ** -0.5
    out = _FlashAttention.apply(*split(qkv), causal, scale)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    ref = attention_reference(*split(ref_in), causal=causal, softmax_scale=scale)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    g, r = qkv.grad.float(), ref_in.grad
    for name, a, b in zip("qkv", split(g), split(r)):
        err = float((a - b).norm() / (b.norm() + 1e-6))
        assert err < 2e-2, (name, err)


@pytest.mark.parametrize("B,S,Hq,Hkv,window", [(1, 256, 2, 1, 64), (2, 640, 4, 2, 200), (1, 512, 2, 2, 129),
                                                  (1, 384, 2, 2, 1000)])
def test_sliding_window_matches_reference(B, S, Hq, Hkv, window):
    """Causal sliding-window attention takes the kernels without the switch (forward and every gradient)."""
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention, attention_reference

    torch.manual_seed(2)
    D = 128
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    ref_in = qkv.detach().float().requires_grad_(True)

    def split(t):
        return [x.view(B, S, -1, D) for x in t.split((Hq * D, Hkv * D, Hkv * D), dim=-1)]

    launches = _lib.launch_count
    out = attention(*split(qkv), causal=True, sliding_window=window)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    assert _lib.launch_count >= launches + 4              # forward + delta + dQ + dK/dV: the kernels ran
    ref = attention_reference(*split(ref_in), causal=True, sliding_window=window)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for name, a, b in zip("qkv", split(qkv.grad.float()), split(ref_in.grad)):
        err = float((a - b).norm() / (b.norm() + 1e-6))
        assert err < 2e-2, (name, err)


@pytest.mark.parametrize("window", [None, 48])
@pytest.mark.parametrize("own,D", [(False, 64), (True, 128)])
def test_packed_sequences_on_gpu_match_reference(window, own, D, monkeypatch):
    """cu_seqlens attention on the GPU - the library varlen kernel by default, the tcgen05 kernels under the switch -
    against the per-sequence PyTorch statement."""
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention, attention_reference

    if own:
        monkeypatch.setenv("LME_ATTENTION", "own")
    else:
        monkeypatch.delenv("LME_ATTENTION", raising=False)
    torch.manual_seed(4)
    Hq, Hkv = 4, 2
    launches = _lib.launch_count
    lens = [37, 128, 5, 200]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    T = sum(lens)
    q = torch.randn(T, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(T, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(T, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    out = attention(q, k, v, causal=True, sliding_window=window, cu_seqlens=cu, max_seqlen=max(lens))
    dout = torch.randn_like(out)
    out.backward(dout)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = attention_reference(*ref_in, causal=True, sliding_window=window, cu_seqlens=cu)
    ref.backward(dout.float())
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    assert (_lib.launch_count >= launches + 4) == own
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for a, b in zip((q, k, v), ref_in):
        assert float((a.grad.float() - b.grad).norm() / (b.grad.norm() + 1e-6)) < 2e-2


def test_sliding_window_with_other_head_dims_uses_the_library_kernel():
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention, attention_reference

    torch.manual_seed(6)
    q = torch.randn(2, 200, 4, 64, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(2, 200, 2, 64, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(2, 200, 2, 64, device="cuda").to(torch.bfloat16).requires_grad_(True)
    launches = _lib.launch_count
    out = attention(q, k, v, causal=True, sliding_window=50)
    assert _lib.launch_count == launches                    # head dim 64: not our kernels
    dout = torch.randn_like(out)
    out.backward(dout)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = attention_reference(*ref_in, causal=True, sliding_window=50)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for a, b in zip((q, k, v), ref_in):
        assert float((a.grad.float() - b.grad).norm() / (b.grad.norm() + 1e-6)) < 2e-2


def test_dispatcher_follows_the_switch(monkeypatch):
    from lm_engine_b200.ops import attention_cuda
    from lm_engine_b200.ops.attention import attention

    q = torch.randn(1, 256, 2, 128, device="cuda").to(torch.bfloat16)
    calls = []
    real = attention_cuda.flash_attention_forward
    monkeypatch.setattr(attention_cuda, "flash_attention_forward", lambda *a, **k: calls.append(1) or real(*a, **k))
    monkeypatch.delenv("LME_ATTENTION", raising=False)
    a = attention(q, q, q, causal=True)
    assert calls == []                         # default: the library kernel
    monkeypatch.setenv("LME_ATTENTION", "own")
    qg = q.clone().requires_grad_(True)
    b = attention(qg, qg, qg, causal=True)
    assert calls == [1]
    b.sum().backward()
    assert qg.grad is not None and torch.isfinite(qg.grad.float()).all()
    torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("method", [None, "headtail"])
def test_ring_attention_blocks_on_kernels_match_block_math(method):
    """The per-block forward / backward of context-parallel ring attention on the attention kernels against the
    PyTorch block statements, for every (query rank, key rank) pair of a 2-way split (no process group needed)."""
    from lm_engine_b200.ops.attention import attention_reference
    from lm_engine_b200.parallel import ring_attention as ra
    from lm_engine_b200.parallel.context_parallel import shard_indices

    torch.manual_seed(5)
    B, S, Hq, Hkv, D, cp = 1, 1024, 4, 2, 128, 2
    scale = D ** -0.5
    q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
    do = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    out_full, lse_full = attention_reference(q.float(), k.float(), v.float(), causal=True, softmax_scale=scale,
                                             return_lse=True)                       # [B,S,Hq,D], [B,S,Hq]
    pos = [shard_indices(S, cp, j, method, device="cuda") for j in range(cp)]
    runs = [ra.shard_runs(S, cp, j, method) for j in range(cp)]
    for j in range(cp):
        assert torch.equal(torch.cat([torch.arange(a, a + n, device="cuda") for a, n in runs[j]]), pos[j])
    for r in range(cp):
        for src in range(cp):
            qs, ks, vs = q[:, pos[r]], k[:, pos[src]], v[:, pos[src]]
            assert ra.kernel_blocks_usable(qs, ks, runs[r], runs[src], True, None)
            if not ra._block_needed(pos[r], pos[src], True, None):
                assert all(ra._relation(a, b, True) == "skip" for a in runs[r] for b in runs[src])
                continue
            o_k, l_k = ra.kernel_block_forward(qs, ks, vs, runs[r], runs[src], scale, True)
            o_r, l_r = ra.block_attention_forward(qs, ks, vs, pos[r], pos[src], scale, True, None)
            seen = ~torch.isinf(l_r)
            assert torch.equal(seen, ~torch.isinf(l_k))
            torch.testing.assert_close(l_k[seen], l_r[seen], rtol=1e-3, atol=1e-3)
            torch.testing.assert_close(o_k[seen], o_r[seen], rtol=2e-2, atol=2e-2)
            args = (do[:, pos[r]], qs, ks, vs, out_full[:, pos[r]], lse_full[:, pos[r]])
            g_k = ra.kernel_block_backward(*args, runs[r], runs[src], scale, True)
            g_r = ra.block_attention_backward(*args, pos[r], pos[src], scale, True, None)
            for a, b in zip(g_k, g_r):
                assert float((a - b).norm() / (b.norm() + 1e-6)) < 2e-2


def test_forward_waits_for_chunk_readiness_words():
    """Keys / values that "arrive" in chunks: with every chunk's word already at the sequence number the kernel gives
    the plain result; the words are only read (no other launch is waited for)."""
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention import attention_reference
    from lm_engine_b200.ops.attention_cuda import flash_attention_forward

    g = torch.Generator(device="cuda").manual_seed(4)
    B, Sq, Skv, Hq, Hkv = 1, 256, 768, 4, 2
    q = torch.randn(B, Sq, Hq, 128, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).to(torch.bfloat16)
    ready = torch.full((B, 3), 7, dtype=torch.int32, device="cuda")       # 3 chunks of 256 rows, all announced
    out, lse = flash_attention_forward(q, k, v, causal=True, softmax_scale=128 ** -0.5, return_lse=True,
                                       kv_ready=ready[0], kv_chunk_rows=256, kv_seq=7)
    ref, ref_lse = attention_reference(q, k, v, causal=True, softmax_scale=128 ** -0.5, return_lse=True)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    assert float((out.float() - ref.float()).norm() / ref.float().norm()) < 1e-2
    assert torch.allclose(lse, ref_lse.transpose(1, 2), atol=2e-2, rtol=1e-3)


def _fp32_attention_by_head_groups(q, k, v, causal, scale, do=None):
    """fp32 oracle at large shapes: one K/V head (and its query heads) at a time so that the score matrices fit."""
    B, S, Hq, D = q.shape
    Hkv = k.size(2)
    G = Hq // Hkv
    outs, grads = [], []
    for h in range(Hkv):
        qh = q[:, :, h * G:(h + 1) * G].float().requires_grad_(do is not None)
        kh = k[:, :, h:h + 1].float().requires_grad_(do is not None)
        vh = v[:, :, h:h + 1].float().requires_grad_(do is not None)
        from lm_engine_b200.ops.attention import attention_reference

        o = attention_reference(qh, kh, vh, causal=causal, softmax_scale=scale)
        if do is not None:
            o.backward(do[:, :, h * G:(h + 1) * G].float())
            grads.append((qh.grad, kh.grad, vh.grad))
        outs.append(o.detach())
    out = torch.cat(outs, dim=2)
    if do is None:
        return out, None
    return out, tuple(torch.cat([g[i] for g in grads], dim=2) for i in range(3))


@pytest.mark.parametrize("B,S,Hq,Hkv", [(2, 4096, 32, 8), (1, 16384, 8, 2)])
def test_attention_at_training_shapes(B, S, Hq, Hkv):
    """The Llama-3-8B attention shape (more query blocks than one wave of CTAs, so the longest-first block order and
    the second wave are exercised) and a 16k sequence, forward and backward against the fp32 statement."""
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.attention_cuda import _FlashAttention

    g = torch.Generator(device="cuda").manual_seed(11)
    D, scale = 128, 128 ** -0.5
    q, k, v = (torch.randn(B, S, h, D, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
               for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    out = _FlashAttention.apply(q, k, v, True, scale)
    out.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    ref, (dq, dk, dv) = _fp32_attention_by_head_groups(q.detach(), k.detach(), v.detach(), True, scale, do)

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-9))

    assert rel(out, ref) < 1e-2
    assert rel(q.grad, dq) < 2e-2 and rel(k.grad, dk) < 2e-2 and rel(v.grad, dv) < 2e-2


def test_attention_kernels_are_deterministic():
    """No atomics anywhere: two runs on the same inputs give the same bits, forward and backward."""
    from lm_engine_b200.ops.attention_cuda import _FlashAttention

    g = torch.Generator(device="cuda").manual_seed(12)
    q, k, v = (torch.randn(2, 1024, h, 128, device="cuda", generator=g).to(torch.bfloat16) for h in (8, 2, 2))
    do = torch.randn(2, 1024, 8, 128, device="cuda", generator=g).to(torch.bfloat16)
    runs = []
    for _ in range(2):
        a, b, c = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = _FlashAttention.apply(a, b, c, True, 128 ** -0.5)
        out.backward(do)
        runs.append((out.detach(), a.grad, b.grad, c.grad))
    for x, y in zip(*runs):
        assert torch.equal(x, y)
