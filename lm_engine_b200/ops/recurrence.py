"""Sequential per-head recurrences of the RNN-family mixers (PyTorch statements; the oracle of the CUDA kernels).

Heads are broadcast between operands with differing head counts (each operand's heads are repeated up to the
largest count), states are carried across calls for generation, and ``gradient_clipping`` clamps the gradient that
flows back through the state at every step - the semantics of lm_engine/modeling_utils/sequence_mixer_blocks/
{rnn/op.py, gru/module.py:261-357, m2rnn/op.py, linear_attention/op.py}.
"""

from __future__ import annotations

import os

import torch

from ..models.layers.activations import clip_gradients, sigmoid, tanh


def _rep(t: torch.Tensor, n: int, dim: int) -> torch.Tensor:
    have = t.size(dim)
    assert n % have == 0
    return t if have == n else t.repeat_interleave(n // have, dim=dim)


def rnn_scan(x, W, h0=None, gradient_clipping=None):
    """``h_t = tanh(h_{t-1} W + x_t)``.  x ``[B, S, Nx, H]``, W ``[Nw, H, H]`` -> ``(y [B, S, N, H], h_S)``."""
    B, S, _, H = x.shape
    N = max(x.size(2), W.size(0))
    x, W = _rep(x, N, 2), _rep(W, N, 0)
    h = torch.zeros(B, N, H, dtype=x.dtype, device=x.device) if h0 is None else h0
    ys = []
    for s in range(S):
        h = tanh(torch.einsum("bnh,nhk->bnk", h, W) + x[:, s])
        h = clip_gradients(h, gradient_clipping)
        ys.append(h)
    return torch.stack(ys, dim=1), h


def gru_scan(x, xf, xr, W, Wf, Wr, h0=None, gradient_clipping=None):
    """``f = sigmoid(h Wf + xf)``, ``r = sigmoid(h Wr + xr)``, ``z = tanh((h * r) W + x)``, ``h = f h + (1 - f) z``."""
    B, S, _, H = x.shape
    N = max(t.size(2) for t in (x, xf, xr)) if True else 0
    N = max(N, W.size(0), Wf.size(0), Wr.size(0))
    x, xf, xr = _rep(x, N, 2), _rep(xf, N, 2), _rep(xr, N, 2)
    W, Wf, Wr = _rep(W, N, 0), _rep(Wf, N, 0), _rep(Wr, N, 0)
    h = torch.zeros(B, N, H, dtype=x.dtype, device=x.device) if h0 is None else h0
    ys = []
    for s in range(S):
        f = sigmoid(torch.einsum("bnh,nhk->bnk", h, Wf) + xf[:, s])
        r = sigmoid(torch.einsum("bnh,nhk->bnk", h, Wr) + xr[:, s])
        z = tanh(torch.einsum("bnh,nhk->bnk", h * r, W) + x[:, s])
        h = f * h + (1 - f) * z
        h = clip_gradients(h, gradient_clipping)
        ys.append(h)
    return torch.stack(ys, dim=1), h


def m2rnn_scan(q, k, v, f, W, h0=None, gradient_clipping=None):
    """Matrix-state RNN: ``z = tanh(h W + k (x) v)``, ``h = f h + (1 - f) z``, ``y = q . h``.
    q/k ``[B, S, N*, K]``, v ``[B, S, Nv, V]``, f ``[B, S, Nf]`` in (0, 1), W ``[Nw, V, V]``, h ``[B, N, K, V]``."""
    B, S, _, K = q.shape
    V = v.size(-1)
    N = max(q.size(2), k.size(2), v.size(2), W.size(0), f.size(-1))
    q, k, v, W, f = _rep(q, N, 2), _rep(k, N, 2), _rep(v, N, 2), _rep(W, N, 0), _rep(f, N, 2)
    h = torch.zeros(B, N, K, V, dtype=k.dtype, device=k.device) if h0 is None else h0
    ys = []
    for s in range(S):
        z = tanh(torch.einsum("bnkv,nvw->bnkw", h, W) + k[:, s, :, :, None] * v[:, s, :, None, :])
        g = f[:, s, :, None, None]
        h = g * h + (1 - g) * z
        h = clip_gradients(h, gradient_clipping)
        ys.append(torch.einsum("bnk,bnkv->bnv", q[:, s], h))
    return torch.stack(ys, dim=1), h


CHUNK = 64   # time steps per block of the chunk-parallel forms below
LONG_CHUNK = 256


def linear_attention_chunked(q, k, v, h0=None, attention_multiplier: float = 1.0, chunk: int = CHUNK):
    """Chunk-parallel form of :func:`linear_attention_scan`: inside a block ``Y = strict_tril(Q K^T) V + Q H``; the
    state entering each block is an exclusive prefix sum of the blocks' ``K^T V`` - batched matmuls instead of one
    tiny step per token."""
    B, S, _, K = q.shape
    V = v.size(-1)
    N = max(q.size(2), k.size(2), v.size(2))
    q, k, v = _rep(q, N, 2), _rep(k, N, 2), _rep(v, N, 2)
    pad = (chunk - S % chunk) % chunk
    if pad:
        q, k, v = (torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
    nc = (S + pad) // chunk
    qc = q.view(B, nc, chunk, N, K).permute(0, 3, 1, 2, 4).float()      # [B, N, nc, L, K]
    kc = k.view(B, nc, chunk, N, K).permute(0, 3, 1, 2, 4).float()
    vc = v.view(B, nc, chunk, N, V).permute(0, 3, 1, 2, 4).float()
    kv = kc.transpose(-1, -2) @ vc                                       # [B, N, nc, K, V]
    h_in = torch.cumsum(kv, dim=2) - kv                                  # state before each block (without h0)
    if h0 is not None:
        h_in = h_in + h0.float()[:, :, None]
    mask = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(-1)
    att = (qc @ kc.transpose(-1, -2)).masked_fill(~mask, 0.0)
    y = att @ vc + qc @ h_in
    y = y.permute(0, 2, 3, 1, 4).reshape(B, nc * chunk, N, V)[:, :S]
    h = h_in[:, :, -1] + kv[:, :, -1]
    return (y * attention_multiplier).to(q.dtype), h


def gated_delta_rule_chunked(q, k, v, g, beta, scale=None, h0=None, use_qk_l2norm: bool = True, chunk: int = CHUNK):
    """Chunk-parallel gated delta rule (same recurrence as :func:`gated_delta_rule_scan`).  With ``G`` the cumulative
    log-decay inside a block and ``S0`` the state entering it, the per-step corrections ``u_t`` solve the unit lower
    triangular system ``(I + strict_tril(beta_t e^{G_t - G_i} k_t.k_i)) U = beta (V - e^{G} K S0)``, so
    ``U = W_v - W_k S0`` with ``W_v, W_k`` computed for all blocks at once; then
    ``Y = e^{G} Q S0 + tril(e^{G_t - G_i} q_t.k_i) U`` and ``S_end = e^{G_L} S0 + (e^{G_L - G} K)^T U``.
    Only the short loop over blocks is sequential."""
    B, S, N, K = q.shape
    V = v.size(-1)
    dtype = v.dtype
    qf, kf, vf = q.float(), k.float(), v.float()
    if use_qk_l2norm:
        qf = qf / (qf.norm(dim=-1, keepdim=True) + 1e-6)
        kf = kf / (kf.norm(dim=-1, keepdim=True) + 1e-6)
    qf = qf * (K**-0.5 if scale is None else scale)
    gf, bf = g.float(), beta.float()
    pad = (chunk - S % chunk) % chunk
    if pad:   # padded steps: no decay (g = 0), no write (beta = 0)
        qf, kf, vf = (torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad)) for t in (qf, kf, vf))
        gf, bf = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (gf, bf))
    nc, L = (S + pad) // chunk, chunk

    def blocks(t):   # [B, S, N, X] -> [B, N, nc, L, X]
        return t.view(B, nc, L, N, -1).permute(0, 3, 1, 2, 4)

    qc, kc, vc = blocks(qf), blocks(kf), blocks(vf)
    G = torch.cumsum(gf.view(B, nc, L, N).permute(0, 3, 1, 2), dim=-1)    # [B, N, nc, L]
    bc = bf.view(B, nc, L, N).permute(0, 3, 1, 2)
    diff = G[..., :, None] - G[..., None, :]                               # G_t - G_i
    strict = torch.ones(L, L, dtype=torch.bool, device=q.device).tril(-1)
    incl = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
    decay_strict = torch.exp(diff.masked_fill(~strict, float("-inf")))
    decay_incl = torch.exp(diff.masked_fill(~incl, float("-inf")))
    T = torch.eye(L, device=q.device) + bc[..., :, None] * decay_strict * (kc @ kc.transpose(-1, -2))
    rhs = torch.cat((bc[..., None] * vc, (bc * torch.exp(G))[..., None] * kc), dim=-1)
    # the inverse of the L x L unit-triangular factor once (a solve with L right-hand sides), then one product with
    # the V + K columns: the solve against all V + K columns costs ten times the product
    eye = torch.eye(L, device=q.device).expand_as(T)
    W = torch.linalg.solve_triangular(T, eye, upper=False, unitriangular=True) @ rhs
    Wv, Wk = W[..., :V], W[..., V:]                                        # [.., L, V], [.., L, K]
    qk = decay_incl * (qc @ kc.transpose(-1, -2))                          # [.., L(t), L(i)]
    qe = torch.exp(G)[..., None] * qc                                      # e^{G_t} q_t
    k_end = torch.exp(G[..., -1:, None] - G[..., None]) * kc               # e^{G_L - G_i} k_i
    a_end = torch.exp(G[..., -1])                                          # decay of a whole block
    h = torch.zeros(B, N, K, V, dtype=torch.float32, device=q.device) if h0 is None else h0.float()
    y, h = delta_chain(Wk, Wv, qe, qk, k_end, a_end, h)
    y = y.permute(0, 2, 3, 1, 4).reshape(B, nc * L, N, V)[:, :S]
    return y.to(dtype), h


def delta_chain_reference(Wk, Wv, qe, qk, ke, a, h):
    """The sequential part of the chunk-parallel delta rule, block by block: ``U = W_v - W_k h``,
    ``y = Q_e h + QK U``, ``h <- a h + K_e^T U``.  Operands ``[B, N, nc, L, *]``, ``a [B, N, nc]``, ``h [B, N, K, V]``."""
    ys = []
    for c in range(Wk.size(2)):
        U = Wv[:, :, c] - Wk[:, :, c] @ h
        ys.append(qe[:, :, c] @ h + qk[:, :, c] @ U)
        h = a[:, :, c, None, None] * h + ke[:, :, c].transpose(-1, -2) @ U
    return torch.stack(ys, dim=2), h


class _DeltaChain(torch.autograd.Function):
    """:func:`delta_chain_reference` as two kernels (csrc/kernels/delta_rule.cu): the forward chain keeps the state of
    64 columns in registers and leaves ``U`` and the state entering every block behind; the backward chain runs the
    state gradient in reverse and leaves ``dU`` and the gradient leaving every block; the operand gradients are
    batched tensor-core GEMMs over all blocks on those."""

    @staticmethod
    def forward(ctx, Wk, Wv, qe, qk, ke, a, h):
        from . import _lib

        B, N, nc, L, K = qe.shape
        V = Wv.size(-1)
        bf, dev = torch.bfloat16, qe.device
        wk_b = None if Wk is None else Wk.to(bf).contiguous()          # None: no correction term (linear attention)
        qe_b, ke_b, qk_b = qe.to(bf).contiguous(), ke.to(bf).contiguous(), qk.to(bf).contiguous()
        ket = ke_b.transpose(-1, -2).contiguous()
        wv, a32, h32 = Wv.float().contiguous(), a.float().contiguous(), h.float().contiguous()
        y = torch.empty((B, N, nc, L, V), dtype=torch.float32, device=dev)
        u_all = torch.empty((B, N, nc, L, V), dtype=bf, device=dev)
        h_all = torch.empty((B, N, nc, K, V), dtype=bf, device=dev)
        h_final = torch.empty((B, N, K, V), dtype=torch.float32, device=dev)
        _lib.check(_lib.cuda_lib().lme_delta_chain_fwd(
            _lib.ptr(wk_b), qe_b.data_ptr(), ket.data_ptr(), qk_b.data_ptr(), wv.data_ptr(), a32.data_ptr(),
            h32.data_ptr(), y.data_ptr(), u_all.data_ptr(), h_all.data_ptr(), h_final.data_ptr(), B * N, nc, K, V,
            _lib.stream_ptr()), f"lme_delta_chain_fwd BN={B * N} nc={nc} K={K} V={V}")
        _lib.count_launch()
        ctx.has_wk = wk_b is not None
        ctx.save_for_backward(*([wk_b] if ctx.has_wk else []), qe_b, ke_b, qk_b, a32, u_all, h_all)
        return y, h_final

    @staticmethod
    def backward(ctx, dy, dh_final):
        from . import _lib
        from .gemm import _bmm_kernel

        saved = list(ctx.saved_tensors)
        wk_b = saved.pop(0) if ctx.has_wk else None
        qe_b, ke_b, qk_b, a32, u_all, h_all = saved
        B, N, nc, L, K = qe_b.shape
        V = u_all.size(-1)
        bf, dev = torch.bfloat16, dy.device
        dy = dy.float().contiguous()
        qkt = qk_b.transpose(-1, -2).contiguous()
        qet = qe_b.transpose(-1, -2).contiguous()
        wkt = None if wk_b is None else wk_b.transpose(-1, -2).contiguous()
        du_all = torch.empty((B, N, nc, L, V), dtype=bf, device=dev)
        dh_all = torch.empty((B, N, nc, K, V), dtype=bf, device=dev)
        dh0 = torch.empty((B, N, K, V), dtype=torch.float32, device=dev)
        dhf = None if dh_final is None else dh_final.float().contiguous()
        _lib.check(_lib.cuda_lib().lme_delta_chain_bwd(
            qkt.data_ptr(), ke_b.data_ptr(), qet.data_ptr(), _lib.ptr(wkt), dy.data_ptr(), a32.data_ptr(),
            _lib.ptr(dhf), du_all.data_ptr(), dh_all.data_ptr(), dh0.data_ptr(), B * N, nc, K, V,
            _lib.stream_ptr()), f"lme_delta_chain_bwd BN={B * N} nc={nc} K={K} V={V}")
        _lib.count_launch()
        # operand gradients: products over the V columns, one batch entry per (batch, head, block)
        n = B * N * nc
        dyb = dy.to(bf).view(n, L, V)
        du, dh = du_all.view(n, L, V), dh_all.view(n, K, V)
        u, hs = u_all.view(n, L, V), h_all.view(n, K, V)
        f32 = torch.float32
        dWk = None if wk_b is None else -_bmm_kernel(du, hs, False, False, f32).view(B, N, nc, L, K)   # -dU h^T
        dqe = _bmm_kernel(dyb, hs, False, False, f32).view(B, N, nc, L, K)       # dy h^T
        dqk = _bmm_kernel(dyb, u, False, False, f32).view(B, N, nc, L, L)        # dy U^T
        dke = _bmm_kernel(u, dh, False, False, f32).view(B, N, nc, L, K)         # U dh^T
        da = (dh_all.float() * h_all.float()).sum((-1, -2))
        return dWk, du_all.float(), dqe, dqk, dke, da, dh0


def delta_chain_kernel_usable(Wk, Wv) -> bool:
    return (Wk.is_cuda and Wk.size(-2) == 64 and Wk.size(-1) in (128, 256) and Wv.size(-1) % 64 == 0
            and Wk.size(0) * Wk.size(1) <= 65535)


def delta_chain(Wk, Wv, qe, qk, ke, a, h):
    if delta_chain_kernel_usable(Wk, Wv):
        return _DeltaChain.apply(Wk, Wv, qe, qk, ke, a, h)
    return delta_chain_reference(Wk, Wv, qe, qk, ke, a, h)


def linear_attention_scan(q, k, v, h0=None, attention_multiplier: float = 1.0):
    """``y_t = q_t . h_{t-1}`` (state read before the update), ``h_t = h_{t-1} + k_t (x) v_t``; fp32 state."""
    B, S, _, K = q.shape
    V = v.size(-1)
    N = max(q.size(2), k.size(2), v.size(2))
    q, k, v = _rep(q, N, 2), _rep(k, N, 2), _rep(v, N, 2)
    h = torch.zeros(B, N, K, V, dtype=torch.float32, device=q.device) if h0 is None else h0.float()
    ys = []
    for s in range(S):
        ys.append(torch.einsum("bnk,bnkv->bnv", q[:, s], h.type_as(q)))
        h = h + k[:, s, :, :, None] * v[:, s, :, None, :]
    return torch.stack(ys, dim=1) * attention_multiplier, h


def gated_delta_rule_scan(q, k, v, g, beta, scale=None, h0=None, use_qk_l2norm: bool = True):
    """Gated delta rule (fp32): ``h = exp(g_t) h``; ``d = beta_t (v_t - h^T k_t)``; ``h = h + k_t (x) d``;
    ``y_t = h^T (scale q_t)``.  q/k ``[B, S, N, K]``, v ``[B, S, N, V]``, g/beta ``[B, S, N]``, h ``[B, N, K, V]``."""
    B, S, N, K = q.shape
    V = v.size(-1)
    dtype = v.dtype
    qf, kf, vf = q.float(), k.float(), v.float()
    if use_qk_l2norm:
        qf = qf / (qf.norm(dim=-1, keepdim=True) + 1e-6)
        kf = kf / (kf.norm(dim=-1, keepdim=True) + 1e-6)
    scale = K**-0.5 if scale is None else scale
    qf = qf * scale
    h = torch.zeros(B, N, K, V, dtype=torch.float32, device=q.device) if h0 is None else h0.float()
    ys = []
    for s in range(S):
        h = h * torch.exp(g[:, s].float())[..., None, None]
        mem = torch.einsum("bnkv,bnk->bnv", h, kf[:, s])
        d = (vf[:, s] - mem) * beta[:, s].float()[..., None]
        h = h + kf[:, s, :, :, None] * d[:, :, None, :]
        ys.append(torch.einsum("bnkv,bnk->bnv", h, qf[:, s]))
    return torch.stack(ys, dim=1).to(dtype), h


def linear_attention_on_chain(q, k, v, h0=None, attention_multiplier: float = 1.0, chain=None):
    """Linear attention as a special case of the delta-rule chain: with ``W_k = 0`` and ``a = 1`` the chain computes
    ``y = Q h + strict_tril(Q K^T) V`` and ``h <- h + K^T V`` per 64-step block, so the forward and backward chain
    kernels serve this mixer as well (key width zero-padded to 128 / 256, value width to a multiple of 64).  ``chain``
    replaces the kernels by another implementation of the same recurrences (the PyTorch block loop in CPU tests)."""
    B, S, _, K = q.shape
    V = v.size(-1)
    N = max(q.size(2), k.size(2), v.size(2))
    q, k, v = _rep(q, N, 2), _rep(k, N, 2), _rep(v, N, 2)
    L = CHUNK
    Kp = 128 if K <= 128 else 256
    Vp = (V + 63) // 64 * 64
    pad = (L - S % L) % L
    pad_fn = torch.nn.functional.pad
    qf = pad_fn(q.float(), (0, Kp - K, 0, 0, 0, pad))
    kf = pad_fn(k.float(), (0, Kp - K, 0, 0, 0, pad))
    vf = pad_fn(v.float(), (0, Vp - V, 0, 0, 0, pad))
    nc = (S + pad) // L

    def blocks(t):   # [B, S, N, X] -> [B, N, nc, L, X]
        return t.view(B, nc, L, N, -1).permute(0, 3, 1, 2, 4)

    qc, kc, vc = blocks(qf), blocks(kf), blocks(vf)
    strict = torch.ones(L, L, dtype=torch.bool, device=q.device).tril(-1)
    qk = (qc @ kc.transpose(-1, -2)).masked_fill(~strict, 0.0)
    h = torch.zeros(B, N, Kp, Vp, dtype=torch.float32, device=q.device)
    if h0 is not None:
        h = pad_fn(h0.float(), (0, Vp - V, 0, Kp - K))
    ones = torch.ones(B, N, nc, dtype=torch.float32, device=q.device)
    if chain is None:
        y, h = _DeltaChain.apply(None, vc, qc, qk, kc, ones, h)
    else:
        y, h = chain(torch.zeros_like(kc), vc, qc, qk, kc, ones, h)
    y = y.permute(0, 2, 3, 1, 4).reshape(B, nc * L, N, Vp)[:, :S, :, :V]
    return (y * attention_multiplier).to(q.dtype), h[:, :, :K, :V]


def linear_attention(q, k, v, h0=None, attention_multiplier: float = 1.0):
    """Token recurrence for short inputs (decode), else the chunk-parallel PyTorch form (the state entering a block
    is a prefix sum, so nothing is sequential).  ``LME_LINEAR_ATTENTION=chain`` selects the delta-rule chain kernels
    instead (key width up to 256): measured slower at the published layout (K = V = 64, 32 heads: 3.2 ms forward +
    backward against 2.2 ms), because the key width is padded to 128 and the operand preparation outweighs the chain."""
    if q.size(1) < 8:
        return linear_attention_scan(q, k, v, h0, attention_multiplier)
    if (q.is_cuda and os.environ.get("LME_LINEAR_ATTENTION", "") == "chain" and q.size(-1) <= 256
            and q.size(0) * max(q.size(2), k.size(2), v.size(2)) <= 65535):
        return linear_attention_on_chain(q, k, v, h0, attention_multiplier)
    return linear_attention_chunked(q, k, v, h0, attention_multiplier)


def gated_delta_rule(q, k, v, g, beta, scale=None, h0=None, use_qk_l2norm: bool = True):
    if q.size(1) < 8:
        return gated_delta_rule_scan(q, k, v, g, beta, scale, h0, use_qk_l2norm)
    if q.is_cuda and q.size(-1) in (128, 256) and v.size(-1) % 64 == 0:
        # the chain over 64-step blocks is one kernel each way
        return gated_delta_rule_chunked(q, k, v, g, beta, scale, h0, use_qk_l2norm, chunk=64)
    # the loop over blocks is the sequential (launch-bound) part and the block-local work is cheap: long sequences
    # take large blocks (the intra-block cost grows with the block length, the number of loop trips falls with it)
    chunk = LONG_CHUNK if q.size(1) >= 4 * LONG_CHUNK else CHUNK
    return gated_delta_rule_chunked(q, k, v, g, beta, scale, h0, use_qk_l2norm, chunk=chunk)


def m2rnn(q, k, v, f, W, h0=None, gradient_clipping=None):
    """Matrix-state RNN: the CUDA scan when the operands qualify, else :func:`m2rnn_scan`."""
    from .m2rnn import m2rnn_cuda, m2rnn_kernel_eligible

    if m2rnn_kernel_eligible(q, k, v, f, W):
        return m2rnn_cuda(q, k, v, f, W, h0, gradient_clipping)
    return m2rnn_scan(q, k, v, f, W, h0, gradient_clipping)


def rnn(x, W, h0=None, gradient_clipping=None):
    """Multi-head tanh RNN: the CUDA scan when the operands qualify, else :func:`rnn_scan`."""
    from .rnn import rnn_cuda, rnn_kernel_eligible

    if rnn_kernel_eligible(x):
        return rnn_cuda(x, W, h0, gradient_clipping)
    return rnn_scan(x, W, h0, gradient_clipping)


def gru(x, xf, xr, W, Wf, Wr, h0=None, gradient_clipping=None):
    """Multi-head GRU: the CUDA scan when the operands qualify, else :func:`gru_scan`."""
    from .rnn import gru_cuda, rnn_kernel_eligible

    if rnn_kernel_eligible(x, xf, xr, gru=True):
        return gru_cuda(x, xf, xr, W, Wf, Wr, h0, gradient_clipping)
    return gru_scan(x, xf, xr, W, Wf, Wr, h0, gradient_clipping)
