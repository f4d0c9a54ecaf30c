"""Sequential per-head recurrences of the RNN-family mixers (PyTorch statements; the oracle of the CUDA kernels).

Heads are broadcast between operands with differing head counts (each operand's heads are repeated up to the
largest count), states are carried across calls for generation, and ``gradient_clipping`` clamps the gradient that
flows back through the state at every step - the semantics of lm_engine/modeling_utils/sequence_mixer_blocks/
{rnn/op.py, gru/module.py:261-357, m2rnn/op.py, linear_attention/op.py}.
"""

from __future__ import annotations

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
