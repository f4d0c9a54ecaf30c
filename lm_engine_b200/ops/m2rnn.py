"""Matrix-state RNN scan on CUDA (csrc/kernels/m2rnn.cu); the PyTorch statement of the same recurrence is
:func:`lm_engine_b200.ops.recurrence.m2rnn_scan`.

Role of ``xma.layers.m2rnn`` in the reference (lm_engine/modeling_utils/sequence_mixer_blocks/m2rnn/module.py:56-67).
Training memory is bounded by segments: the forward pass keeps one fp32 state snapshot per segment, the backward
pass replays a segment at a time into two bf16 record buffers of at most ``RECORD_BYTES`` each.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

RECORD_BYTES = 256 << 20     # per record buffer (h_{t-1} and z_t / da_t of one segment)
_TC = 8                      # steps per staged chunk in the kernels; segments are multiples of it


class _Args(ctypes.Structure):
    _fields_ = ([(n, c_void_p) for n in ("q", "k", "v", "f", "W")]
                + [(n, c_longlong) for n in ("q_b", "q_t", "k_b", "k_t", "v_b", "v_t")]
                + [(n, c_int) for n in ("B", "S", "N", "K", "V", "Nq", "Nk", "Nv", "Nf", "Nw")]
                + [(n, c_void_p) for n in ("h0", "h_out", "y_part", "ckpt")]
                + [(n, c_int) for n in ("seg_len", "t0", "T", "Tcap")]
                + [(n, c_void_p) for n in ("hprev", "z", "dy", "dh", "dq", "dk", "dv_part", "df_part")]
                + [("clip", c_float), ("dW_part", c_void_p)])


def m2rnn_kernel_eligible(q, k, v, f, W) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.size(-1) % 16 == 0 and v.size(-1) in (16, 32, 64) and W.size(-1) == v.size(-1))


def _head_major(t: torch.Tensor) -> torch.Tensor:
    """[B, S, n, D] view usable by the kernel (heads contiguous, 16-byte aligned strides) or a contiguous copy."""
    D = t.size(-1)
    ok = (t.stride(3) == 1 and t.stride(2) == D and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def segment_length(B: int, N: int, K: int, V: int, S: int) -> int:
    per_step = B * N * K * V * 2
    steps = max(_TC, (RECORD_BYTES // per_step) // _TC * _TC)
    return min(steps, (S + _TC - 1) // _TC * _TC)


def _launch(a: _Args, mode: int, what: str) -> None:
    from . import _lib

    _lib.check(_lib.cuda_lib().lme_m2rnn(ctypes.byref(a), mode, _lib.stream_ptr()), what)
    _lib.count_launch()


def _fill(a: _Args, q, k, v, f, W, N: int) -> None:
    B, S, Nq, K = q.shape
    a.q, a.k, a.v, a.f, a.W = q.data_ptr(), k.data_ptr(), v.data_ptr(), f.data_ptr(), W.data_ptr()
    a.q_b, a.q_t, a.k_b, a.k_t, a.v_b, a.v_t = (q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0),
                                                v.stride(1))
    a.B, a.S, a.N, a.K, a.V = B, S, N, K, v.size(-1)
    a.Nq, a.Nk, a.Nv, a.Nf, a.Nw = Nq, k.size(2), v.size(2), f.size(2), W.size(0)


class _M2RNN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, f, W, h0, clip):
        q, k, v = _head_major(q), _head_major(k), _head_major(v)
        f32 = f.float().contiguous()
        Wb = W.to(torch.bfloat16).contiguous()
        B, S, _, K = q.shape
        V = v.size(-1)
        N = max(q.size(2), k.size(2), v.size(2), f.size(2), W.size(0))
        RB = K // 16
        dev = q.device
        needs_grad = any(ctx.needs_input_grad)
        seg = segment_length(B, N, K, V, S)
        nseg = (S + seg - 1) // seg
        h0f = h0.float().contiguous() if h0 is not None else None
        y_part = torch.empty((RB, B, S, N, V), dtype=torch.float32, device=dev)
        h_out = torch.empty((B, N, K, V), dtype=torch.float32, device=dev)
        ckpt = torch.empty((B, N, nseg, K, V), dtype=torch.float32, device=dev) if needs_grad else None
        a = _Args()
        _fill(a, q, k, v, f32, Wb, N)
        a.h0 = h0f.data_ptr() if h0f is not None else None
        a.h_out, a.y_part = h_out.data_ptr(), y_part.data_ptr()
        a.ckpt = ckpt.data_ptr() if ckpt is not None else None
        a.seg_len, a.t0, a.T, a.Tcap = seg, 0, S, seg
        _launch(a, 0, f"lme_m2rnn forward B={B} S={S} N={N} K={K} V={V}")
        y = (y_part[0] if RB == 1 else y_part.sum(0)).to(q.dtype)
        if needs_grad:
            ctx.save_for_backward(q, k, v, f32, Wb, ckpt)
            ctx.meta = (N, seg, clip, h0 is not None, f.dtype, W.dtype, h0.dtype if h0 is not None else None)
        return y, h_out.to(q.dtype)

    @staticmethod
    def backward(ctx, dy, dh_out):
        from .gemm import _bmm_kernel

        q, k, v, f32, Wb, ckpt = ctx.saved_tensors
        N, seg, clip, has_h0, f_dtype, W_dtype, h0_dtype = ctx.meta
        B, S, Nq, K = q.shape
        V = v.size(-1)
        RB = K // 16
        dev = q.device
        dy = dy.to(torch.bfloat16).contiguous()
        dh = (dh_out.float().contiguous().clone() if dh_out is not None
              else torch.zeros((B, N, K, V), dtype=torch.float32, device=dev))
        dq = torch.empty((B, S, N, K), dtype=torch.float32, device=dev)
        dk = torch.empty_like(dq)
        dv_part = torch.empty((RB, B, S, N, V), dtype=torch.float32, device=dev)
        df_part = torch.empty((RB, B, S, N), dtype=torch.float32, device=dev)
        hprev = torch.empty((B, N, seg, K, V), dtype=torch.bfloat16, device=dev)
        z = torch.empty_like(hprev)
        in_kernel_dw = V <= 32      # the backward kernel accumulates dW itself; V = 64 leaves it to a batched GEMM
        dW = torch.zeros((N, V, V), dtype=torch.float32, device=dev)
        dW_part = torch.zeros((B, N, RB, V, V), dtype=torch.float32, device=dev) if in_kernel_dw else None
        a = _Args()
        _fill(a, q, k, v, f32, Wb, N)
        a.ckpt, a.seg_len, a.Tcap = ckpt.data_ptr(), seg, seg
        a.hprev, a.z, a.dy, a.dh = hprev.data_ptr(), z.data_ptr(), dy.data_ptr(), dh.data_ptr()
        a.dq, a.dk, a.dv_part, a.df_part = dq.data_ptr(), dk.data_ptr(), dv_part.data_ptr(), df_part.data_ptr()
        a.clip = float(clip) if clip is not None else 0.0
        a.dW_part = dW_part.data_ptr() if in_kernel_dw else None
        for s in reversed(range((S + seg - 1) // seg)):
            a.t0, a.T = s * seg, min(seg, S - s * seg)
            _launch(a, 1, f"lme_m2rnn replay t0={a.t0} T={a.T}")
            _launch(a, 2, f"lme_m2rnn backward t0={a.t0} T={a.T}")
            if not in_kernel_dw:
                hp = hprev[:, :, :a.T].reshape(B * N, a.T * K, V)
                da = z[:, :, :a.T].reshape(B * N, a.T * K, V)
                # h^T da over the segment's steps and state rows: both read as MN-major operands where they are
                dW += _bmm_kernel(hp, da, True, True, torch.float32).view(B, N, V, V).sum(0)
        if in_kernel_dw:
            dW = dW_part.sum((0, 2))

        def fold(t: torch.Tensor, heads: int, dtype) -> torch.Tensor:      # [B, S, N, ...] -> [B, S, heads, ...]
            if heads != N:
                t = t.view(B, S, heads, N // heads, *t.shape[3:]).sum(3)
            return t.to(dtype)

        dv = dv_part[0] if RB == 1 else dv_part.sum(0)
        df = df_part[0] if RB == 1 else df_part.sum(0)
        Nw = Wb.size(0)
        dWg = dW if Nw == N else dW.view(Nw, N // Nw, V, V).sum(1)
        return (fold(dq, Nq, q.dtype), fold(dk, k.size(2), k.dtype), fold(dv, v.size(2), v.dtype),
                fold(df, f32.size(2), f_dtype), dWg.to(W_dtype), dh.to(h0_dtype) if has_h0 else None, None)


def m2rnn_cuda(q, k, v, f, W, h0=None, gradient_clipping=None):
    """Same contract as :func:`lm_engine_b200.ops.recurrence.m2rnn_scan`: ``(y [B, S, N, V], h_S [B, N, K, V])``."""
    return _M2RNN.apply(q, k, v, f, W, h0, gradient_clipping)
