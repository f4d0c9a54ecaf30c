"""Vector-state RNN / GRU scans on CUDA (csrc/kernels/rnn.cu); the PyTorch statements of the same recurrences are
:func:`lm_engine_b200.ops.recurrence.rnn_scan` and :func:`gru_scan`.

Role of ``xma.layers.rnn`` / ``xma.layers.gru`` in the reference (lm_engine/modeling_utils/sequence_mixer_blocks/
rnn/module.py:189-197, gru/module.py:218-230).  Every state is an output, so nothing but the inputs and the output
is kept for the backward pass; the weight gradients are batched GEMMs over the sequence.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .m2rnn import _head_major


class _Args(ctypes.Structure):
    _fields_ = ([(n, c_void_p) for n in ("x", "xf", "xr", "W", "Wf", "Wr")]
                + [(n, c_longlong) for n in ("x_b", "x_t", "xf_b", "xf_t", "xr_b", "xr_t")]
                + [(n, c_int) for n in ("B", "S", "N", "H", "Nx", "Nxf", "Nxr", "Nw", "Nwf", "Nwr", "gru", "pad_")]
                + [(n, c_void_p) for n in ("h0", "y", "dy", "dh", "dx", "dxf", "dxr", "hr")]
                + [("clip", c_float)])


def rnn_kernel_eligible(x: torch.Tensor, *others: torch.Tensor, gru: bool = False) -> bool:
    H = x.size(-1)
    return (x.is_cuda and x.dtype == torch.bfloat16 and all(t.dtype == torch.bfloat16 for t in others if t.dim() == 4)
            and H in ((16, 32) if gru else (16, 32, 64)))


def _launch(a: _Args, mode: int, what: str) -> None:
    from . import _lib

    _lib.check(_lib.cuda_lib().lme_rnn(ctypes.byref(a), mode, _lib.stream_ptr()), what)
    _lib.count_launch()


def _weight_grad(left: torch.Tensor, right: torch.Tensor, heads: int) -> torch.Tensor:
    """``sum_{b,s} left[b,s,n,:]^T right[b,s,n,:]`` per head ``[N, H, H]`` fp32, folded to ``heads`` weight heads."""
    from .gemm import _bmm_kernel

    B, S, N, H = left.shape
    # per head: left^T right over the B * S steps: both operands are read as [steps, H] = MN-major (no transposes)
    lt = left.permute(2, 0, 1, 3).reshape(N, B * S, H)
    rt = right.permute(2, 0, 1, 3).reshape(N, B * S, H)
    dW = _bmm_kernel(lt, rt, True, True, torch.float32)
    return dW if heads == N else dW.view(heads, N // heads, H, H).sum(1)


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, xf, xr, W, Wf, Wr, h0, clip, gru: bool):
        x = _head_major(x)
        B, S, _, H = x.shape
        ws = [W.to(torch.bfloat16).contiguous()]
        xs = [x]
        if gru:
            xs += [_head_major(xf), _head_major(xr)]
            ws += [Wf.to(torch.bfloat16).contiguous(), Wr.to(torch.bfloat16).contiguous()]
        N = max(*(t.size(2) for t in xs), *(w.size(0) for w in ws))
        dev = x.device
        h0b = (h0.to(torch.bfloat16).contiguous() if h0 is not None
               else torch.zeros((B, N, H), dtype=torch.bfloat16, device=dev))
        y = torch.empty((B, S, N, H), dtype=torch.bfloat16, device=dev)
        a = _Args()
        _Scan._fill(a, xs, ws, N, gru)
        a.h0, a.y = h0b.data_ptr(), y.data_ptr()
        _launch(a, 0, f"lme_rnn forward gru={gru} B={B} S={S} N={N} H={H}")
        ctx.save_for_backward(*xs, *ws, h0b, y)
        ctx.meta = (N, gru, clip, h0 is not None, h0.dtype if h0 is not None else None,
                    [W.dtype] + ([Wf.dtype, Wr.dtype] if gru else []))
        return y, y[:, -1].clone()

    @staticmethod
    def _fill(a: _Args, xs, ws, N: int, gru: bool) -> None:
        x = xs[0]
        B, S, _, H = x.shape
        a.B, a.S, a.N, a.H, a.gru = B, S, N, H, int(gru)
        a.x, a.x_b, a.x_t, a.Nx = x.data_ptr(), x.stride(0), x.stride(1), x.size(2)
        a.W, a.Nw = ws[0].data_ptr(), ws[0].size(0)
        if gru:
            xf, xr = xs[1], xs[2]
            a.xf, a.xf_b, a.xf_t, a.Nxf = xf.data_ptr(), xf.stride(0), xf.stride(1), xf.size(2)
            a.xr, a.xr_b, a.xr_t, a.Nxr = xr.data_ptr(), xr.stride(0), xr.stride(1), xr.size(2)
            a.Wf, a.Nwf, a.Wr, a.Nwr = ws[1].data_ptr(), ws[1].size(0), ws[2].data_ptr(), ws[2].size(0)
        else:
            a.Nxf = a.Nxr = a.Nwf = a.Nwr = 1

    @staticmethod
    def backward(ctx, dy, dh_out):
        N, gru, clip, has_h0, h0_dtype, w_dtypes = ctx.meta
        saved = ctx.saved_tensors
        nx = 3 if gru else 1
        xs, ws, h0b, y = list(saved[:nx]), list(saved[nx:2 * nx]), saved[2 * nx], saved[2 * nx + 1]
        B, S, _, H = y.shape
        dev = y.device
        dy = (dy.to(torch.bfloat16).contiguous() if dy is not None else torch.zeros_like(y))
        dh = (dh_out.float().contiguous().clone() if dh_out is not None
              else torch.zeros((B, N, H), dtype=torch.float32, device=dev))
        outs = [torch.empty_like(y) for _ in range(4 if gru else 1)]      # dx (, dxf, dxr, hr)
        a = _Args()
        _Scan._fill(a, xs, ws, N, gru)
        a.h0, a.y, a.dy, a.dh, a.dx = h0b.data_ptr(), y.data_ptr(), dy.data_ptr(), dh.data_ptr(), outs[0].data_ptr()
        if gru:
            a.dxf, a.dxr, a.hr = outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr()
        a.clip = float(clip) if clip is not None else 0.0
        _launch(a, 1, f"lme_rnn backward gru={gru} B={B} S={S} N={N} H={H}")
        hprev = torch.cat((h0b[:, None], y[:, :-1]), dim=1)

        def fold(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
            heads = like.size(2)
            return t if heads == N else t.view(B, S, heads, N // heads, H).float().sum(3).to(like.dtype)

        if gru:
            dW = _weight_grad(outs[3], outs[0], ws[0].size(0)).to(w_dtypes[0])
            dWf = _weight_grad(hprev, outs[1], ws[1].size(0)).to(w_dtypes[1])
            dWr = _weight_grad(hprev, outs[2], ws[2].size(0)).to(w_dtypes[2])
            dxs = [fold(outs[i], xs[i]) for i in range(3)]
        else:
            dW, dWf, dWr = _weight_grad(hprev, outs[0], ws[0].size(0)).to(w_dtypes[0]), None, None
            dxs = [fold(outs[0], xs[0]), None, None]
        return (*dxs, dW, dWf, dWr, dh.to(h0_dtype) if has_h0 else None, None, None)


def rnn_cuda(x, W, h0=None, gradient_clipping=None):
    """Same contract as :func:`lm_engine_b200.ops.recurrence.rnn_scan`."""
    return _Scan.apply(x, None, None, W, None, None, h0, gradient_clipping, False)


def gru_cuda(x, xf, xr, W, Wf, Wr, h0=None, gradient_clipping=None):
    """Same contract as :func:`lm_engine_b200.ops.recurrence.gru_scan`."""
    return _Scan.apply(x, xf, xr, W, Wf, Wr, h0, gradient_clipping, True)
