"""Mixture-of-experts token routing primitives: expert histogram, grouped (per-expert) linear, and the expert-parallel
all-to-all exchange.

``grouped_linear(x, weight, counts)`` applies ``weight[e]`` to the ``counts[e]`` consecutive rows of ``x`` that were
routed to expert ``e`` (rows sorted by expert) - the operation the reference gets from ScatterMoE
(lm_engine/modeling_utils/mlp_blocks/moe/experts.py:137-149,212-225) or, without it, from a per-expert loop.  On CUDA
bf16 every expert's product runs on the tcgen05 GEMM (including the transposed dgrad / wgrad forms through autograd).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .gemm import linear


def expert_histogram(sorted_expert_idxs: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Tokens per expert (int64 ``[num_experts]``); the input need not be sorted."""
    return torch.bincount(sorted_expert_idxs, minlength=num_experts)


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, counts: list[int],
                   bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x [sum(counts), in]``, ``weight [E, out, in]`` -> ``[sum(counts), out]``."""
    outs = []
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        outs.append(linear(x[start:start + n], weight[e], None if bias is None else bias[e]))
        start += n
    if not outs:
        return x.new_zeros((0, weight.size(1)))
    return torch.cat(outs, dim=0)


# ---------------------------------------------------------------------------------------------------- grouped GEMM
TILE_ROWS = 128


class GroupLayout:
    """Padded per-expert row layout: expert ``e`` owns rows ``[start[e], start[e] + pad[e])`` with ``pad[e]`` the
    count rounded up to the 128-row GEMM tile, so every tile belongs to one expert.  Everything is computed on the
    device from the per-expert counts; the row capacity is the static upper bound ``rows + E * 127`` (rounded up),
    tiles past the last expert are marked unused and skipped by the kernels.  No host synchronisation."""

    def __init__(self, sorted_experts: torch.Tensor, freq: torch.Tensor, order: torch.Tensor | None = None,
                 top_k: int = 1) -> None:
        E, total = freq.numel(), sorted_experts.numel()
        dev = freq.device
        pad = (freq + (TILE_ROWS - 1)) // TILE_ROWS * TILE_ROWS
        end = pad.cumsum(0)
        start = end - pad
        first_sorted = freq.cumsum(0) - freq
        self.capacity = (total + E * (TILE_ROWS - 1) + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS
        self.dest = start[sorted_experts] + (torch.arange(total, device=dev) - first_sorted[sorted_experts])
        tile_start = torch.arange(self.capacity // TILE_ROWS, device=dev) * TILE_ROWS
        grp = torch.searchsorted(end, tile_start, right=True)
        self.tile_group = torch.where(grp < E, grp, torch.full_like(grp, -1)).to(torch.int32)
        self.k0 = start.to(torch.int32)
        self.kb = (pad // 64).to(torch.int32)
        self.num_groups = E
        # slot[t, k]: padded row of the k-th assignment of token t (``order`` maps sorted position -> t * top_k + k)
        self.slot = None
        if order is not None:
            flat = torch.empty(total, dtype=torch.int32, device=dev)
            flat.scatter_(0, order, self.dest.to(torch.int32))
            self.slot = flat.view(total // top_k, top_k)

    @classmethod
    def from_selection(cls, selected: torch.Tensor, num_experts: int) -> "GroupLayout":
        """The same layout straight from the unsorted ``selected [T, K]`` (int64, CUDA): three small kernels (per-CTA
        histograms, one scan, stable ranks) instead of a sort, a histogram, two scans, a search and a scatter.
        ``freq`` (int64 ``[E]``) is filled as a by-product; ``dest`` is not (the layout is reached through ``slot``)."""
        from . import _lib

        sel = selected.contiguous()
        total, dev = sel.numel(), sel.device
        self = cls.__new__(cls)
        self.capacity = (total + num_experts * (TILE_ROWS - 1) + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS
        ntiles = self.capacity // TILE_ROWS
        lib = _lib.cuda_lib()
        ints = torch.empty(lib.lme_moe_route_chunks(total) * num_experts + 2 * num_experts + ntiles + total,
                           dtype=torch.int32, device=dev)
        scratch, self.k0, self.kb, self.tile_group, flat = ints.split(
            [ints.numel() - 2 * num_experts - ntiles - total, num_experts, num_experts, ntiles, total])
        self.freq = torch.empty(num_experts, dtype=torch.int64, device=dev)
        _lib.check(lib.lme_moe_route_layout(sel.data_ptr(), total, num_experts, scratch.data_ptr(),
                                            self.freq.data_ptr(), self.k0.data_ptr(), self.kb.data_ptr(),
                                            self.tile_group.data_ptr(), ntiles, flat.data_ptr(), _lib.stream_ptr()),
                   f"lme_moe_route_layout total={total} E={num_experts}")
        _lib.count_launch(3)
        self.num_groups, self.dest = num_experts, None
        self.slot = flat.view(selected.shape)
        return self

    def scatter(self, rows: torch.Tensor) -> torch.Tensor:
        """Rows sorted by expert -> padded layout (padding rows zero)."""
        out = torch.zeros((self.capacity, rows.size(1)), dtype=rows.dtype, device=rows.device)
        return out.index_copy(0, self.dest, rows)

    def gather(self, padded: torch.Tensor) -> torch.Tensor:
        return padded.index_select(0, self.dest)


def _grouped_gemm(a: torch.Tensor, w2d: torch.Tensor, layout: GroupLayout, n: int, k: int, b_mn: bool,
                  swiglu: bool = False, preact: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """``out`` (optional): a buffer of the result's shape to write into; rows of tiles without an expert keep what
    they held."""
    from . import _lib
    from .gemm import _max_ctas

    if out is None:
        # rows of tiles without an expert are never written and never read (every consumer walks the same tile table
        # or the slots), so the buffer is not cleared: with a capacity of twice the routed rows the fills cost more
        # than a millisecond per layer
        out = torch.empty((a.size(0), n // 2 if swiglu else n), dtype=torch.bfloat16, device=a.device)
    else:
        assert out.shape == (a.size(0), n // 2 if swiglu else n) and out.dtype == torch.bfloat16
        out = out.view(out.shape)          # a new tensor object per call: autograd hangs its node on the object
    rc = _lib.cuda_lib().lme_gemm_bf16_grouped(
        a.data_ptr(), a.stride(0), w2d.data_ptr(), int(b_mn), w2d.stride(0), out.data_ptr(), out.stride(0),
        a.size(0), n, k, layout.num_groups, _lib.GEMM_SWIGLU if swiglu else 0, _lib.ptr(preact),
        preact.stride(0) if preact is not None else 0, layout.tile_group.data_ptr(), _max_ctas(a.device),
        _lib.stream_ptr())
    _lib.check(rc, f"lme_gemm_bf16_grouped rows={a.size(0)} N={n} K={k} groups={layout.num_groups}")
    _lib.count_launch()
    return out


class _GroupedLinear(torch.autograd.Function):
    """``y[rows of e] = x[rows of e] @ W[e].T`` (optionally followed by the packed SwiGLU in the epilogue) on rows in
    the padded layout: one persistent tcgen05 kernel over all experts for each of forward, dgrad and wgrad."""

    @staticmethod
    def forward(ctx, x_pad, weight, layout: GroupLayout, swiglu: bool, out=None, dgrad_out=None):
        E, N, K = weight.shape
        pre = torch.empty((x_pad.size(0), N), dtype=x_pad.dtype, device=x_pad.device) if swiglu else None
        y = _grouped_gemm(x_pad, weight.view(E * N, K), layout, N, K, False, swiglu, pre, out=out)
        ctx.save_for_backward(x_pad, weight, pre)
        ctx.layout, ctx.swiglu, ctx.dgrad_out = layout, swiglu, dgrad_out
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _lib
        from .activation import swiglu_backward
        from .gemm import _max_ctas

        x_pad, weight, pre = ctx.saved_tensors
        layout = ctx.layout
        E, N, K = weight.shape
        dy = dy.contiguous()
        if ctx.swiglu:
            dy = swiglu_backward(pre, dy, layout.tile_group)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx = dy @ W[e]: W[e] is [N, K] = the MN-major operand whose contraction rows are offset by e * N
            dx = _grouped_gemm(dy, weight.view(E * N, K), layout, K, N, True, out=ctx.dgrad_out)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            stale = getattr(weight, "main_grad_stale", False)
            if main_grad is not None:
                out, flags = main_grad, (0 if stale else _lib.GEMM_ACCUMULATE)
            else:
                out, flags = torch.empty_like(weight), 0
            if out.dtype == torch.float32:
                flags |= _lib.GEMM_OUT_F32
            rc = _lib.cuda_lib().lme_gemm_bf16_grouped_wgrad(
                dy.data_ptr(), dy.stride(0), x_pad.data_ptr(), x_pad.stride(0), out.data_ptr(), K, N, K,
                dy.size(0), E, layout.k0.data_ptr(), layout.kb.data_ptr(), flags, _max_ctas(dy.device),
                _lib.stream_ptr())
            _lib.check(rc, f"lme_gemm_bf16_grouped_wgrad N={N} K={K} groups={E}")
            _lib.count_launch()
            if main_grad is not None:
                if stale:
                    weight.main_grad_stale = False
            else:
                dw = out
        return dx, dw, None, None, None, None


def grouped_linear_padded(x_pad: torch.Tensor, weight: torch.Tensor, layout: GroupLayout, swiglu: bool = False,
                          out: torch.Tensor | None = None, dgrad_out: torch.Tensor | None = None) -> torch.Tensor:
    """``out`` / ``dgrad_out``: buffers that receive the result / the input gradient (the expert-parallel exchange
    passes its output slabs, so that the rows are published where the kernels wrote them)."""
    return _GroupedLinear.apply(x_pad, weight, layout, swiglu, out, dgrad_out)


def _rows_call(fn_name: str, src, slot, w, dst, T, H, K) -> None:
    from . import _lib

    rc = getattr(_lib.cuda_lib(), fn_name)(src.data_ptr(), slot.data_ptr(), _lib.ptr(w), dst.data_ptr(), T, H, K,
                                            _lib.stream_ptr())
    _lib.check(rc, f"{fn_name} T={T} H={H} K={K}")
    _lib.count_launch()


class _Dispatch(torch.autograd.Function):
    """Tokens ``[T, H]`` -> padded per-expert rows (each token copied to its ``top_k`` slots); backward sums a
    token's slots.  One pass each way, no atomics."""

    @staticmethod
    def forward(ctx, x, slot, capacity: int):
        x = x.contiguous()
        out = torch.zeros((capacity, x.size(1)), dtype=x.dtype, device=x.device)
        _rows_call("lme_moe_scatter_rows", x, slot, None, out, x.size(0), x.size(1), slot.size(1))
        ctx.slot, ctx.shape = slot, x.shape
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dx = torch.empty(ctx.shape, dtype=g.dtype, device=g.device)
        _rows_call("lme_moe_gather_reduce", g, ctx.slot, None, dx, ctx.shape[0], ctx.shape[1], ctx.slot.size(1))
        return dx, None, None


class _Combine(torch.autograd.Function):
    """``out[t] = sum_k gates[t, k] * y_pad[slot[t, k]]``; backward scatters ``gates * dout`` to the slots and takes
    the row dot products for the gate gradients."""

    @staticmethod
    def forward(ctx, y_pad, gates, slot, grad_buffer=None):
        y_pad, gates = y_pad.contiguous(), gates.contiguous()
        ctx.grad_buffer = grad_buffer
        T, K = slot.shape
        out = torch.empty((T, y_pad.size(1)), dtype=y_pad.dtype, device=y_pad.device)
        _rows_call("lme_moe_gather_reduce", y_pad, slot, gates, out, T, y_pad.size(1), K)
        ctx.save_for_backward(y_pad, gates)
        ctx.slot = slot
        return out

    @staticmethod
    def backward(ctx, dout):
        y_pad, gates = ctx.saved_tensors
        dout = dout.contiguous()
        T, K = ctx.slot.shape
        H = y_pad.size(1)
        dy = dg = None
        if ctx.needs_input_grad[0]:
            # grad_buffer: a caller-owned buffer of y_pad's shape whose every row is some token's slot (nothing to clear)
            dy = torch.zeros_like(y_pad) if ctx.grad_buffer is None else ctx.grad_buffer.view(y_pad.shape)
            _rows_call("lme_moe_scatter_rows", dout, ctx.slot, gates, dy, T, H, K)
        if ctx.needs_input_grad[1]:
            dg = torch.empty_like(gates)
            _rows_call("lme_moe_row_dots", y_pad, ctx.slot, dout, dg, T, H, K)
        return dy, dg, None, None


class _TopKSoftmax(torch.autograd.Function):
    """Router weights and selection in one kernel each way (one warp per token): top-k of the logits, softmax over
    the selected ones (``normalized``) or over all experts."""

    @staticmethod
    def forward(ctx, logits, k: int, normalized: bool):
        from . import _lib

        logits = logits.contiguous()
        T, E = logits.shape
        w = torch.empty((T, k), dtype=logits.dtype, device=logits.device)
        sel = torch.empty((T, k), dtype=torch.int64, device=logits.device)
        lse = None if normalized else torch.empty(T, dtype=torch.float32, device=logits.device)
        _lib.check(_lib.cuda_lib().lme_moe_topk_softmax_fwd(logits.data_ptr(), T, E, k, int(normalized), w.data_ptr(),
                                                            sel.data_ptr(), _lib.ptr(lse), _lib.stream_ptr()),
                   f"lme_moe_topk_softmax_fwd T={T} E={E} K={k}")
        _lib.count_launch()
        ctx.save_for_backward(logits, sel, *([] if lse is None else [lse]))
        ctx.normalized = normalized
        ctx.mark_non_differentiable(sel)
        return w, sel

    @staticmethod
    def backward(ctx, dw, _dsel):
        from . import _lib

        logits, sel, *rest = ctx.saved_tensors
        T, E = logits.shape
        dl = torch.empty_like(logits)
        dw = dw.contiguous()
        _lib.check(_lib.cuda_lib().lme_moe_topk_softmax_bwd(logits.data_ptr(), sel.data_ptr(), dw.data_ptr(),
                                                            _lib.ptr(rest[0] if rest else None), T, E, sel.size(1),
                                                            int(ctx.normalized), dl.data_ptr(), _lib.stream_ptr()),
                   f"lme_moe_topk_softmax_bwd T={T} E={E} K={sel.size(1)}")
        _lib.count_launch()
        return dl, None, None


def topk_softmax_eligible(logits: torch.Tensor, k: int) -> bool:
    return (logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2 and k <= 32
            and k <= logits.size(1) <= 512)


def topk_softmax(logits: torch.Tensor, k: int, normalized: bool):
    """``(weights [T, k] in the logits' dtype, selected [T, k] int64)`` of the router
    (role of lm_engine/modeling_utils/mlp_blocks/moe/__init__.py's top-k + softmax in either order)."""
    return _TopKSoftmax.apply(logits, k, normalized)


def dispatch_tokens(x: torch.Tensor, layout: GroupLayout) -> torch.Tensor:
    return _Dispatch.apply(x, layout.slot, layout.capacity)


def combine_tokens(y_pad: torch.Tensor, gates: torch.Tensor, layout: GroupLayout) -> torch.Tensor:
    return _Combine.apply(y_pad, gates, layout.slot, getattr(layout, "grad_buffer", None))


def grouped_kernels_eligible(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and all(
        w.dtype == torch.bfloat16 and w.is_contiguous() and w.size(1) % 64 == 0 and w.size(2) % 64 == 0
        for w in weights)


class _AllToAll(torch.autograd.Function):
    """Variable-size all-to-all of rows; backward is the all-to-all with the split lists swapped."""

    @staticmethod
    def forward(ctx, x, send_counts: list[int], recv_counts: list[int], group):
        ctx.group, ctx.send, ctx.recv = group, send_counts, recv_counts
        out = x.new_empty((sum(recv_counts), *x.shape[1:]))
        if x.is_cuda:
            dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts,
                                   input_split_sizes=send_counts, group=group)
        else:
            # gloo: emulate with all_gather of padded blocks
            world, r = dist.get_world_size(group), dist.get_rank(group)
            counts = [None] * world
            dist.all_gather_object(counts, send_counts, group=group)
            mx = max(max(c) for c in counts) if counts else 0
            pad = x.new_zeros((world, max(mx, 1), *x.shape[1:]))
            off = 0
            for j, n in enumerate(send_counts):
                pad[j, :n] = x[off:off + n]
                off += n
            gathered = [torch.empty_like(pad) for _ in range(world)]
            dist.all_gather(gathered, pad, group=group)
            pieces = [gathered[src][r, :counts[src][r]] for src in range(world)]
            out = torch.cat(pieces, dim=0) if pieces else out
        return out

    @staticmethod
    def backward(ctx, g):
        return _AllToAll.apply(g, ctx.recv, ctx.send, ctx.group), None, None, None


def all_to_all_rows(x: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    return _AllToAll.apply(x, send_counts, recv_counts, group)
