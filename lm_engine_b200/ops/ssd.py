"""Mamba-2 state-space-duality (SSD) scan.

``y_t = C_t . h_t + D x_t``,  ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t (x) x_t``  per head, evaluated chunk by chunk:
intra-chunk as a masked ``(C B^T) . decay`` product (tensor-core shaped), chunk summaries ``S_c``, a short sequential
pass over chunk boundaries, and the contribution of the carried state.  Same results as the token-by-token
recurrence (and as ``mamba_chunk_scan_combined`` / the reference's ``mamba2_torch``,
lm_engine/modeling_utils/sequence_mixer_blocks/mamba2/op.py:225-457) without materialising a
``[chunks, L, L, heads, state]`` tensor.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

FUSED_INTRA_CHUNK = True   # tests switch it off to compare the two paths


def ssd_recurrent_step(x, dt, A, B, C, D, h):
    """One token.  x ``[b, N, P]``, dt ``[b, N]``, B/C ``[b, G, Sd]``, h ``[b, N, P, Sd]`` (fp32)."""
    N, G = x.size(1), B.size(1)
    Bh = B.float().repeat_interleave(N // G, dim=1)
    Ch = C.float().repeat_interleave(N // G, dim=1)
    dA = torch.exp(dt.float() * A.float())[..., None, None]
    h = h.float() * dA + (dt.float()[..., None] * x.float())[..., None] * Bh[:, :, None, :]
    y = (h * Ch[:, :, None, :]).sum(-1) + D.float()[None, :, None] * x.float()
    return y.to(x.dtype), h


def _group_mm(a: torch.Tensor, b: torch.Tensor, lowp: bool) -> torch.Tensor:
    """``a @ b`` over the leading (batch, chunk, group) dims with an fp32 result; bf16 operands on the tensor cores
    (the batched tcgen05 GEMM, ``b`` read as its MN-major operand) when the model computes in bf16, plain fp32
    otherwise."""
    lead = a.shape[:-2]
    a2, b2 = a.reshape(-1, *a.shape[-2:]), b.reshape(-1, *b.shape[-2:])
    if lowp:
        from .gemm import bmm

        out = bmm(a2.to(torch.bfloat16), b2.to(torch.bfloat16), b_mn=True)
    else:
        out = torch.bmm(a2.float(), b2.float())
    return out.view(*lead, a.size(-2), b.size(-1))


class _IntraChunk(torch.autograd.Function):
    """``y[l] = sum_{s<=l} exp(cum[l]-cum[s]) CB[l,s] xdt[s]`` per (batch, chunk, head) on CUDA: the decay-masked
    matrix is built in one kernel (bf16), the two products run as batched tensor-core GEMMs, and the backward needs
    one more kernel (group sum of ``dM * decay``); the gradient of ``cum`` follows from ``dy . y`` and
    ``xdt . dxdt`` without another L x L pass."""

    @staticmethod
    def forward(ctx, CB, ct, xdt):
        # CB [b, nc, G, L, L] bf16, ct [b, nc, N, L] fp32, xdt [b, nc, N, L, P] bf16
        from . import _lib

        b, nc, G, L, _ = CB.shape
        N, P = ct.size(2), xdt.size(-1)
        CB, ct, xdt = CB.contiguous(), ct.contiguous(), xdt.contiguous()
        M = torch.empty((b, nc, N, L, L), dtype=torch.bfloat16, device=CB.device)
        _lib.check(_lib.cuda_lib().lme_ssd_decay_matrix(CB.data_ptr(), ct.data_ptr(), M.data_ptr(), b * nc, N, G, L,
                                                        _lib.stream_ptr()), "lme_ssd_decay_matrix")
        _lib.count_launch()
        from .gemm import _bmm_kernel

        # y = M xdt: M is [l, s] (K-major), xdt is [s, P] = [K, N] (MN-major)
        y = _bmm_kernel(M.view(-1, L, L), xdt.view(-1, L, P), False, True, torch.float32).view(b, nc, N, L, P)
        ctx.save_for_backward(M, ct, xdt, y)
        ctx.G = G
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _lib

        M, ct, xdt, y = ctx.saved_tensors
        b, nc, N, L, P = xdt.shape
        G = ctx.G
        dy32 = dy.contiguous().float()
        dy = dy32.to(torch.bfloat16)
        dyv, xv = dy.view(-1, L, P), xdt.view(-1, L, P)
        from .gemm import _bmm_kernel

        dM = _bmm_kernel(dyv, xv, False, False, torch.bfloat16)          # dy xdt^T  [bcn, L, L]
        # M^T dy: M read as the MN-major A operand, dy [l, P] = [K, N] as the MN-major B operand
        dxdt = _bmm_kernel(M.view(-1, L, L), dyv, True, True, torch.float32).view(b, nc, N, L, P)
        dCB = torch.empty((b, nc, G, L, L), dtype=torch.bfloat16, device=dy.device)
        _lib.check(_lib.cuda_lib().lme_ssd_dcb(dM.data_ptr(), ct.data_ptr(), dCB.data_ptr(), b * nc, N, G, L,
                                               _lib.stream_ptr()), "lme_ssd_dcb")
        _lib.count_launch()
        dct = (dy32 * y).sum(-1) - (xdt.float() * dxdt).sum(-1)   # [b, nc, N, L]
        return dCB, dct, dxdt


class _ScanPrep(torch.autograd.Function):
    """``xh[b,c,n,l,:] = x dt`` and ``xwT[b,c,n,:,l] = x dt tail`` (bf16 operands of the intra-chunk and the
    chunk-state products) from ``x [b, nc, L, N, P]`` bf16 and ``dt``, ``tail [b, nc, L, N]`` fp32, in one kernel;
    one more for all three gradients."""

    @staticmethod
    def forward(ctx, x, dt, tail):
        from . import _lib

        b, nc, L, N, P = x.shape
        x, dt, tail = x.contiguous(), dt.contiguous(), tail.contiguous()
        xh = torch.empty((b, nc, N, L, P), dtype=torch.bfloat16, device=x.device)
        xwT = torch.empty((b, nc, N, P, L), dtype=torch.bfloat16, device=x.device)
        _lib.check(_lib.cuda_lib().lme_ssd_prep(x.data_ptr(), dt.data_ptr(), tail.data_ptr(), xh.data_ptr(),
                                                xwT.data_ptr(), None, None, None, None, None, b * nc, N, L, P, 0,
                                                _lib.stream_ptr()), "lme_ssd_prep")
        _lib.count_launch()
        ctx.save_for_backward(x, dt, tail)
        return xh, xwT

    @staticmethod
    def backward(ctx, dxh, dxwT):
        from . import _lib

        x, dt, tail = ctx.saved_tensors
        b, nc, L, N, P = x.shape
        dxh = (torch.zeros((b, nc, N, L, P), dtype=torch.float32, device=x.device) if dxh is None
               else dxh.float().contiguous())
        dxwT = (torch.zeros((b, nc, N, P, L), dtype=torch.bfloat16, device=x.device) if dxwT is None
                else dxwT.to(torch.bfloat16).contiguous())
        dx = torch.empty_like(x)
        ddt, dtail = torch.empty_like(dt), torch.empty_like(tail)
        _lib.check(_lib.cuda_lib().lme_ssd_prep(x.data_ptr(), dt.data_ptr(), tail.data_ptr(), None, None,
                                                dxh.data_ptr(), dxwT.data_ptr(), dx.data_ptr(), ddt.data_ptr(),
                                                dtail.data_ptr(), b * nc, N, L, P, 1, _lib.stream_ptr()),
                   "lme_ssd_prep(backward)")
        _lib.count_launch()
        return dx, ddt, dtail


class _ScanCombine(torch.autograd.Function):
    """``y = yin^T + off ecum + D x`` in bf16 ``[b, nc, L, N, P]`` from the intra-chunk result ``yin [b,nc,N,L,P]``,
    the carried-state product ``off [b,nc,G,L,(N/G) P]`` (both fp32), ``ecum [b,nc,L,N]``, ``D [N]`` and ``x``."""

    @staticmethod
    def forward(ctx, yin, off, ecum, D, x):
        from . import _lib

        b, nc, L, N, P = x.shape
        G = off.size(2)
        yin, off, ecum, D, x = yin.contiguous(), off.contiguous(), ecum.contiguous(), D.contiguous(), x.contiguous()
        y = torch.empty_like(x)
        _lib.check(_lib.cuda_lib().lme_ssd_combine(yin.data_ptr(), off.data_ptr(), ecum.data_ptr(), D.data_ptr(),
                                                   x.data_ptr(), y.data_ptr(), None, None, None, None, None, None,
                                                   b * nc, N, L, G, P, 0, _lib.stream_ptr()), "lme_ssd_combine")
        _lib.count_launch()
        ctx.save_for_backward(off, ecum, D, x)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _lib

        off, ecum, D, x = ctx.saved_tensors
        b, nc, L, N, P = x.shape
        G = off.size(2)
        dy = dy.to(torch.bfloat16).contiguous()
        dyin = torch.empty((b, nc, N, L, P), dtype=torch.bfloat16, device=x.device)
        doff = torch.empty(off.shape, dtype=torch.bfloat16, device=x.device)
        decum = torch.empty_like(ecum)
        dDp = torch.empty_like(ecum)
        dx = torch.empty_like(x)
        _lib.check(_lib.cuda_lib().lme_ssd_combine(None, off.data_ptr(), ecum.data_ptr(), D.data_ptr(), x.data_ptr(),
                                                   None, dy.data_ptr(), dyin.data_ptr(), doff.data_ptr(),
                                                   decum.data_ptr(), dDp.data_ptr(), dx.data_ptr(), b * nc, N, L, G,
                                                   P, 1, _lib.stream_ptr()), "lme_ssd_combine(backward)")
        _lib.count_launch()
        return dyin, doff, decum, dDp.sum((0, 1, 2)), dx


class _BoundaryScan(torch.autograd.Function):
    """``h_{c+1} = decay[c] h_c + S_c`` over the chunks of every (batch, head) in one kernel each way.  Returns the
    state at every chunk start in bf16 (``[b, nc, N, P, Sd]``, the operand of the carried-state product) and the
    final state in fp32."""

    @staticmethod
    def forward(ctx, states, decay, h_init):
        from . import _lib

        b, nc, N, P, Sd = states.shape
        states, decay = states.contiguous(), decay.contiguous()
        h_init = None if h_init is None else h_init.float().contiguous()
        h0 = torch.empty((b, nc, N, P, Sd), dtype=torch.bfloat16, device=states.device)
        keep = any(ctx.needs_input_grad)      # the backward pass walks the fp32 states
        h0f = torch.empty((b, nc, N, P, Sd), dtype=torch.float32, device=states.device) if keep else None
        hf = torch.empty((b, N, P, Sd), dtype=torch.float32, device=states.device)
        _lib.check(_lib.cuda_lib().lme_ssd_boundary_fwd(states.data_ptr(), decay.data_ptr(), _lib.ptr(h_init),
                                                        h0.data_ptr(), _lib.ptr(h0f), hf.data_ptr(), b, nc, N,
                                                        P * Sd, _lib.stream_ptr()), "lme_ssd_boundary_fwd")
        _lib.count_launch()
        ctx.save_for_backward(h0f, decay)
        ctx.has_init = h_init is not None
        return h0, hf

    @staticmethod
    def backward(ctx, dh0, dhf):
        from . import _lib

        h0f, decay = ctx.saved_tensors
        b, nc, N, P, Sd = h0f.shape
        dh0 = None if dh0 is None else dh0.float().contiguous()
        dhf = None if dhf is None else dhf.float().contiguous()
        dstates = torch.empty_like(h0f)
        ddecay = torch.empty_like(decay)
        dinit = torch.empty((b, N, P, Sd), dtype=torch.float32, device=h0f.device) if ctx.has_init else None
        _lib.check(_lib.cuda_lib().lme_ssd_boundary_bwd(_lib.ptr(dh0), _lib.ptr(dhf), h0f.data_ptr(),
                                                        decay.data_ptr(), dstates.data_ptr(), ddecay.data_ptr(),
                                                        _lib.ptr(dinit), b, nc, N, P * Sd, _lib.stream_ptr()),
                   "lme_ssd_boundary_bwd")
        _lib.count_launch()
        return dstates, ddecay, dinit


def scan_glue_eligible(x: torch.Tensor, L: int) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and L % 32 == 0 and L <= 1024 and x.size(-1) in (32, 64, 128)
            and FUSED_INTRA_CHUNK)


def _intra_chunk_fused(Cc, Bc, ct, xdt):
    """CUDA path of the intra-chunk term.  Cc / Bc ``[b, nc, L, G, Sd]``, ct ``[b, nc, N, L]`` fp32,
    xdt ``[b, nc, L, N, P]`` fp32 -> ``[b, nc, L, N, P]`` fp32."""
    Cg = Cc.permute(0, 1, 3, 2, 4).to(torch.bfloat16)                    # [b, nc, G, L, Sd]
    Bg = Bc.permute(0, 1, 3, 2, 4).to(torch.bfloat16)
    from .gemm import bmm

    CB = bmm(Cg.reshape(-1, *Cg.shape[-2:]), Bg.reshape(-1, *Bg.shape[-2:]),
             out_dtype=torch.bfloat16).view(*Cg.shape[:-1], Cg.size(-2))  # [b, nc, G, L, L] bf16
    xh = xdt.permute(0, 1, 3, 2, 4).to(torch.bfloat16)                   # [b, nc, N, L, P]
    y = _IntraChunk.apply(CB, ct, xh)
    return y.permute(0, 1, 3, 2, 4)


def ssd_chunk_scan(x, dt, A, B, C, D, chunk_size: int, initial_state=None):
    """x ``[b, S, N, P]``, dt ``[b, S, N]`` (already softplus'ed), A ``[N]`` (negative), B/C ``[b, S, G, Sd]``,
    D ``[N]``.  Returns ``(y [b, S, N, P], final_state [b, N, P, Sd] fp32)``."""
    b, S, N, P = x.shape
    G, Sd = B.shape[-2:]
    dtype = x.dtype
    L = chunk_size
    pad = (L - S % L) % L
    kernels = scan_glue_eligible(x, L)          # then x is consumed in bf16 by the glue kernels: no fp32 copy of it
    xf, dtf, Bf, Cf = (None if kernels else x.float()), dt.float(), B.float(), C.float()
    if pad:
        if not kernels:
            xf = torch.nn.functional.pad(xf, (0, 0, 0, 0, 0, pad))
        dtf = torch.nn.functional.pad(dtf, (0, 0, 0, pad))
        Bf = torch.nn.functional.pad(Bf, (0, 0, 0, 0, 0, pad))
        Cf = torch.nn.functional.pad(Cf, (0, 0, 0, 0, 0, pad))
    nc = (S + pad) // L
    xc = None if kernels else xf.view(b, nc, L, N, P)
    dtc = dtf.view(b, nc, L, N)
    Bc = Bf.view(b, nc, L, G, Sd)
    Cc = Cf.view(b, nc, L, G, Sd)
    rep = N // G
    dA = dtc * A.float()                                      # [b, nc, L, N]
    cum = torch.cumsum(dA, dim=2)
    if kernels:
        return _chunk_scan_kernels(x, pad, dtc, cum, Bc, Cc, D, initial_state, b, S, nc, L, N, P, G, Sd)
    # ---- intra-chunk: y[t] = sum_{s<=t} exp(cum[t]-cum[s]) (C_t.B_s) dt_s x_s
    ct = cum.permute(0, 1, 3, 2)                              # [b, nc, N, L]
    xdt = xc * dtc[..., None]                                 # [b, nc, L, N, P]
    if x.is_cuda and dtype == torch.bfloat16 and L % 8 == 0 and L <= 1024 and FUSED_INTRA_CHUNK:
        y = _intra_chunk_fused(Cc, Bc, ct, xdt)
    else:
        CB = torch.einsum("bclgn,bcsgn->bcgls", Cc, Bc)       # [b, nc, G, L, L]
        CB = CB.repeat_interleave(rep, dim=2)                 # [b, nc, N, L, L]
        seg = ct[..., :, None] - ct[..., None, :]             # cum[t] - cum[s]
        causal = torch.ones(L, L, dtype=torch.bool, device=x.device).tril()
        decay = torch.exp(seg.masked_fill(~causal, float("-inf")))
        y = torch.einsum("bcnls,bcsnp->bclnp", CB * decay, xdt)
    # ---- chunk summaries: S_c = sum_s exp(cum[L-1]-cum[s]) B_s (x) (dt_s x_s)
    # The heads of a group share B and C, so both state products are batched GEMMs over (batch, chunk, group) with
    # the group's heads folded into the GEMM's M / N dimension: no per-head copies of B or C are made.
    lowp = x.is_cuda and dtype == torch.bfloat16
    tail = torch.exp(cum[:, :, -1:, :] - cum)                 # [b, nc, L, N]
    xw = (xdt * tail[..., None]).view(b, nc, L, G, rep * P)   # [b, nc, L, G, rep*P]
    states = _group_mm(xw.permute(0, 1, 3, 4, 2), Bc.permute(0, 1, 3, 2, 4), lowp)   # [b, nc, G, rep*P, Sd]
    states = states.view(b, nc, N, P, Sd)
    # ---- boundary states: h_c = exp(sum dA of chunk c-1) h_{c-1} + S_{c-1}
    h = (torch.zeros(b, N, P, Sd, dtype=torch.float32, device=x.device) if initial_state is None
         else initial_state.float())
    chunk_decay = torch.exp(cum[:, :, -1, :])                 # [b, nc, N]
    starts = []
    for c in range(nc):
        starts.append(h)
        h = h * chunk_decay[:, c, :, None, None] + states[:, c]
    h0 = torch.stack(starts, dim=1)                           # [b, nc, N, P, Sd] state at chunk start
    # ---- carried state contribution: exp(cum[t]) C_t . h_c
    hg = h0.view(b, nc, G, rep * P, Sd)
    off = _group_mm(Cc.permute(0, 1, 3, 2, 4), hg.transpose(-1, -2), lowp)            # [b, nc, G, L, rep*P]
    off = off.permute(0, 1, 3, 2, 4).reshape(b, nc, L, N, P)
    y = y + off * torch.exp(cum)[..., None]
    y = y + D.float()[None, None, None, :, None] * xc
    y = y.reshape(b, nc * L, N, P)[:, :S]
    if pad:
        # padded steps have dt = 0: decay 1, no input, so ``h`` already is the state after the last real token
        pass
    return y.to(dtype), h


def _chunk_scan_kernels(x, pad, dtc, cum, Bc, Cc, D, initial_state, b, S, nc, L, N, P, G, Sd):
    """The CUDA composition of :func:`ssd_chunk_scan`: the element-wise passes are two kernels (:class:`_ScanPrep`,
    :class:`_ScanCombine`), the L x L part is :class:`_IntraChunk`, every product is the batched tcgen05 GEMM
    (:func:`lm_engine_b200.ops.gemm.bmm`), the recurrence over chunk boundaries is :class:`_BoundaryScan`; only
    per-(token, head) scalars (decays, their cumulative sums) stay PyTorch ops."""
    rep = N // G
    xb = torch.nn.functional.pad(x, (0, 0, 0, 0, 0, pad)) if pad else x
    xc = xb.reshape(b, nc, L, N, P)
    tail = torch.exp(cum[:, :, -1:, :] - cum)                 # [b, nc, L, N]
    xh, xwT = _ScanPrep.apply(xc, dtc, tail)
    # intra-chunk
    Cg = Cc.permute(0, 1, 3, 2, 4).to(torch.bfloat16).contiguous()        # [b, nc, G, L, Sd]
    Bg = Bc.permute(0, 1, 3, 2, 4).to(torch.bfloat16).contiguous()
    from .gemm import bmm

    CB = bmm(Cg.view(b * nc * G, L, Sd), Bg.view(b * nc * G, L, Sd),
             out_dtype=torch.bfloat16).view(b, nc, G, L, L)              # C B^T per (batch, chunk, group)
    yin = _IntraChunk.apply(CB, cum.permute(0, 1, 3, 2), xh)             # [b, nc, N, L, P] fp32
    # chunk summaries S_c [b, nc, G, rep*P, Sd] (the heads of a group folded into the GEMM's M dimension);
    # B_c is [L, Sd] = [K, N]: the MN-major operand
    states = bmm(xwT.view(b * nc * G, rep * P, L), Bg.view(b * nc * G, L, Sd), b_mn=True).view(b, nc, N, P, Sd)
    chunk_decay = torch.exp(cum[:, :, -1, :])                 # [b, nc, N]
    h0, h = _BoundaryScan.apply(states, chunk_decay, initial_state)      # [b, nc, N, P, Sd] bf16, [b, N, P, Sd]
    # carried-state contribution C_t . h_c: the states [rep*P, Sd] are the K-major B operand as they are
    off = bmm(Cg.view(b * nc * G, L, Sd), h0.view(b * nc * G, rep * P, Sd)).view(b, nc, G, L, rep * P)
    y = _ScanCombine.apply(yin, off, torch.exp(cum), D.float(), xc)
    return y.reshape(b, nc * L, N, P)[:, :S], h


def ssd_context_parallel_initial_state(final_zero_init: torch.Tensor, total_decay: torch.Tensor, group) -> torch.Tensor:
    """State entering this rank's sequence shard.  ``final_zero_init [b, N, P, Sd]``: the shard's final state when
    started from zero; ``total_decay [b, N]``: ``exp(A sum dt)`` over the shard.  The entering state of rank r is
    ``sum_{j<r} (prod_{j<i<r} decay_i) final_j`` (lm_engine/modeling_utils/sequence_mixer_blocks/mamba2/op.py:73-145)."""
    return _CPPrefix.apply(final_zero_init, total_decay, group)


class _CPPrefix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f, d, group):
        world, r = dist.get_world_size(group), dist.get_rank(group)
        fs = [torch.empty_like(f) for _ in range(world)]
        ds = [torch.empty_like(d) for _ in range(world)]
        dist.all_gather(fs, f.contiguous(), group=group)
        dist.all_gather(ds, d.contiguous(), group=group)
        h = torch.zeros_like(f)
        for j in range(r):
            h = h * ds[j][..., None, None] + fs[j]
        ctx.group = group
        ctx.save_for_backward(torch.stack(fs), torch.stack(ds))
        return h

    @staticmethod
    def backward(ctx, g):
        fs, ds = ctx.saved_tensors
        group = ctx.group
        world, r = dist.get_world_size(group), dist.get_rank(group)
        # every rank needs d(loss_i)/d(f_r), d(loss_i)/d(d_r) for the later ranks i > r: exchange the incoming grads
        gs = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(gs, g.contiguous(), group=group)
        gf = torch.zeros_like(g)
        gd = torch.zeros_like(ds[0])
        for i in range(r + 1, world):
            # h_i = sum_{j<i} (prod_{j<k<i} d_k) f_j
            coef = torch.ones_like(ds[0])
            for k in range(r + 1, i):
                coef = coef * ds[k]
            gf = gf + gs[i] * coef[..., None, None]
            # dependence on d_r (r >= 1 contributes to h_i through the terms with j < r)
            if r >= 1:
                prefix = torch.zeros_like(g)
                for j in range(r):
                    prefix = prefix * ds[j][..., None, None] + fs[j]   # = h_r
                gd = gd + (gs[i] * prefix).sum((-1, -2)) * coef
        return gf, gd, None
