"""ZeRO / FSDP runtime on flat buffers, with block activation checkpointing and a sharded fused AdamW.

One *unit* per decoder block plus one for the embedding and one for the final norm + LM head (the reference wraps
the same modules with ``fully_shard``, lm_engine/distributed.py:303-385).  Per unit:

* ``flat_param``  compute-dtype (bf16) buffer holding every parameter of the unit back to back, ordered by optimizer
  group; module parameters are views into it.  ZeRO-3 keeps only this rank's slice between uses and all-gathers the
  rest into one of three rotating buffers just before the unit runs (the next unit - and the one behind it when the
  next is a lone norm - is prefetched on a side stream by copy engines out of symmetric memory; the first units of a
  step are prefetched right behind the optimizer step).
* ``main_grad``   gradient buffer of the same layout.  The wgrad GEMM epilogue accumulates straight into it (see
  :mod:`lm_engine_b200.ops.gemm`); other parameters' ``.grad`` are folded in by a hook.  After the unit's backward it
  is reduce-scattered on a side stream, overlapped with the backward of the next unit: by ONE kernel of this
  library that reads the peers' buffers over NVLink, averages in fp32, writes the shard and leaves the partial sums
  of squares of the gradient norm (csrc/kernels/reduce_scatter.cu), or by NCCL (HSDP, expert units, ZeRO-0).
* ``master / exp_avg / exp_avg_sq``  fp32 shards, updated by one fused AdamW launch per optimizer group that also
  refreshes the bf16 slice; the squared gradient norm is reduced on the device and the clip coefficient is read by
  the AdamW kernel from device memory, so a step never synchronises with the host.

Stages: 0 = replicate everything (DDP); 1/2 = shard optimizer state and gradients, keep bf16 parameters whole;
3 = shard parameters too.  ``ddp x fsdp`` (HSDP) all-reduces the sharded gradients over the replication group.
"""

from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..parameter import is_parameter_with_mup_learning_rate, is_parameter_with_no_weight_decay
from .manager import ProcessGroupManager

_ALIGN = 128  # elements; keeps every shard / group boundary 256-byte aligned in bf16


def _pad(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class _Slot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: torch.Size
    group: str


@dataclass
class GroupRange:
    name: str          # "normal" | "no_weight_decay" | "mup"
    start: int         # offsets in the (padded) flat buffer
    end: int


class ShardedUnit:
    """Flat storage of the parameters of a list of modules."""

    def __init__(self, name: str, modules: list[nn.Module], prefixes: list[str], device: torch.device,
                 compute_dtype: torch.dtype, grad_dtype: torch.dtype, shard_world: int, shard_rank: int,
                 shard_params: bool, shard_state: bool, use_mup_group: bool, group=None, replica_group=None,
                 param_filter: Callable[[nn.Parameter], bool] | None = None, is_expert: bool = False,
                 state_device: torch.device | None = None) -> None:
        self.name = name
        self.modules = modules
        # group that shards this unit (the data-parallel sharding group; for expert-parallel parameters the ranks
        # that hold the same experts) and the group that replicates it (HSDP)
        self.group, self.replica_group, self.is_expert = group, replica_group, is_expert
        self.children: list[ShardedUnit] = []   # expert-parallel parameters of the same modules
        self.peer_shards = None
        self.grad_post_scale = 1.0
        self.grad_scaled = False
        self.device, self.compute_dtype, self.grad_dtype = device, compute_dtype, grad_dtype
        self.world, self.rank = shard_world, shard_rank
        self.shard_params = shard_params and shard_world > 1
        self.shard_state = shard_state and shard_world > 1
        # ---- layout: parameters ordered by optimizer group so each group is one contiguous range
        named: list[tuple[str, nn.Parameter]] = []
        seen = set()
        for prefix, m in zip(prefixes, modules):
            for n, p in m.named_parameters():
                if id(p) in seen or (param_filter is not None and not param_filter(p)):
                    continue
                seen.add(id(p))
                named.append((f"{prefix}.{n}" if prefix else n, p))

        def group_of(p: nn.Parameter) -> str:
            if is_parameter_with_no_weight_decay(p):
                return "no_weight_decay"
            if use_mup_group and is_parameter_with_mup_learning_rate(p):
                return "mup"
            return "normal"

        order = {"normal": 0, "mup": 1, "no_weight_decay": 2}
        named.sort(key=lambda np_: (order[group_of(np_[1])], np_[0]))
        self.slots: list[_Slot] = []
        self.group_ranges: list[GroupRange] = []
        off = 0
        for gname in ("normal", "mup", "no_weight_decay"):
            start = off
            for n, p in named:
                if group_of(p) != gname:
                    continue
                self.slots.append(_Slot(n, p, off, p.numel(), p.shape, gname))
                off = _pad(off + p.numel(), 8)
            off = _pad(off, _ALIGN)
            if off > start:
                self.group_ranges.append(GroupRange(gname, start, off))
        self.numel = _pad(max(off, _ALIGN), _ALIGN * self.world)
        if self.group_ranges:
            self.group_ranges[-1].end = self.numel
        self.shard_size = self.numel // self.world
        # element ranges of the flat buffer not covered by any parameter (alignment padding)
        self.gaps: list[tuple[int, int]] = []
        cursor = 0
        for sl in sorted(self.slots, key=lambda t: t.offset):
            if sl.offset > cursor:
                self.gaps.append((cursor, sl.offset))
            cursor = sl.offset + sl.numel
        if cursor < self.numel:
            self.gaps.append((cursor, self.numel))
        self.state_lo = self.rank * self.shard_size if self.shard_state else 0
        self.state_hi = self.state_lo + (self.shard_size if self.shard_state else self.numel)
        # ---- storage
        n_state = self.state_hi - self.state_lo
        # optimizer state lives on `state_device` (pinned host memory with cpu_offload, else the compute device)
        sdev = state_device or device
        pin = sdev.type == "cpu" and device.type == "cuda"
        self.master = torch.zeros(n_state, dtype=torch.float32, device=sdev, pin_memory=pin)
        self.exp_avg = torch.zeros(n_state, dtype=torch.float32, device=sdev, pin_memory=pin)
        self.exp_avg_sq = torch.zeros(n_state, dtype=torch.float32, device=sdev, pin_memory=pin)
        self.grad_shard: torch.Tensor | None = None   # reduced gradient of [state_lo, state_hi)
        if self.shard_params:
            self.lp_shard = torch.zeros(self.shard_size, dtype=compute_dtype, device=device)
            self.flat_param: torch.Tensor | None = None
        else:
            self.flat_param = torch.zeros(self.numel, dtype=compute_dtype, device=device)
            self.lp_shard = self.flat_param[self.state_lo:self.state_hi]
        self.main_grad: torch.Tensor | None = None
        self.unsharded = not self.shard_params
        self.ag_event: torch.cuda.Event | None = None
        self.rs_event: torch.cuda.Event | None = None
        self.grad_ready = False
        self.grad_shard_fresh = True   # next reduced gradient overwrites grad_shard instead of accumulating
        self.pending_backward = 0      # forward uses of the current step whose backward has not run yet
        self.keep_unsharded = False    # stay gathered between forward and backward (tied embedding)

    # ------------------------------------------------------------------ parameter views
    def bind_params(self, flat: torch.Tensor) -> None:
        for s in self.slots:
            s.param.data = flat[s.offset:s.offset + s.numel].view(s.shape)

    def bind_grads(self, flat_grad: torch.Tensor) -> None:
        self.main_grad = flat_grad
        for s in self.slots:
            s.param.main_grad = flat_grad[s.offset:s.offset + s.numel].view(s.shape)

    def release_params(self) -> None:
        empty = torch.empty(0, dtype=self.compute_dtype, device=self.device)
        for s in self.slots:
            s.param.data = empty

    def local_group_ranges(self) -> list[GroupRange]:
        """Group ranges intersected with this rank's optimizer-state slice, relative to that slice."""
        out = []
        for g in self.group_ranges:
            lo, hi = max(g.start, self.state_lo), min(g.end, self.state_hi)
            if hi > lo:
                out.append(GroupRange(g.name, lo - self.state_lo, hi - self.state_lo))
        return out


class _RNGState:
    def __init__(self, device: torch.device) -> None:
        self.cpu = torch.get_rng_state()
        self.cuda = torch.cuda.get_rng_state(device) if device.type == "cuda" else None

    def restore(self, device: torch.device) -> None:
        torch.set_rng_state(self.cpu)
        if self.cuda is not None:
            torch.cuda.set_rng_state(self.cuda, device)


class _UnitFunction(torch.autograd.Function):
    """Runs one unit.  Handles (a) parameter gathering before forward / backward, (b) block activation checkpointing
    (forward without graph, recompute in backward), (c) gradient reduction after the unit's backward."""

    @staticmethod
    def forward(ctx, engine: "FSDPEngine", unit: ShardedUnit, fn: Callable, checkpoint: bool, preserve_rng: bool,
                anchor: torch.Tensor, *inputs: torch.Tensor):
        # ``anchor`` is a 1-element leaf that requires grad: it makes autograd call ``backward`` even when no real
        # input does (the embedding unit only sees integer token ids).
        ctx.engine, ctx.unit, ctx.fn, ctx.checkpoint = engine, unit, fn, checkpoint
        engine.pre_forward(unit, training=True)
        if checkpoint:
            ctx.rng = _RNGState(engine.device) if preserve_rng else None
            ctx.save_for_backward(*inputs)
            with torch.no_grad():
                out = fn(*inputs)
        else:
            with torch.enable_grad():
                detached = [t.detach().requires_grad_(t.requires_grad) for t in inputs]
                out = fn(*detached)
            ctx.detached, ctx.out = detached, out
        engine.post_forward(unit, training=True)
        if isinstance(out, torch.Tensor):
            return out.detach() if not checkpoint else out
        return tuple(o.detach() if isinstance(o, torch.Tensor) else o for o in out)

    @staticmethod
    def backward(ctx, *grads):
        engine, unit = ctx.engine, ctx.unit
        engine.pre_backward(unit)
        if ctx.checkpoint:
            inputs = ctx.saved_tensors
            detached = [t.detach().requires_grad_(t.is_floating_point()) for t in inputs]
            if ctx.rng is not None:
                now = _RNGState(engine.device)
                ctx.rng.restore(engine.device)
            with torch.enable_grad():
                out = ctx.fn(*detached)
            if ctx.rng is not None:
                now.restore(engine.device)
        else:
            detached, out = ctx.detached, ctx.out
        outs = (out,) if isinstance(out, torch.Tensor) else tuple(out)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad
                 and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        engine.post_backward(unit)
        return (None, None, None, None, None, None, *[t.grad if t.requires_grad else None for t in detached])


class FSDPEngine:
    """Owns the units of one model (one pipeline stage) and the sharded optimizer state."""

    def __init__(self, model: nn.Module, units: list[tuple[str, list[nn.Module], list[str]]], *, stage: int = 3,
                 compute_dtype: torch.dtype = torch.bfloat16, grad_dtype: torch.dtype | None = None,
                 device: torch.device | None = None, use_mup_group: bool = False,
                 checkpoint_units: set[str] | None = None, preserve_rng: bool = False,
                 init_fn: Callable[[nn.Module], None] | None = None, seed: int = 0,
                 cpu_offload: bool = False) -> None:
        assert stage in (0, 1, 2, 3)
        self.model, self.stage = model, stage
        self.cpu_offload = cpu_offload
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.compute_dtype = compute_dtype
        self.grad_dtype = grad_dtype or compute_dtype
        self.shard_group = ProcessGroupManager.get_sharding_group() if stage > 0 else None
        self.replica_group = (ProcessGroupManager.get_replication_group() if stage > 0
                              else ProcessGroupManager.get_data_parallel_group())
        self.world = dist.get_world_size(self.shard_group) if self.shard_group is not None else 1
        self.rank = dist.get_rank(self.shard_group) if self.shard_group is not None else 0
        self.checkpoint_units = checkpoint_units or set()
        self.preserve_rng = preserve_rng
        self.is_cuda = self.device.type == "cuda"
        # Expert-parallel parameters differ between the ranks of the expert-parallel group, so they are sharded /
        # reduced over the ranks that own the same experts only; they form a child unit of their block.
        self.ep_group = ProcessGroupManager.get_expert_parallel_group()
        self.ep_world = ProcessGroupManager.get_expert_parallel_world_size()
        edp_group = ProcessGroupManager.get_expert_data_parallel_group() if self.ep_world > 1 else None
        edp_world = dist.get_world_size(edp_group) if edp_group is not None else 1
        edp_rank = dist.get_rank(edp_group) if edp_group is not None else 0

        def is_expert_param(p: nn.Parameter) -> bool:
            return self.ep_world > 1 and getattr(p, "ep_shard_dim", None) is not None

        state_device = torch.device("cpu") if cpu_offload else None
        self.units: list[ShardedUnit] = []        # execution order (prefetch neighbours)
        self.all_units: list[ShardedUnit] = []    # + expert children, for everything that walks the state
        for name, modules, prefixes in units:
            u = ShardedUnit(name, modules, prefixes, self.device, compute_dtype, self.grad_dtype, self.world,
                            self.rank, shard_params=stage == 3, shard_state=stage >= 1, use_mup_group=use_mup_group,
                            group=self.shard_group, replica_group=self.replica_group,
                            param_filter=lambda p: not is_expert_param(p), state_device=state_device)
            self.units.append(u)
            self.all_units.append(u)
            if any(is_expert_param(p) for m in modules for p in m.parameters()):
                assert self.replica_group is None or stage == 0, "expert parallel with HSDP is not supported"
                sharded = stage >= 1 and edp_world > 1
                c = ShardedUnit(name + ".experts", modules, prefixes, self.device, compute_dtype, self.grad_dtype,
                                edp_world if sharded else 1, edp_rank if sharded else 0, shard_params=stage == 3,
                                shard_state=stage >= 1, use_mup_group=use_mup_group,
                                group=edp_group if sharded else None,
                                replica_group=edp_group if (not sharded and edp_world > 1) else None,
                                param_filter=is_expert_param, is_expert=True, state_device=state_device)
                # every rank of the expert-parallel group adds the tokens it sent here, each weighted for the mean
                # over its own micro-batch: the mean over all data-parallel ranks needs 1 / ep on top of the
                # average over the ranks that replicate these experts
                c.grad_post_scale = 1.0 / self.ep_world
                u.children.append(c)
                self.all_units.append(c)
        self.by_name = {u.name: u for u in self.all_units}
        covered = {id(s.param) for u in self.all_units for s in u.slots}
        missing = [n for n, p in model.named_parameters() if id(p) not in covered]
        assert not missing, f"parameters not covered by any unit: {missing[:5]}"
        self._materialize(init_fn, seed)
        # rotating buffers for gathered parameters / unreduced gradients of the sharded units
        self._param_pool: dict[int, list[torch.Tensor]] = {}
        self._grad_pool: dict[int, list[torch.Tensor]] = {}
        self._pool_cursor: dict[tuple[str, int], int] = {}
        if self.is_cuda:
            self.ag_stream = torch.cuda.Stream(self.device)
            self.rs_stream = torch.cuda.Stream(self.device)
            if self.world > 1 or self.replica_group is not None:
                import os
                import sys

                sys.modules["lm_engine_b200.ops.gemm"].RESERVED_SMS = int(os.environ.get("LME_COMM_SMS", "0"))
        self._anchor = torch.zeros(1, device=self.device, requires_grad=True)
        self._buffer_events: dict[int, torch.cuda.Event] = {}
        self._fence_word = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._inflight: dict[str, torch.Tensor] = {}
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.sumsq_experts = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=self.device)
        self.step_count = 0
        self.micro_step = 0
        self.pipeline_mode = False   # several micro-batches in flight: reshard / reduce after every pass
        self.post_reduce_hook: Callable[[ShardedUnit], None] | None = None   # optimizer-in-backward
        self._setup_grad_buffers()
        self._install_grad_hooks()
        self.copy_engine_gather = False
        self.copy_engine_reduce = False
        if self.is_cuda and self.world > 1 and self.stage == 3:
            import os

            if os.environ.get("LME_ALLGATHER", "ce") == "ce":
                self._setup_symmetric_shards()
        # Gradient reduce-scatter: "fused" (default) = one kernel of ours per unit that reads the peers' buffers over
        # NVLink, averages, writes the shard and the partial squared norm; "nvls" = the same kernel reading through
        # the switch (multimem.ld_reduce); "ce" = copy-engine pulls + a local sum; "nccl" = the library collective.
        self.reduce_mode = "nccl"
        self.fused_reduce_ctas = self.fused_reduce_tail_ctas = 0
        if self.is_cuda and 1 < self.world <= 8 and self.stage >= 1:
            import os

            mode = os.environ.get("LME_REDUCE_SCATTER", "fused")
            if mode in ("fused", "nvls", "ce"):
                self._setup_symmetric_reduce()
                if self.copy_engine_reduce:
                    self.reduce_mode = mode
                    self.fused_reduce_ctas = int(os.environ.get("LME_RS_CTAS", "48"))
                    self.fused_reduce_tail_ctas = int(os.environ.get("LME_RS_TAIL_CTAS", "296"))
                    self.copy_engine_reduce = mode == "ce"

    # ------------------------------------------------------------------ initialisation
    @torch.no_grad()
    def _materialize(self, init_fn, seed: int) -> None:
        """Gives every unit real storage: parameters are (re)initialised in fp32 into a temporary full buffer, the
        fp32 master slice and the bf16 copy are cut from it."""
        tp_rank = ProcessGroupManager.get_tensor_parallel_rank()
        ep_rank = ProcessGroupManager.get_expert_parallel_rank() if self.ep_world > 1 else 0
        for ui, u in enumerate(self.all_units):
            full = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
            meta = any(s.param.is_meta for s in u.slots)
            old = {id(s.param): s.param.data for s in u.slots} if not meta else {}
            if meta:
                self._replace_meta_parameters(u)
            for s in u.slots:
                view = full[s.offset:s.offset + s.numel].view(s.shape)
                if not meta:
                    view.copy_(old[id(s.param)])
                s.param.data = view
            if meta:
                # keyed by the unit's global name, so that a pipeline split initialises the same weights
                gen_seed = (seed + zlib.crc32(u.name.encode()) + 104729 * tp_rank
                            + (1299709 * ep_rank if u.is_expert else 0)) % (2 ** 63)
                mine = {id(s.param) for s in u.slots}
                devs = [self.device] if self.is_cuda else []
                with torch.random.fork_rng(devices=devs):
                    torch.manual_seed(gen_seed)
                    for m in u.modules:
                        for sub in m.modules():
                            # only modules that directly own a parameter of this unit (a block's expert weights
                            # live in a child unit that is initialised on its own turn)
                            own = [p for p in sub._parameters.values() if p is not None]
                            if hasattr(sub, "reset_parameters") and (not own or any(id(p) in mine for p in own)) \
                                    and (own or not u.is_expert):
                                sub.reset_parameters()
                    if init_fn is not None:
                        init_fn(u)
                self._sync_replicated(u)
            u.master.copy_(full[u.state_lo:u.state_hi])
            if u.shard_params:
                u.lp_shard.copy_(full[u.rank * u.shard_size:(u.rank + 1) * u.shard_size])
                u.release_params()
            else:
                u.flat_param.copy_(full)
                u.bind_params(u.flat_param)
            del full
        # buffers (RoPE tables etc.) that are still on meta
        for mod in self.model.modules():
            for bname, buf in list(mod.named_buffers(recurse=False)):
                if buf.is_meta and hasattr(mod, "reset_parameters"):
                    mod.reset_parameters()
        for mod in self.model.modules():
            for bname, buf in list(mod.named_buffers(recurse=False)):
                if buf.device != self.device and not buf.is_meta:
                    mod._buffers[bname] = buf.to(self.device)

    def _replace_meta_parameters(self, u: ShardedUnit) -> None:
        """Meta parameters cannot adopt real storage: swap each for a fresh ``nn.Parameter`` carrying the same
        markers (attributes) in its owning module."""
        owners: dict[int, list[tuple[nn.Module, str]]] = {}
        for m in u.modules:
            for sub in m.modules():
                for pname, p in sub._parameters.items():
                    if p is not None:
                        owners.setdefault(id(p), []).append((sub, pname))
        for s in u.slots:
            old = s.param
            new = nn.Parameter(torch.empty(0, dtype=self.compute_dtype, device=self.device),
                               requires_grad=old.requires_grad)
            new.__dict__.update(old.__dict__)
            for sub, pname in owners.get(id(old), []):
                sub._parameters[pname] = new
            s.param = new

    def _sync_replicated(self, u: ShardedUnit) -> None:
        """Parameters replicated over the TP group must be identical on all of its ranks after a per-rank init."""
        tp_group = ProcessGroupManager.get_tensor_parallel_group()
        if tp_group is None:
            return
        src = ProcessGroupManager.get_tensor_parallel_first_rank()
        for s in u.slots:
            if getattr(s.param, "tp_shard_dim", None) is None:
                dist.broadcast(s.param.data, src=src, group=tp_group)

    def _setup_grad_buffers(self) -> None:
        for u in self.all_units:
            if u.world == 1 or self.stage == 0:
                # the unreduced buffer is the final gradient
                g = torch.zeros(u.numel, dtype=self.grad_dtype, device=self.device)
                u.bind_grads(g)
                u.grad_shard = g[u.state_lo:u.state_hi]
            else:
                u.grad_shard = torch.zeros(u.shard_size, dtype=self.grad_dtype, device=self.device)
                u.main_grad = None

    def _install_grad_hooks(self) -> None:
        def make_hook():
            def hook(p: nn.Parameter) -> None:
                if p.grad is None:
                    return
                mg = getattr(p, "main_grad", None)
                if mg is not None:
                    if getattr(p, "main_grad_stale", False):
                        mg.copy_(p.grad.view_as(mg))
                        p.main_grad_stale = False
                    else:
                        mg.add_(p.grad.view_as(mg))
                p.grad = None

            return hook

        for u in self.all_units:
            for s in u.slots:
                s.param.register_post_accumulate_grad_hook(make_hook())

    # ------------------------------------------------------------------ symmetric-memory parameter shards
    def _setup_symmetric_shards(self) -> None:
        """Moves the bf16 parameter shards of all units into one symmetric-memory allocation so that every rank can
        read its peers' shards directly.  The parameter all-gather then is ``world`` peer-to-peer copies executed by
        the copy engines over NVLink: no SM is taken from the GEMMs it overlaps with (an NCCL all-gather kernel
        competes with the persistent GEMM CTAs for SMs)."""
        try:
            import torch.distributed._symmetric_memory as symm_mem

            units = [u for u in self.units if u.shard_params]
            total = sum(u.shard_size for u in units)
            arena = symm_mem.empty(total, dtype=self.compute_dtype, device=self.device)
            handle = symm_mem.rendezvous(arena, self.shard_group)
            off = 0
            for u in units:
                mine = arena[off:off + u.shard_size]
                mine.copy_(u.lp_shard)
                u.lp_shard = mine
                u.peer_shards = [handle.get_buffer(r, (u.shard_size,), self.compute_dtype, off)
                                 for r in range(self.world)]
                off += u.shard_size
            self._symm_arena, self._symm_handle = arena, handle
            self.copy_engine_gather = True
            self._cross_rank_fence()
        except Exception as e:  # noqa: BLE001 - symmetric memory unavailable: keep the NCCL all-gather
            import logging

            from ..logging_utils import log_rank_0

            log_rank_0(logging.WARNING, f"symmetric-memory parameter shards unavailable ({e}); using NCCL all-gather")
            self.copy_engine_gather = False

    # ------------------------------------------------------------------ copy-engine gradient reduce-scatter
    def _setup_symmetric_reduce(self) -> None:
        """Gradient buffers of the sharded units live in symmetric memory; a reduce-scatter then is: announce the
        buffer (one-thread kernel writing a sequence number into every peer's pad), per peer wait for its
        announcement (bounded one-thread kernel) and pull this rank's slice of its buffer with a copy engine, then
        one local kernel that sums the slices in fp32, scales and writes / accumulates the gradient shard.  The
        transfer takes no SM from the backward GEMMs it overlaps with."""
        try:
            import ctypes
            import os

            import torch.distributed._symmetric_memory as symm_mem

            self._rs_pad = symm_mem.empty(16, dtype=torch.int32, device=self.device)
            self._rs_pad.zero_()
            handle = symm_mem.rendezvous(self._rs_pad, self.shard_group)
            ptrs = [handle.get_buffer(r, (16,), torch.int32, 0).data_ptr() for r in range(self.world)]
            self._rs_pad_handle = handle
            self._rs_pad_arr = (ctypes.c_void_p * 8)(*(ptrs + [None] * (8 - self.world)))
            self._rs_seq = 0
            self._rs_stage: torch.Tensor | None = None
            self._symm_grad: dict[int, list[torch.Tensor]] = {}
            self._symm_grad_mc: dict[int, int] = {}            # buffer -> multicast address (0: none)
            self._rs_args: dict[tuple[int, int], tuple] = {}   # (buffer, shard size) -> pointer arrays
            self._rs_partials: torch.Tensor | None = None
            self._rs_partial_slot: dict[str, int] = {}
            self._last_reduced_buf: int | None = None
            self.copy_engine_reduce = True
            from ..ops import _lib

            # ranks drift apart by seconds around evaluation, checkpoints and first-step allocations
            _lib.raise_peer_wait_limit()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.shard_group)
        except Exception as e:  # noqa: BLE001 - symmetric memory unavailable: keep the NCCL reduce-scatter
            import logging

            from ..logging_utils import log_rank_0

            log_rank_0(logging.WARNING, f"symmetric-memory gradient buffers unavailable ({e}); using NCCL")
            self.copy_engine_reduce = False

    def _ce_reduce_applies(self, u: ShardedUnit) -> bool:
        """Units whose gradient buffers live in symmetric memory (reduced by our own kernel or by copy engines)."""
        return (self.reduce_mode != "nccl" and u.world > 1 and u.group is self.shard_group
                and u.replica_group is None and not u.is_expert and self.world <= 8)

    def _symmetric_grad_buffer(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty(numel, dtype=dtype, device=self.device)
        handle = symm_mem.rendezvous(buf, self.shard_group)      # collective: every rank allocates in the same order
        self._symm_grad[buf.data_ptr()] = [handle.get_buffer(r, (numel,), dtype, 0) for r in range(self.world)]
        mc = 0
        if self.reduce_mode == "nvls":
            try:
                mc = int(handle.multicast_ptr or 0)
            except Exception:  # noqa: BLE001 - no NVLS mapping on this machine
                mc = 0
        self._symm_grad_mc[buf.data_ptr()] = mc
        self._symm_grad_handles = getattr(self, "_symm_grad_handles", []) + [handle]
        return buf

    def _reduce_scatter_ce(self, u: ShardedUnit, full: torch.Tensor, scale: float) -> None:
        """Runs on the reduction stream."""
        import ctypes

        from ..ops import _lib

        lib, st = _lib.cuda_lib(), _lib.stream_ptr()
        S, world, rank = u.shard_size, self.world, self.rank
        peers = self._symm_grad[full.data_ptr()]
        self._rs_seq += 1
        seq = self._rs_seq
        if self._rs_stage is None or self._rs_stage.size(1) < S or self._rs_stage.dtype != full.dtype:
            cap = max(x.shard_size for x in self.units)
            self._rs_stage = torch.empty((world - 1, cap), dtype=full.dtype, device=self.device)
        _lib.check(lib.lme_gather_signal(self._rs_pad_arr, rank, world, seq, st), "lme_gather_signal")
        srcs = [full[rank * S:(rank + 1) * S]]
        for i in range(1, world):
            p = (rank + i) % world
            _lib.check(lib.lme_gather_wait_peer(self._rs_pad.data_ptr(), p, seq, st), "lme_gather_wait_peer")
            stage = self._rs_stage[i - 1, :S]
            stage.copy_(peers[p][rank * S:(rank + 1) * S], non_blocking=True)
            srcs.append(stage)
        arr = (ctypes.c_void_p * 8)(*([t.data_ptr() for t in srcs] + [None] * (8 - world)))
        _lib.check(lib.lme_reduce_slices(arr, world, u.grad_shard.data_ptr(), S, int(full.dtype == torch.bfloat16),
                                         scale, int(not u.grad_shard_fresh), st), "lme_reduce_slices")
        _lib.count_launch(2)
        u.grad_shard_fresh = False

    def _reduce_scatter_fused(self, u: ShardedUnit, full: torch.Tensor, scale: float) -> None:
        """One launch on the reduction stream: announce this rank's buffer, wait (bounded) for the peers', read this
        rank's slice of every buffer over NVLink, average in fp32, write / accumulate the gradient shard and leave
        the partial sums of squares for the gradient norm."""
        import ctypes

        from ..ops import _lib

        S, world, rank = u.shard_size, self.world, self.rank
        key = (full.data_ptr(), S)
        args = self._rs_args.get(key)
        if args is None:
            peers = self._symm_grad[full.data_ptr()]
            esz = full.element_size()
            srcs = (ctypes.c_void_p * 8)(*([peers[p].data_ptr() + rank * S * esz for p in range(world)]
                                           + [None] * (8 - world)))
            mc = self._symm_grad_mc.get(full.data_ptr(), 0)
            args = self._rs_args[key] = (srcs, (mc + rank * S * esz) if mc else None)
        srcs, mc_src = args
        # The reduction of the unit whose backward runs last (the first unit of the model) has nothing left to hide
        # behind: it gets enough CTAs to run at link rate.  The others share the SMs with the backward GEMMs and
        # have a whole unit's backward of time, so they stay small.
        tail = u is self.units[0]
        ctas = self.fused_reduce_tail_ctas if tail else self.fused_reduce_ctas
        stride = max(self.fused_reduce_tail_ctas, self.fused_reduce_ctas)
        if self._rs_partials is None:
            self._rs_partial_stride = stride
            self._rs_partials = torch.zeros(len(self.all_units) * stride, dtype=torch.float32, device=self.device)
        slot = self._rs_partial_slot.setdefault(u.name, len(self._rs_partial_slot))
        self._rs_seq += 1
        _lib.check(_lib.cuda_lib().lme_reduce_scatter_peers(
            srcs, self._rs_pad_arr, mc_src, rank, world, self._rs_seq, u.grad_shard.data_ptr(), S,
            int(full.dtype == torch.bfloat16), scale, int(not u.grad_shard_fresh),
            self._rs_partials.data_ptr() + slot * stride * 4, ctas, _lib.stream_ptr()), "lme_reduce_scatter_peers")
        _lib.count_launch()
        u.grad_shard_fresh = False

    def _cross_rank_fence(self) -> None:
        """Orders this rank's writes to its parameter shard (optimizer step, checkpoint load) before the peers'
        next reads: a tiny all-reduce on the compute stream; the gather stream waits on the compute stream."""
        if self.copy_engine_gather and self.shard_group is not None:
            dist.all_reduce(self._fence_word, group=self.shard_group)

    # ------------------------------------------------------------------ buffer pools
    def _take(self, pool: dict[int, list[torch.Tensor]], kind: str, u: ShardedUnit, dtype) -> torch.Tensor:
        bufs = pool.setdefault(u.numel, [])
        symmetric = kind == "g" and self._ce_reduce_applies(u)
        # A gradient buffer that the peers read is free again only once the reduction AFTER its own has finished
        # here (see _reduce_grads).  With two buffers the backward pass of unit i - 2 would then wait for the
        # reduction of unit i - 1, which has only just been issued: nothing would overlap.  A third buffer moves
        # that wait one unit back.
        # gathered parameters: the running unit plus up to two prefetched ones (see _prefetch) are live at once
        depth = 3 if kind == "p" else 2
        if symmetric:   # units of a size that occurs once or twice per step never meet that wait: one buffer each
            depth = min(3, sum(1 for x in self.all_units if x.numel == u.numel and self._ce_reduce_applies(x)))
        if len(bufs) < depth:
            if symmetric:
                bufs.append(self._symmetric_grad_buffer(u.numel, dtype))
            else:
                bufs.append(torch.empty(u.numel, dtype=dtype, device=self.device))
            return bufs[-1]
        key = (kind, u.numel)
        i = self._pool_cursor.get(key, 0)
        self._pool_cursor[key] = i + 1
        return bufs[i % depth]

    # ------------------------------------------------------------------ gather / reduce
    def _all_gather(self, u: ShardedUnit, for_graph: bool = False) -> None:
        """Starts the all-gather of ``u`` (side stream on CUDA) unless it is already gathered or in flight.
        ``for_graph``: the gathered weights feed a forward pass whose autograd graph outlives the unit's forward."""
        if u.unsharded or u.name in self._inflight:
            return
        if for_graph and u.name not in self.checkpoint_units:
            # This forward records an autograd graph that lives until the unit's backward, and ops may save views
            # of the gathered weights in it.  A pooled buffer would be overwritten by the next unit's gather in the
            # meantime, so such a gather gets storage of its own (released with the graph).
            buf = torch.empty(u.numel, dtype=self.compute_dtype, device=self.device)
        else:
            buf = self._take(self._param_pool, "p", u, self.compute_dtype)
        if self.is_cuda:
            self.ag_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.ag_stream):
                if self.copy_engine_gather and u.peer_shards is not None:
                    S = u.shard_size
                    for i in range(u.world):   # own shard first, then the peers in a rank-rotated order
                        p = (u.rank + i) % u.world
                        buf[p * S:(p + 1) * S].copy_(u.peer_shards[p], non_blocking=True)
                else:
                    dist.all_gather_into_tensor(buf, u.lp_shard, group=u.group)
                u.ag_event = torch.cuda.Event()
                u.ag_event.record(self.ag_stream)
        else:
            dist.all_gather_into_tensor(buf, u.lp_shard, group=u.group)
        self._inflight[u.name] = buf

    def _wait_gather(self, u: ShardedUnit, for_graph: bool = False) -> None:
        if u.unsharded:
            return
        self._all_gather(u, for_graph)
        buf = self._inflight.pop(u.name)
        if self.is_cuda and u.ag_event is not None:
            torch.cuda.current_stream().wait_event(u.ag_event)
        u.flat_param = buf
        u.bind_params(buf)
        u.unsharded = True

    def _reshard(self, u: ShardedUnit) -> None:
        if not u.shard_params or not u.unsharded:
            return
        u.release_params()
        u.flat_param = None
        u.unsharded = False

    def _neighbour(self, u: ShardedUnit, step: int) -> ShardedUnit | None:
        i = self.units.index(u) + step
        return self.units[i] if 0 <= i < len(self.units) else None

    # ------------------------------------------------------------------ hooks called by _UnitFunction
    @staticmethod
    def _family(u: ShardedUnit | None) -> tuple[ShardedUnit, ...]:
        return () if u is None else (u, *u.children)

    # a unit below this many elements (a lone norm) runs for a few microseconds: the gather of the unit behind it
    # would not be hidden, so prefetching looks one unit further
    _TINY_UNIT = 1 << 20

    def _prefetch(self, u: ShardedUnit, step: int, for_graph: bool) -> None:
        """Starts the gathers of the unit(s) that run after ``u`` (``step`` +1: forward order, -1: backward)."""
        nxt = self._neighbour(u, step)
        for x in self._family(nxt):
            if x.shard_params:
                self._all_gather(x, for_graph)
        if nxt is not None and nxt.numel < self._TINY_UNIT:
            for x in self._family(self._neighbour(nxt, step)):
                if x.shard_params:
                    self._all_gather(x, for_graph)

    def pre_forward(self, u: ShardedUnit, training: bool) -> None:
        for x in self._family(u):
            if training:
                x.pending_backward += 1
            self._wait_gather(x, for_graph=training)
        self._prefetch(u, +1, for_graph=training)

    def post_forward(self, u: ShardedUnit, training: bool) -> None:
        # the last unit's backward starts right after its forward: keep it gathered
        if u.keep_unsharded or (training and u is self.units[-1] and not self.pipeline_mode):
            return
        for x in self._family(u):
            self._reshard(x)

    def pre_backward(self, u: ShardedUnit) -> None:
        for x in self._family(u):
            self._wait_gather(x)
        self._prefetch(u, -1, for_graph=False)
        for x in self._family(u):
            self._bind_grad_buffer(x)

    def _bind_grad_buffer(self, u: ShardedUnit) -> None:
        if u.main_grad is None:
            buf = self._take(self._grad_pool, "g", u, self.grad_dtype)
            # the buffer may still be read by the reduce-scatter of the unit that used it last (two units ago)
            ev = self._buffer_events.get(buf.data_ptr())
            if self.is_cuda and ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            # parameters overwrite on their first gradient write; only the padding between them is cleared
            for lo, hi in u.gaps:
                buf[lo:hi].zero_()
            u.bind_grads(buf)
            for s in u.slots:
                s.param.main_grad_stale = True

    def post_backward(self, u: ShardedUnit) -> None:
        for x in self._family(u):
            x.pending_backward -= 1
            if x.pending_backward > 0 and not self.pipeline_mode:
                continue  # the unit ran more than once in forward (tied embedding / LM head): reduce after the last
            self._reduce_grads(x)
            if not u.keep_unsharded:
                self._reshard(x)

    def _reduce_grads(self, u: ShardedUnit) -> None:
        tp_group = ProcessGroupManager.get_tensor_parallel_group()
        if tp_group is not None:
            for s in u.slots:
                if getattr(s.param, "sequence_parallel_grad", False):
                    dist.all_reduce(s.param.main_grad, group=tp_group)
        if u.world == 1 and u.replica_group is None:
            u.grad_ready = True
            if self.post_reduce_hook is not None and u.pending_backward <= 0:
                self.post_reduce_hook(u)
            return
        full = u.main_grad
        for sl in u.slots:   # parameters that received no gradient in this pass
            if getattr(sl.param, "main_grad_stale", False) and u.world > 1 and self.stage != 0:
                sl.param.main_grad.zero_()
                sl.param.main_grad_stale = False
        avg = dist.ReduceOp.AVG if self.is_cuda else dist.ReduceOp.SUM
        # ranks that hold a copy of these parameters (all data-parallel ranks; for experts, the expert replicas)
        dp_total = u.world * (dist.get_world_size(u.replica_group) if u.replica_group is not None else 1)

        def run() -> None:
            if self.stage == 0 or u.world == 1:
                if u.replica_group is not None:
                    if not self.is_cuda:
                        full.div_(dp_total)
                    dist.all_reduce(full, op=avg, group=u.replica_group)
                return
            if self.is_cuda and full.data_ptr() in getattr(self, "_symm_grad", {}):
                if self.reduce_mode == "ce":
                    self._reduce_scatter_ce(u, full, 1.0 / dp_total)
                else:
                    self._reduce_scatter_fused(u, full, 1.0 / dp_total)
                return
            out = torch.empty(u.shard_size, dtype=full.dtype, device=self.device)
            if self.is_cuda:
                dist.reduce_scatter_tensor(out, full, op=avg, group=u.group)
            else:
                tmp = full / dp_total
                dist.all_reduce(tmp, group=u.group)
                out.copy_(tmp[u.rank * u.shard_size:(u.rank + 1) * u.shard_size])
            if u.replica_group is not None:
                if self.is_cuda:
                    dist.all_reduce(out, op=avg, group=u.replica_group)
                else:
                    dist.all_reduce(out, group=u.replica_group)
            if u.grad_shard_fresh:
                u.grad_shard.copy_(out)
                u.grad_shard_fresh = False
            else:
                u.grad_shard.add_(out)

        if self.is_cuda:
            self.rs_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.rs_stream):
                run()
                u.rs_event = torch.cuda.Event()
                u.rs_event.record(self.rs_stream)
                if full.data_ptr() in getattr(self, "_symm_grad", {}):
                    # Peers pull from this buffer too: it is free for new gradients once the NEXT reduction has
                    # finished here (that one waited for every peer's announcement, which a peer sends after its
                    # own pulls of this reduction, in stream order).  The step boundary is covered by the fence.
                    if self._last_reduced_buf is not None:
                        self._buffer_events[self._last_reduced_buf] = u.rs_event
                    self._last_reduced_buf = full.data_ptr()
                else:
                    self._buffer_events[full.data_ptr()] = u.rs_event
                if self.post_reduce_hook is not None:
                    self.post_reduce_hook(u)       # optimizer step of this unit, behind its reduction
        else:
            run()
            if self.post_reduce_hook is not None:
                self.post_reduce_hook(u)
        if self.stage != 0 and u.world > 1:
            u.main_grad = None
            for s in u.slots:
                s.param.main_grad = None
        u.grad_ready = True

    # ------------------------------------------------------------------ public API
    def run_unit(self, name: str, fn: Callable, *inputs: torch.Tensor):
        """Executes ``fn(*inputs)`` (the forward of the modules of unit ``name``) under the engine."""
        u = self.by_name[name]
        if not torch.is_grad_enabled():
            self.pre_forward(u, training=False)
            out = fn(*inputs)
            self.post_forward(u, training=False)
            return out
        return _UnitFunction.apply(self, u, fn, name in self.checkpoint_units, self.preserve_rng, self._anchor,
                                   *inputs)

    def zero_grad(self) -> None:
        """Starts a new accumulation window.  Persistent gradient buffers (single shard / ZeRO-0) are not cleared:
        every parameter is flagged so that its first gradient write of the step overwrites instead of accumulating;
        parameters that received no gradient are cleared in :meth:`finish_backward`."""
        for u in self.all_units:
            lazy = u.world == 1 or self.stage == 0
            u.grad_scaled = False
            if lazy and u.main_grad is not None:
                for s in u.slots:
                    s.param.main_grad_stale = True
            elif u.grad_shard is not None:
                u.grad_shard_fresh = True
            u.grad_ready = False
            u.pending_backward = 0
        self.micro_step = 0

    def finish_backward(self) -> None:
        """Joins the reduction stream; call once after the last ``backward`` of a step."""
        for u in self.all_units:
            for s in u.slots:
                if getattr(s.param, "main_grad_stale", False):
                    mg = getattr(s.param, "main_grad", None)
                    if mg is not None:
                        mg.zero_()
                    s.param.main_grad_stale = False
        if self.is_cuda:
            torch.cuda.current_stream().wait_stream(self.rs_stream)
            torch.cuda.current_stream().wait_stream(self.ag_stream)
        for u in self.all_units:
            if u.grad_shard_fresh and u.main_grad is None and u.grad_shard is not None:
                u.grad_shard.zero_()
                slot = getattr(self, "_rs_partial_slot", {}).get(u.name)
                if slot is not None:
                    c = self._rs_partial_stride
                    self._rs_partials[slot * c:(slot + 1) * c].zero_()
            u.grad_shard_fresh = False if u.main_grad is None else u.grad_shard_fresh
            if u.grad_post_scale != 1.0 and not u.grad_scaled:
                u.grad_shard.mul_(u.grad_post_scale)
                u.grad_scaled = True

    @torch.no_grad()
    def clip_and_step(self, *, lr: float, lr_by_group: dict[str, float] | None = None, betas=(0.9, 0.95),
                      eps: float = 1e-10, weight_decay: float = 0.1, max_grad_norm: float | None = 1.0,
                      extra_sumsq: torch.Tensor | None = None,
                      total_sumsq: torch.Tensor | None = None) -> torch.Tensor:
        """Global-norm clipping + AdamW on every shard.  Returns the (device) pre-clip gradient norm.
        ``total_sumsq`` (from :meth:`local_sumsq` of every pipeline chunk, summed over the pipeline group) replaces
        the norm computation when several engines share one clip coefficient."""
        self.step_count += 1
        if total_sumsq is not None:
            self.sumsq.copy_(total_sumsq)
        else:
            self.local_sumsq(include_pipeline_group=True)
            if extra_sumsq is not None:
                self.sumsq.add_(extra_sumsq)
        ops.clip_coef_(self.sumsq, max_grad_norm, self.grad_norm, self.clip_coef)
        lr_by_group = lr_by_group or {}
        if self.cpu_offload and self.is_cuda:
            self._offloaded_step(lr, lr_by_group, betas, eps, weight_decay)
            self._cross_rank_fence()
            self.prefetch_first_units()
            return self.grad_norm
        refreshes = []
        for u in self.all_units:
            for g in u.local_group_ranges():
                sl = slice(g.start, g.end)
                ops.adamw_step(u.master[sl], u.exp_avg[sl], u.exp_avg_sq[sl], u.grad_shard[sl], u.lp_shard[sl],
                               lr=lr_by_group.get(g.name, lr), betas=betas, eps=eps,
                               weight_decay=0.0 if g.name == "no_weight_decay" else weight_decay,
                               step=self.step_count, gscale=self.clip_coef)
            if self.stage in (1, 2) and u.world > 1:
                # ZeRO-1 / 2 keep whole parameters: refresh them from the updated shards.  Issued asynchronously, so
                # that the gather of one unit runs under the update of the next instead of holding the stream.
                refreshes.append(dist.all_gather_into_tensor(u.flat_param, u.lp_shard.clone(), group=u.group,
                                                             async_op=True))
        for work in refreshes:
            work.wait()
        self._cross_rank_fence()
        self.prefetch_first_units()
        return self.grad_norm

    def _offloaded_step(self, lr, lr_by_group, betas, eps, weight_decay) -> None:
        """``cpu_offload`` (lm_engine/distributed.py:334,343 passes a CPUOffloadPolicy to FSDP-2): the fp32 master
        weights and both moments stay in pinned host memory.  Per unit the reduced gradient shard is copied to the
        host, AdamW runs there, and the refreshed low-precision shard is copied back.  Slow by construction (PCIe
        and host arithmetic); meant for models whose optimizer state does not fit next to the activations."""
        from ..ops.optimizer import adamw_reference

        coef = float(self.clip_coef)                      # one read-back of the clip coefficient per step
        for u in self.all_units:
            g_host = u.grad_shard.to("cpu", non_blocking=False).float()
            for g in u.local_group_ranges():
                sl = slice(g.start, g.end)
                adamw_reference(u.master[sl], u.exp_avg[sl], u.exp_avg_sq[sl], g_host[sl] * coef, None,
                                lr_by_group.get(g.name, lr), betas[0], betas[1], eps,
                                0.0 if g.name == "no_weight_decay" else weight_decay, self.step_count)
            u.lp_shard.copy_(u.master, non_blocking=True)
            if self.stage in (1, 2) and u.world > 1:
                dist.all_gather_into_tensor(u.flat_param, u.lp_shard.clone(), group=u.group)

    def prefetch_first_units(self) -> None:
        """Starts the parameter gathers of the first units of the next forward pass right behind the optimizer step
        (every rank's update is complete after the fence), so that they run under the step's host-side tail
        (metric reduction, read-back, next batch) instead of in front of the first kernel of the next step."""
        if self.stage != 3 or not self.is_cuda or self.world == 1 or self.pipeline_mode or not self.units:
            return
        first = self.units[0]
        for x in self._family(first):
            if x.shard_params:
                self._all_gather(x, for_graph=True)
        self._prefetch(first, +1, for_graph=True)

    @torch.no_grad()
    def local_sumsq(self, include_pipeline_group: bool = False) -> torch.Tensor:
        """Joins the backward pass and returns the squared gradient norm of this engine's parameters (summed over
        the sharding and tensor-parallel groups; over the pipeline group too when asked)."""
        self.finish_backward()
        first = True
        fused = getattr(self, "_rs_partial_slot", {})
        if fused:
            # the reduce-scatter kernels left per-CTA sums of squares of every shard they wrote: one launch adds them
            from ..ops import _lib

            _lib.check(_lib.cuda_lib().lme_sum_partials(self._rs_partials.data_ptr(),
                                                        len(fused) * self._rs_partial_stride,
                                                        self.sumsq.data_ptr(), 0, _lib.stream_ptr()),
                       "lme_sum_partials")
            _lib.count_launch()
            first = False
        for u in self.all_units:
            if not u.is_expert and u.name not in fused:
                ops.sumsq_(u.grad_shard, self.sumsq, accumulate=not first)
                first = False
        experts = [u for u in self.all_units if u.is_expert]
        if experts:
            # distinct experts on every rank of the expert-parallel group; shards over the expert replicas
            for i, u in enumerate(experts):
                ops.sumsq_(u.grad_shard, self.sumsq_experts, accumulate=i > 0)
            if experts[0].group is not None:
                dist.all_reduce(self.sumsq_experts, group=experts[0].group)
            dist.all_reduce(self.sumsq_experts, group=self.ep_group)
        self._reduce_norm(include_pipeline_group)
        return self.sumsq

    def _replicated_grad_views(self) -> list[torch.Tensor]:
        """This rank's pieces of the gradients of parameters that are replicated over the tensor-parallel group."""
        cached = getattr(self, "_rep_views", None)
        if cached is None or cached[0] != [u.grad_shard.data_ptr() for u in self.all_units]:
            views = []
            for u in self.all_units:
                for s in u.slots:
                    if getattr(s.param, "tp_shard_dim", None) is None:
                        lo = max(s.offset, u.state_lo) - u.state_lo
                        hi = min(s.offset + s.numel, u.state_hi) - u.state_lo
                        if hi > lo:
                            views.append(u.grad_shard[lo:hi])
            cached = ([u.grad_shard.data_ptr() for u in self.all_units], views)
            self._rep_views = cached
        return cached[1]

    def _reduce_norm(self, include_pipeline_group: bool = True) -> None:
        """Sum of squares over every group that holds a distinct piece of the model."""
        if self.stage >= 1 and self.shard_group is not None:
            dist.all_reduce(self.sumsq, group=self.shard_group)
        if self.ep_world > 1:
            self.sumsq.add_(self.sumsq_experts)
        tp = ProcessGroupManager.get_tensor_parallel_group()
        if tp is not None:
            # replicated parameters were counted tp times; their share is small and the reference counts DTensor
            # replicas once, so subtract the surplus
            rep = torch.zeros(1, dtype=torch.float32, device=self.device)
            views = self._replicated_grad_views()
            if views:
                # one multi-tensor launch over all replicated pieces (the gradient buffers are allocated once, so
                # the views are too), not a Python loop of reductions per parameter
                rep += torch.stack(torch._foreach_norm(views, 2, dtype=torch.float32)).pow(2).sum()
            if self.stage >= 1 and self.shard_group is not None:
                dist.all_reduce(rep, group=self.shard_group)
            tpw = dist.get_world_size(tp)
            dist.all_reduce(self.sumsq, group=tp)
            self.sumsq.sub_(rep * (tpw - 1))
        pp = ProcessGroupManager.get_pipeline_parallel_group()
        if pp is not None and include_pipeline_group:
            dist.all_reduce(self.sumsq, group=pp)

    # ------------------------------------------------------------------ state access (checkpointing, tests)
    @torch.no_grad()
    def gather_full(self, u: ShardedUnit, which: str = "master") -> torch.Tensor:
        """Full fp32 flat tensor of ``master`` / ``exp_avg`` / ``exp_avg_sq`` / ``grad`` on every rank."""
        t = which if isinstance(which, torch.Tensor) else {
            "master": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq, "grad": u.grad_shard}[which]
        if t.device != self.device:       # offloaded optimizer state
            t = t.to(self.device)
        if not u.shard_state:
            return t.float().clone()
        out = torch.empty(u.numel, dtype=t.dtype, device=self.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=u.group)
        return out.float()

    # ------------------------------------------------------------------ row chunks for sharded checkpoints
    def can_exchange_row_chunks(self, u: ShardedUnit) -> bool:
        """Whether :meth:`row_chunks` applies: state sharded over the data-parallel sharding group and no expert
        parallelism (expert slices keep the gather-based path).  Under tensor parallelism the rows are those of the
        rank's tensor-parallel slice."""
        return u.shard_state and u.group is self.shard_group and not u.is_expert and self.ep_world == 1

    @torch.no_grad()
    def row_chunks(self, u: ShardedUnit, which: str | torch.Tensor = "master") -> dict[str, torch.Tensor]:
        """For every parameter of the unit, this rank's block of rows in the even split over the sharding group
        (rows ``[r * per, (r + 1) * per)`` with ``per = ceil(rows / world)``: the layout of a ``Shard(0)`` DTensor),
        cut out of the flat per-rank state with ONE all-to-all in which every rank sends only what the others'
        blocks overlap with its own flat slice.  A checkpoint save then moves ``numel / world`` elements per rank
        instead of gathering the whole unit on every rank."""
        t = which if isinstance(which, torch.Tensor) else {
            "master": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq, "grad": u.grad_shard}[which]
        if t.device != self.device:
            t = t.to(self.device)
        t = t.float()
        W, S, me = u.world, u.shard_size, u.rank

        def block(sl: _Slot, r: int) -> tuple[int, int]:       # flat element range of rank r's rows of this slot
            n0 = sl.shape[0] if len(sl.shape) > 0 else 1
            row = sl.numel // max(n0, 1)
            per = -(-n0 // W)
            lo, hi = min(r * per, n0), min((r + 1) * per, n0)
            return sl.offset + lo * row, sl.offset + hi * row

        send_parts: list[list[torch.Tensor]] = [[] for _ in range(W)]
        recv_sizes = [0] * W
        layout: list[tuple[_Slot, list[tuple[int, int]]]] = []      # per slot: (source rank, elements) pieces
        for sl in u.slots:
            for r in range(W):
                lo, hi = block(sl, r)
                a, b = max(lo, me * S), min(hi, (me + 1) * S)       # what rank r needs of my slice
                if b > a:
                    send_parts[r].append(t[a - me * S:b - me * S])
            lo, hi = block(sl, me)
            pieces = []
            for q in range(W):
                a, b = max(lo, q * S), min(hi, (q + 1) * S)
                if b > a:
                    pieces.append((q, b - a))
                    recv_sizes[q] += b - a
            layout.append((sl, pieces))
        send_sizes = [sum(p.numel() for p in parts) for parts in send_parts]
        flat_send = (torch.cat([p for parts in send_parts for p in parts]) if sum(send_sizes)
                     else t.new_empty(0))
        flat_recv = t.new_empty(sum(recv_sizes))
        dist.all_to_all_single(flat_recv, flat_send.contiguous(), recv_sizes, send_sizes, group=u.group)
        starts = [sum(recv_sizes[:q]) for q in range(W)]
        cursor = list(starts)
        out: dict[str, torch.Tensor] = {}
        for sl, pieces in layout:
            chunks = []
            for q, n in pieces:
                chunks.append(flat_recv[cursor[q]:cursor[q] + n])
                cursor[q] += n
            n0 = sl.shape[0] if len(sl.shape) > 0 else 1
            per = -(-n0 // W)
            rows = max(min((me + 1) * per, n0) - min(me * per, n0), 0)
            data = torch.cat(chunks) if chunks else flat_recv.new_empty(0)
            out[sl.name] = data.view(rows, *sl.shape[1:]) if len(sl.shape) > 0 else data.view(sl.shape)
        return out

    @torch.no_grad()
    def load_row_chunks(self, u: ShardedUnit, chunks: dict[str, torch.Tensor], which: str = "master") -> None:
        """Inverse of :meth:`row_chunks`: every parameter of the unit arrives as this rank's block of rows (what a
        checkpoint load delivers into the ``Shard(0)`` layout), and ONE all-to-all moves the pieces to the ranks whose
        flat state slices they belong to.  No rank ever holds the whole unit."""
        dst = {"master": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq}[which]
        W, S, me = u.world, u.shard_size, u.rank

        def block(sl: _Slot, r: int) -> tuple[int, int]:
            n0 = sl.shape[0] if len(sl.shape) > 0 else 1
            row = sl.numel // max(n0, 1)
            per = -(-n0 // W)
            lo, hi = min(r * per, n0), min((r + 1) * per, n0)
            return sl.offset + lo * row, sl.offset + hi * row

        send_parts: list[list[torch.Tensor]] = [[] for _ in range(W)]
        recv_plan: list[list[tuple[int, int]]] = [[] for _ in range(W)]    # per source rank: (offset in my slice, n)
        for sl in u.slots:
            lo, hi = block(sl, me)
            mine = chunks[sl.name].to(self.device, torch.float32).reshape(-1)
            assert mine.numel() == hi - lo, (sl.name, mine.numel(), hi - lo)
            for q in range(W):                                   # my rows that lie in rank q's flat slice
                a, b = max(lo, q * S), min(hi, (q + 1) * S)
                if b > a:
                    send_parts[q].append(mine[a - lo:b - lo])
            for r in range(W):                                   # rank r's rows that lie in my flat slice
                lo_r, hi_r = block(sl, r)
                a, b = max(lo_r, me * S), min(hi_r, (me + 1) * S)
                if b > a:
                    recv_plan[r].append((a - me * S, b - a))
        send_sizes = [sum(p.numel() for p in parts) for parts in send_parts]
        recv_sizes = [sum(n for _, n in plan) for plan in recv_plan]
        flat_send = (torch.cat([p for parts in send_parts for p in parts]) if sum(send_sizes)
                     else torch.empty(0, dtype=torch.float32, device=self.device))
        flat_recv = torch.empty(sum(recv_sizes), dtype=torch.float32, device=self.device)
        dist.all_to_all_single(flat_recv, flat_send.contiguous(), recv_sizes, send_sizes, group=u.group)
        local = torch.zeros(u.state_hi - u.state_lo, dtype=torch.float32, device=self.device)
        local.copy_(dst.to(self.device, torch.float32))           # padding past the last parameter keeps its value
        cursor = 0
        for r in range(W):
            for off, n in recv_plan[r]:
                local[off - (u.state_lo - me * S):off - (u.state_lo - me * S) + n].copy_(flat_recv[cursor:cursor + n])
                cursor += n
        dst.copy_(local.to(dst.device, dst.dtype))
        if which == "master":
            if u.shard_params:
                u.lp_shard.copy_(u.master.to(self.device))
            else:
                dist.all_gather_into_tensor(u.flat_param, u.master.to(self.device, u.flat_param.dtype).contiguous(),
                                            group=u.group)
            if self._inflight:
                if self.is_cuda:
                    torch.cuda.synchronize(self.device)
                self._inflight.clear()
            self._cross_rank_fence()

    def _slot_full(self, s: "_Slot", local: torch.Tensor) -> torch.Tensor:
        """Expert-parallel parameters: the tensor over all experts (concatenated over the expert-parallel group)."""
        dim = getattr(s.param, "ep_shard_dim", None)
        if self.ep_world == 1 or dim is None:
            return local
        parts = [torch.empty_like(local) for _ in range(self.ep_world)]
        dist.all_gather(parts, local.contiguous(), group=self.ep_group)
        return torch.cat(parts, dim=dim)

    def _slot_local(self, s: "_Slot", full: torch.Tensor) -> torch.Tensor:
        dim = getattr(s.param, "ep_shard_dim", None)
        if self.ep_world == 1 or dim is None or full.size(dim) == s.shape[dim]:
            return full
        return full.chunk(self.ep_world, dim=dim)[ProcessGroupManager.get_expert_parallel_rank()]

    @torch.no_grad()
    def full_state_dict(self, which: str = "master") -> dict[str, torch.Tensor]:
        out = {}
        for u in self.all_units:
            full = self.gather_full(u, which)
            for s in u.slots:
                out[s.name] = self._slot_full(s, full[s.offset:s.offset + s.numel].view(s.shape).clone())
        return out

    @torch.no_grad()
    def load_full_state_dict(self, sd: dict[str, torch.Tensor], which: str = "master") -> None:
        for u in self.all_units:
            if not any(s.name in sd for s in u.slots):      # the same keys on every rank: no collective is skipped
                continue                                    # on one rank only
            full = self.gather_full(u, which)
            for s in u.slots:
                if s.name in sd:
                    full[s.offset:s.offset + s.numel].copy_(
                        self._slot_local(s, sd[s.name]).reshape(-1).to(full.device))
            piece = full[u.state_lo:u.state_hi]
            {"master": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq}[which].copy_(piece)
            if which == "master":
                if u.shard_params:
                    u.lp_shard.copy_(full[u.rank * u.shard_size:(u.rank + 1) * u.shard_size])
                else:
                    u.flat_param.copy_(full)
        if which == "master":
            # gathers started before the load hold the old weights
            if self._inflight:
                if self.is_cuda:
                    torch.cuda.synchronize(self.device)
                self._inflight.clear()
            self._cross_rank_fence()

    @torch.no_grad()
    def local_piece_from_slots(self, u: ShardedUnit, sd: dict[str, torch.Tensor], local: torch.Tensor) -> torch.Tensor:
        """This rank's state slice of unit ``u`` after replacing the slots named in ``sd`` (full tensors) inside
        the unit-wide tensor whose local slice is ``local`` (used for optimizer state that is not the engine's own)."""
        full = self.gather_full(u, local)
        for s in u.slots:
            if s.name in sd:
                full[s.offset:s.offset + s.numel].copy_(self._slot_local(s, sd[s.name]).reshape(-1).to(full.device))
        return full[u.state_lo:u.state_hi].clone()

    def num_parameters(self) -> int:
        return sum(s.numel for u in self.all_units for s in u.slots)
