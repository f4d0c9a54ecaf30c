"""Expert-parallel token exchange on peer memory: tokens travel to the ranks that own their experts and back through
kernels that store to / load from the peers' symmetric-memory slabs over NVLink.  No library collective, no host
round trip (the per-expert counts never leave the devices), no per-expert Python work.

The reference keeps all experts on every rank (lm_engine/modeling_utils/mlp_blocks/moe/module.py:276-291); the usual
expert-parallel extension of that design is ``all_to_all`` (counts) -> host split sizes -> ``all_to_all`` (rows) ->
experts -> ``all_to_all`` back, which this engine also has as its portable path (``MoE._expert_parallel``).

One layer call (csrc/kernels/ep_exchange.cu documents the flags):

* every rank derives the padded per-expert row layout of ITS tokens with the counting-sort kernels, publishes its
  counts to all peers, and computes - from the same table on every rank - where its rows go inside each owner's slab;
* ``_Dispatch``: the source stages its rows in symmetric memory and stores one 8-byte table entry per assignment at
  the owner; the owner waits for the arrival flags and pulls the rows of its tiles into a private buffer (rows
  without an entry - the tail of an expert's last tile - become zero);
* the grouped tcgen05 GEMMs run on the owner's rows exactly as without expert parallelism;
* ``_Collect``: the owner publishes its output slab (the last GEMM wrote into it), the sources pull their rows back;
  the router-weighted sum is the ordinary combine kernel on the local rows.

All row traffic is pulled with peer loads (scattered peer stores of rows measured at 0.47 of the peer-copy rate,
peer loads at 0.8).  The backward pass mirrors the forward pass on a second set of buffers.  An owner's layout holds
``capacity_factor * tokens * top_k`` rows.  The default factor is the group size, the worst case (every token of every
rank routed to one owner), so nothing can overflow; no kernel touches rows of tiles without an expert, so the unused
capacity costs address space and allocator memory, not time.  ``LME_EP_CAPACITY_FACTOR`` lowers it (a router in
its first steps was seen to send more than twice the mean to one of four owners): overflow is then detected on the
device (every rank sees it in the same table), the overflowing rows are dropped and the status word makes the
training loop raise at the end of the step.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.moe import TILE_ROWS, GroupLayout, combine_tokens

_BUFFERS = ("x_stage", "x_table", "y_out", "dy_stage", "dy_table", "dx_out", "counts", "pad_f", "pad_b")
_CONTEXTS: dict[tuple, "RankBuffers"] = {}


def _ptr_array(ptrs: list[int]):
    return (ctypes.c_void_p * 8)(*(ptrs + [None] * (8 - len(ptrs))))


class Plan:
    """Routing of one layer call: ``dest [A, 2]`` (owner, row) of this rank's assignments, and the layout of the rows
    this rank receives as an owner (a :class:`GroupLayout` over its local experts)."""

    def __init__(self) -> None:
        self.dest = self.owner_layout = self.rows_own = None
        self.T = self.K = self.seq_f = self.seq_b = 0


class RankBuffers:
    """Everything one rank of the expert-parallel group holds: its slabs, count table and flag blocks, the addresses
    of the peers' copies, and the round counters.  ``tensors[name]`` is the list over ranks of the buffer ``name``
    (``[rank]`` = local memory); in production the others are peer mappings of symmetric memory."""

    def __init__(self, rank: int, world: int, num_experts: int, cap: int, hidden: int,
                 tensors: dict[str, list[torch.Tensor]]) -> None:
        """``tensors``: see :meth:`sizes`."""
        assert world <= 8 and num_experts % world == 0 and cap % TILE_ROWS == 0 and hidden % 8 == 0
        self.rank, self.world, self.E, self.cap, self.H = rank, world, num_experts, cap, hidden
        self.local_experts = num_experts // world
        self.tensors = tensors
        self.arr = {name: _ptr_array([t.data_ptr() for t in tensors[name]]) for name in _BUFFERS}
        for name in _BUFFERS:
            setattr(self, name, tensors[name][rank])
        dev = self.y_out.device
        self.counter = torch.zeros(4, dtype=torch.int32, device=dev)
        self.seq_f = self.seq_b = 0
        self._identity: dict[tuple[int, int], GroupLayout] = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def sizes(cls, world: int, num_experts: int, cap: int, hidden: int, tokens: int, top_k: int
              ) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        words, bf = 32, torch.bfloat16
        return {"x_stage": ((tokens, hidden), bf), "x_table": ((cap, 2), torch.int32), "y_out": ((cap, hidden), bf),
                "dy_stage": ((tokens * top_k, hidden), bf), "dy_table": ((cap, 2), torch.int32),
                "dx_out": ((cap, hidden), bf), "counts": ((world, num_experts), torch.int32),
                "pad_f": ((words,), torch.int32), "pad_b": ((words,), torch.int32)}

    @classmethod
    def symmetric(cls, group, num_experts: int, cap: int, hidden: int, tokens: int, top_k: int,
                  device: torch.device) -> "RankBuffers":
        import torch.distributed._symmetric_memory as symm_mem

        world, rank = dist.get_world_size(group), dist.get_rank(group)
        sizes = cls.sizes(world, num_experts, cap, hidden, tokens, top_k)
        offsets, total = {}, 0
        for name, (shape, dtype) in sizes.items():
            offsets[name] = total
            total += (math.prod(shape) * dtype.itemsize + 255) // 256 * 256
        arena = symm_mem.empty(total, dtype=torch.uint8, device=device)
        arena.zero_()
        handle = symm_mem.rendezvous(arena, group)
        tensors = {name: [handle.get_buffer(r, shape, dtype, offsets[name] // dtype.itemsize) for r in range(world)]
                   for name, (shape, dtype) in sizes.items()}
        self = cls(rank, world, num_experts, cap, hidden, tensors)
        self._arena, self._handle = arena, handle
        _lib.raise_peer_wait_limit()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        return self

    @classmethod
    def emulated(cls, world: int, num_experts: int, cap: int, hidden: int, tokens: int, top_k: int,
                 device) -> list["RankBuffers"]:
        """All ranks of a group on ONE device (plain tensors instead of peer mappings): lets a single GPU run the
        kernels of every rank one phase after the other, so that no wait ever has to spin."""
        sizes = cls.sizes(world, num_experts, cap, hidden, tokens, top_k)
        tensors = {name: [torch.zeros(shape, dtype=dtype, device=device) for _ in range(world)]
                   for name, (shape, dtype) in sizes.items()}
        return [cls(r, world, num_experts, cap, hidden, tensors) for r in range(world)]

    # ------------------------------------------------------------------ phases (each is one or two launches)
    def publish_counts(self, layout: GroupLayout) -> int:
        self.seq_f += 1
        _lib.check(_lib.cuda_lib().lme_ep_publish_counts(layout.freq.data_ptr(), self.arr["counts"], self.arr["pad_f"],
                                                         self.rank, self.world, self.E, self.seq_f,
                                                         _lib.stream_ptr()), "lme_ep_publish_counts")
        _lib.count_launch()
        return self.seq_f

    def make_plan(self, selected: torch.Tensor, layout: GroupLayout, seq: int) -> Plan:
        """After every rank's :meth:`publish_counts` of round ``seq`` (the kernel waits for their flags)."""
        lib, dev = _lib.cuda_lib(), selected.device
        A, Le, ntiles = selected.numel(), self.local_experts, self.cap // TILE_ROWS
        ints = torch.empty(self.E + 3 * Le + ntiles, dtype=torch.int32, device=dev)
        base, k0, kb, rows, tile_group = ints.split([self.E, Le, Le, Le, ntiles])
        dest = torch.empty((A, 2), dtype=torch.int32, device=dev)          # read as 8-byte pairs: own allocation
        _lib.check(lib.lme_ep_bases(self.counts.data_ptr(), self.pad_f.data_ptr(), self.rank, self.world, self.E, seq,
                                    self.cap, base.data_ptr(), k0.data_ptr(), kb.data_ptr(), rows.data_ptr(),
                                    tile_group.data_ptr(), _lib.stream_ptr()), "lme_ep_bases")
        _lib.check(lib.lme_ep_dest(selected.data_ptr(), layout.slot.data_ptr(), layout.k0.data_ptr(), base.data_ptr(),
                                   A, self.E, self.world, self.cap, dest.data_ptr(), _lib.stream_ptr()),
                   "lme_ep_dest")
        _lib.count_launch(2)
        plan = Plan()
        plan.dest, plan.rows_own, plan.seq_f = dest, rows, seq
        plan.T, plan.K = selected.shape
        own = GroupLayout.__new__(GroupLayout)
        own.capacity, own.num_groups, own.k0, own.kb, own.tile_group = self.cap, Le, k0, kb, tile_group
        own.slot = own.dest = None
        # the last expert GEMM and the first one's input-gradient GEMM write straight into the slabs the peers pull from
        own.output_buffer, own.input_grad_buffer = self.y_out, self.dx_out
        plan.owner_layout = own
        return plan

    def _dir(self, forward: bool) -> tuple[str, str, str, str, int]:
        """(staging buffer, row table, output slab, flag block, counter word) of a direction."""
        return (("x_stage", "x_table", "y_out", "pad_f", 0) if forward
                else ("dy_stage", "dy_table", "dx_out", "pad_b", 1))

    def offer(self, src: torch.Tensor, plan: Plan, forward: bool, seq: int) -> None:
        """Source side: stage the rows where the owners can read them, store the table entries, publish arrival."""
        stage, table, _, pad, word = self._dir(forward)
        staged = getattr(self, stage)
        if src.data_ptr() != staged.data_ptr():
            staged.copy_(src)
        _lib.check(_lib.cuda_lib().lme_ep_offer_rows(plan.dest.data_ptr(), self.arr[table], self.arr[pad],
                                                     plan.dest.size(0), self.counter[word:].data_ptr(), self.rank,
                                                     self.world, seq, _lib.stream_ptr()),
                   f"lme_ep_offer_rows A={plan.dest.size(0)}")
        _lib.count_launch()

    def land(self, plan: Plan, forward: bool, seq: int) -> torch.Tensor:
        """Owner side: wait for every source's arrival flag, pull the rows of the used tiles into a private buffer
        (rows of tiles without an expert stay uninitialised; no kernel reads them)."""
        stage, table, _, pad, _ = self._dir(forward)
        lib = _lib.cuda_lib()
        _lib.check(lib.lme_ep_wait(getattr(self, pad).data_ptr(), 0, self.world, seq, _lib.stream_ptr()),
                   "lme_ep_wait")
        rows = torch.empty((self.cap, self.H), dtype=torch.bfloat16, device=self.y_out.device)
        _lib.check(lib.lme_ep_land_rows(self.arr[stage], getattr(self, table).data_ptr(),
                                        plan.owner_layout.tile_group.data_ptr(), rows.data_ptr(), self.cap, self.H,
                                        plan.K if forward else 1, seq, self.world, _lib.stream_ptr()),
                   f"lme_ep_land_rows cap={self.cap} H={self.H}")
        _lib.count_launch(2)
        return rows

    def publish_output(self, rows: torch.Tensor, forward: bool, seq: int) -> None:
        _, _, out, pad, _ = self._dir(forward)
        slab = getattr(self, out)
        if rows.data_ptr() != slab.data_ptr():
            slab.copy_(rows)
        _lib.check(_lib.cuda_lib().lme_ep_signal_done(self.arr[pad], self.rank, self.world, seq, _lib.stream_ptr()),
                   "lme_ep_signal_done")
        _lib.count_launch()

    def pull(self, plan: Plan, reduce: bool, forward: bool, seq: int) -> torch.Tensor:
        """After every owner's :meth:`publish_output` (the wait kernel checks their flags)."""
        _, _, out, pad, _ = self._dir(forward)
        lib = _lib.cuda_lib()
        _lib.check(lib.lme_ep_wait(getattr(self, pad).data_ptr(), 1, self.world, seq, _lib.stream_ptr()),
                   "lme_ep_wait")
        rows = torch.empty((plan.T if reduce else plan.T * plan.K, self.H), dtype=torch.bfloat16,
                           device=self.y_out.device)
        _lib.check(lib.lme_ep_pull_rows(self.arr[out], plan.dest.data_ptr(), rows.data_ptr(), plan.T, plan.K, self.H,
                                        int(reduce), self.world, _lib.stream_ptr()),
                   f"lme_ep_pull_rows T={plan.T} K={plan.K} H={self.H}")
        _lib.count_launch(2)
        return rows

    def identity_layout(self, T: int, K: int) -> GroupLayout:
        """``slot[t, k] = t * K + k``: the pulled rows, one per assignment, seen as a padded layout by the combine
        kernels."""
        if (T, K) not in self._identity:
            lay = GroupLayout.__new__(GroupLayout)
            lay.slot = torch.arange(T * K, dtype=torch.int32, device=self.y_out.device).view(T, K)
            lay.capacity, lay.dest = T * K, None
            # the combine kernel's backward writes the row gradients where the owners will read them
            lay.grad_buffer = self.dy_stage
            self._identity[(T, K)] = lay
        return self._identity[(T, K)]


class _Dispatch(torch.autograd.Function):
    """Tokens ``[T, H]`` -> this owner's padded rows ``[cap, H]`` (of ALL ranks' tokens for its experts); backward:
    the owners publish the row gradients, each source pulls and sums the ``K`` gradients of a token."""

    @staticmethod
    def forward(ctx, x, rk: RankBuffers, plan: Plan):
        rk.offer(x, plan, True, plan.seq_f)
        ctx.rk, ctx.plan = rk, plan
        return rk.land(plan, True, plan.seq_f)

    @staticmethod
    def backward(ctx, dx_pad):
        rk, plan = ctx.rk, ctx.plan
        rk.publish_output(dx_pad, False, plan.seq_b)
        return rk.pull(plan, True, False, plan.seq_b), None, None


class _Collect(torch.autograd.Function):
    """This owner's output rows ``[cap, H]`` -> the rows of this rank's own assignments ``[T * K, H]``, pulled from
    their owners; backward offers the row gradients to the owners."""

    @staticmethod
    def forward(ctx, y_pad, rk: RankBuffers, plan: Plan):
        rk.publish_output(y_pad, True, plan.seq_f)
        ctx.rk, ctx.plan = rk, plan
        return rk.pull(plan, False, True, plan.seq_f)

    @staticmethod
    def backward(ctx, dy_rows):
        rk, plan = ctx.rk, ctx.plan
        rk.seq_b += 1
        plan.seq_b = rk.seq_b
        rk.offer(dy_rows, plan, False, plan.seq_b)
        return rk.land(plan, False, plan.seq_b), None, None


def capacity_rows(assignments: int, local_experts: int, world: int) -> int:
    factor = min(max(float(os.environ.get("LME_EP_CAPACITY_FACTOR", str(world))), 1.0), float(world))
    rows = int(math.ceil(factor * assignments))
    return (rows + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS + local_experts * TILE_ROWS


def enabled() -> bool:
    return os.environ.get("LME_EP_EXCHANGE", "peer") == "peer"


def eligible(x: torch.Tensor, selected: torch.Tensor, num_experts: int, group) -> bool:
    """bf16 rows on CUDA whose count is the same on every rank of the group (fixed-shape batches), at most 1024
    experts and 8 ranks."""
    if not (enabled() and x.is_cuda and x.dtype == torch.bfloat16 and x.size(1) % 8 == 0 and selected.numel() > 0):
        return False
    world = dist.get_world_size(group)
    return world <= 8 and num_experts <= 1024 and num_experts % world == 0


def buffers_for(group, num_experts: int, tokens: int, top_k: int, hidden: int, device: torch.device) -> RankBuffers:
    key = (id(group), num_experts, tokens, top_k, hidden)
    if key not in _CONTEXTS:
        world = dist.get_world_size(group)
        cap = capacity_rows(tokens * top_k, num_experts // world, world)
        _CONTEXTS[key] = RankBuffers.symmetric(group, num_experts, cap, hidden, tokens, top_k, device)
    return _CONTEXTS[key]


def expert_parallel_mlp(x: torch.Tensor, weights: torch.Tensor, selected: torch.Tensor, num_experts: int, group,
                        mlp) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [T, H]``, router ``weights`` / ``selected [T, K]`` -> ``(sum_k w * expert(x) [T, H], counts [E])``;
    ``mlp(x_pad, layout)`` applies this rank's experts to rows in the padded layout."""
    rk = buffers_for(group, num_experts, selected.size(0), selected.size(1), x.size(1), x.device)
    layout = GroupLayout.from_selection(selected, num_experts)
    plan = rk.make_plan(selected.contiguous(), layout, rk.publish_counts(layout))
    y_pad = mlp(_Dispatch.apply(x, rk, plan), plan.owner_layout)
    y_rows = _Collect.apply(y_pad, rk, plan)
    return combine_tokens(y_rows, weights.to(x.dtype), rk.identity_layout(plan.T, plan.K)), layout.freq
