"""Pipeline parallelism: schedule generation, a lock-step executor over point-to-point messages, and the optimizer step
across stages (role of lm_engine/distributed.py:88-117,448-512, lm_engine/parallel/pipeline_parallel.py:11-21 and
lm_engine/train.py:49-132, which delegate to ``torch.distributed.pipelining``).

Design
------
* Stage ``s`` lives on pipeline rank ``s % pp`` (round robin), so a rank owns ``V = num_stages / pp`` model chunks.
* A schedule is first written as one ordered action list per rank (``F`` = forward of a chunk on a micro-batch, ``B`` =
  its backward).  The lists are then *simulated* into a global timetable of ticks: in a tick every rank runs at most
  one action, and an action runs only when the action that produces its input ran in an earlier tick.  Every rank
  derives the same timetable from ``(schedule, pp, V, micro-batches)`` with no communication.
* After each tick, every rank posts ONE batched group of sends / receives: the output of its own action and whatever
  its neighbours produced for it in that tick.  Because the groups of all ranks are derived from the same timetable,
  every send has its matching receive in the peer's group of the same tick, which makes the exchange deadlock-free for
  every schedule (no rank can sit in a send while its peer sits in another send).  Received tensors are parked until
  the tick that consumes them.
* Micro-batch gradients accumulate in the sharded engine exactly as with gradient accumulation; the global gradient
  norm is summed over local chunks, then over the pipeline group, and each chunk's fused clip + AdamW runs with it.

Schedules: ``GPipe`` (all forwards, then all backwards), ``1F1B``, ``Interleaved1F1B`` / ``FlexibleInterleaved1F1B``
(depth-first over chunks in groups of ``pp`` micro-batches), ``LoopedBFS`` (breadth-first over chunks).
``InterleavedZeroBubble`` is accepted and runs the interleaved 1F1B order: weight-gradient GEMMs here write straight
into the sharded gradient buffers from their epilogue, so they are not split from the input-gradient pass.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..logging_utils.metrics import MetricsTrackingDict
from .manager import ProcessGroupManager

F, B = "F", "B"


@dataclass(frozen=True)
class Action:
    kind: str      # "F" | "B"
    stage: int     # global stage id
    microbatch: int


# ---------------------------------------------------------------------------------------------------- rank orders
def _order_gpipe(rank: int, pp: int, V: int, M: int) -> list[Action]:
    stages = [rank + i * pp for i in range(V)]
    fwd = [Action(F, s, m) for s in stages for m in range(M)]
    bwd = [Action(B, s, m) for s in reversed(stages) for m in range(M)]
    return fwd + bwd


def _order_1f1b(rank: int, pp: int, V: int, M: int) -> list[Action]:
    assert V == 1, "1F1B runs one stage per rank; use Interleaved1F1B for more"
    warm = min(pp - rank - 1, M)
    out = [Action(F, rank, m) for m in range(warm)]
    f, b = warm, 0
    while f < M:
        out.append(Action(F, rank, f))
        out.append(Action(B, rank, b))
        f, b = f + 1, b + 1
    out.extend(Action(B, rank, m) for m in range(b, M))
    return out


def _order_interleaved(rank: int, pp: int, V: int, M: int) -> list[Action]:
    """Depth-first interleaving: micro-batches advance in groups of ``pp`` through chunk 0, 1, ... of this rank."""
    if V == 1:
        return _order_1f1b(rank, pp, V, M)
    group = pp if M % pp == 0 else M
    total = M * V

    def nth(k: int, forward: bool) -> tuple[int, int]:
        g, r = divmod(k, group * V)
        chunk, j = divmod(r, group)
        if not forward:
            chunk = V - 1 - chunk
        return rank + chunk * pp, g * group + j

    warm = min((pp - rank - 1) * 2 + (V - 1) * group, total)
    out = [Action(F, *nth(k, True)) for k in range(warm)]
    f, b = warm, 0
    while f < total:
        out.append(Action(F, *nth(f, True)))
        out.append(Action(B, *nth(b, False)))
        f, b = f + 1, b + 1
    out.extend(Action(B, *nth(k, False)) for k in range(b, total))
    return out


_ORDERS = {
    "GPipe": _order_gpipe, "ScheduleGPipe": _order_gpipe,
    "1F1B": _order_1f1b, "Schedule1F1B": _order_1f1b,
    "Interleaved1F1B": _order_interleaved, "ScheduleInterleaved1F1B": _order_interleaved,
    "FlexibleInterleaved1F1B": _order_interleaved, "ScheduleFlexibleInterleaved1F1B": _order_interleaved,
    "InterleavedZeroBubble": _order_interleaved, "ScheduleInterleavedZeroBubble": _order_interleaved,
    "LoopedBFS": _order_gpipe, "ScheduleLoopedBFS": _order_gpipe,
}


def rank_orders(schedule: str, pp: int, num_stages: int, num_microbatches: int) -> list[list[Action]]:
    if schedule not in _ORDERS:
        raise ValueError(f"unknown pipeline schedule ({schedule}); known: {sorted(_ORDERS)}")
    assert num_stages % pp == 0
    V = num_stages // pp
    if _ORDERS[schedule] is _order_1f1b and V > 1:
        raise ValueError("1F1B needs num_pipeline_stages == pipeline_parallel_world_size")
    return [_ORDERS[schedule](r, pp, V, num_microbatches) for r in range(pp)]


def build_timetable(orders: list[list[Action]], num_stages: int) -> list[list[Action | None]]:
    """Simulates the per-rank orders into ticks.  ``timetable[t][r]`` is the action of rank ``r`` in tick ``t``."""
    pp = len(orders)
    cursor = [0] * pp
    done: dict[Action, int] = {}
    table: list[list[Action | None]] = []
    remaining = sum(len(o) for o in orders)
    while remaining:
        tick: list[Action | None] = [None] * pp
        for r in range(pp):
            if cursor[r] == len(orders[r]):
                continue
            a = orders[r][cursor[r]]
            if a.kind == F:
                dep = Action(F, a.stage - 1, a.microbatch) if a.stage > 0 else None
            elif a.stage == num_stages - 1:
                dep = Action(F, a.stage, a.microbatch)
            else:
                dep = Action(B, a.stage + 1, a.microbatch)
            own_forward = a.kind == F or Action(F, a.stage, a.microbatch) in done
            if (dep is None or dep in done) and own_forward:
                tick[r] = a
        if all(a is None for a in tick):
            raise RuntimeError("pipeline schedule deadlocks: no rank can make progress")
        for r, a in enumerate(tick):
            if a is not None:
                done[a] = len(table)
                cursor[r] += 1
                remaining -= 1
        table.append(tick)
    return table


def bubble_fraction(table: list[list[Action | None]]) -> float:
    """Idle share of the timetable with a backward costing twice a forward."""
    cost = {F: 1.0, B: 2.0}
    pp = len(table[0])
    busy = sum(cost[a.kind] for tick in table for a in tick if a is not None)
    span = sum(max((cost[a.kind] for a in tick if a is not None), default=0.0) for tick in table)
    return 1.0 - busy / (span * pp)


# ---------------------------------------------------------------------------------------------------- executor
class PipelineSchedule:
    """Executes one optimizer step's worth of micro-batches through the local chunks of this pipeline rank."""

    def __init__(self, model_container, schedule: str, num_stages: int, num_microbatches: int, micro_batch_size: int,
                 sequence_length: int, dtype: torch.dtype, has_aux_loss: bool) -> None:
        self.group = ProcessGroupManager.get_pipeline_parallel_group()
        self.pp = ProcessGroupManager.get_pipeline_parallel_world_size()
        self.rank = ProcessGroupManager.get_pipeline_parallel_rank()
        self.num_stages, self.M = num_stages, num_microbatches
        self.micro_batch_size, self.sequence_length = micro_batch_size, sequence_length
        self.dtype, self.has_aux_loss = dtype, has_aux_loss
        self.schedule_name = schedule
        self.chunks = {w.pipeline_stage_id: w for w in model_container}
        assert sorted(self.chunks) == [self.rank + i * self.pp for i in range(num_stages // self.pp)]
        self.table = build_timetable(rank_orders(schedule, self.pp, num_stages, num_microbatches), num_stages)
        # global ranks of the pipeline group, indexed by pipeline rank
        self.global_ranks = (dist.get_process_group_ranks(self.group) if self.group is not None
                             else [dist.get_rank() if dist.is_initialized() else 0])
        for w in model_container:
            if w.engine is not None:
                w.engine.pipeline_mode = True

    # -------------------------------------------------------------- helpers
    def _device(self) -> torch.device:
        w = next(iter(self.chunks.values()))
        return w.engine.device if w.engine is not None else next(w.model.parameters()).device

    def _hidden_like(self, stage: int) -> torch.Tensor:
        w = next(iter(self.chunks.values()))
        return w.model.get_dummy_intermediate_tensor(self.micro_batch_size, self.sequence_length, self.dtype,
                                                     self._device())

    def _message(self, a: Action) -> tuple[int, int] | None:
        """(source stage, destination stage) of the message produced by ``a``; None when nothing is sent."""
        if a.kind == F:
            return (a.stage, a.stage + 1) if a.stage < self.num_stages - 1 else None
        return (a.stage, a.stage - 1) if a.stage > 0 else None

    def _exchange(self, tick: list[Action | None], produced: dict, inbox: dict, keep: list) -> None:
        ops, recvs = [], []
        for r, a in enumerate(tick):   # canonical order: by producing rank
            if a is None:
                continue
            msg = self._message(a)
            if msg is None:
                continue
            src, dst = msg
            src_rank, dst_rank = src % self.pp, dst % self.pp
            key = (a.kind, dst, a.microbatch)
            if src_rank == self.rank and dst_rank == self.rank:
                inbox[key] = produced.pop((a.kind, src, a.microbatch))   # hand-off between two local chunks
                continue
            if src_rank == self.rank:
                tensors = produced.pop((a.kind, src, a.microbatch))
                for t in tensors:
                    ops.append(dist.P2POp(dist.isend, t, self.global_ranks[dst_rank], group=self.group))
                keep.append(tensors)
            elif dst_rank == self.rank:
                bufs = [self._hidden_like(dst)]
                if self.has_aux_loss:
                    bufs.append(torch.empty(1, dtype=torch.float32, device=self._device()))
                for t in bufs:
                    ops.append(dist.P2POp(dist.irecv, t, self.global_ranks[src_rank], group=self.group))
                recvs.append((key, bufs))
        if ops:
            for work in dist.batch_isend_irecv(ops):
                work.wait()
        for key, bufs in recvs:
            inbox[key] = bufs

    # -------------------------------------------------------------- one step
    def step(self, batch: torch.Tensor | None) -> torch.Tensor | None:
        """Runs all micro-batches.  ``batch`` is ``[micro_batch_size * M, sequence_length + 1]`` token ids (needed by
        the first and the last stage).  Returns the summed (already ``1/M``-weighted) loss dict on the rank that owns
        the last stage, else None."""
        M = self.M
        micro = list(batch.chunk(M, dim=0)) if batch is not None else [None] * M
        produced: dict = {}   # (kind, stage, mb) -> tensors to send
        inbox: dict = {}      # (kind, dst stage, mb) -> received tensors
        saved: dict = {}      # (stage, mb) -> (inputs requiring grad, outputs)
        keep: list = []
        totals: dict[str, torch.Tensor] = {}
        for tick in self.table:
            a = tick[self.rank]
            if a is not None:
                w = self.chunks[a.stage]
                first, last = a.stage == 0, a.stage == self.num_stages - 1
                if a.kind == F:
                    if first:
                        hidden_in, aux_in = None, 0
                    else:
                        got = inbox.pop((F, a.stage, a.microbatch))
                        hidden_in = got[0].detach().requires_grad_(True)
                        aux_in = got[1].detach().requires_grad_(True) if self.has_aux_loss else 0
                    out = w.forward_pipeline_stage(micro[a.microbatch], hidden_in, aux_in)
                    if last:
                        loss = out["loss"] / M
                        saved[(a.stage, a.microbatch)] = ([hidden_in, aux_in], [loss])
                        with torch.no_grad():
                            for k, v in out.items():
                                if isinstance(v, torch.Tensor):
                                    totals[k] = totals.get(k, 0) + v.detach() / M
                    else:
                        hidden, aux = out
                        outs = [hidden]
                        send = [hidden.detach()]
                        if self.has_aux_loss:
                            aux = aux if isinstance(aux, torch.Tensor) else hidden.new_zeros(1, dtype=torch.float32)
                            aux = aux.reshape(1).float()
                            if aux.requires_grad:
                                outs.append(aux)
                            send.append(aux.detach().contiguous())
                        saved[(a.stage, a.microbatch)] = ([hidden_in, aux_in], outs)
                        produced[(F, a.stage, a.microbatch)] = [t.contiguous() for t in send]
                else:
                    inputs, outs = saved.pop((a.stage, a.microbatch))
                    if last:
                        outs[0].backward()
                    else:
                        got = inbox.pop((B, a.stage, a.microbatch))
                        grads = [got[0]] + ([got[1]] if len(outs) > 1 else [])
                        torch.autograd.backward(outs, grads)
                    if not first:
                        hidden_in, aux_in = inputs
                        send = [hidden_in.grad if hidden_in.grad is not None else torch.zeros_like(hidden_in)]
                        if self.has_aux_loss:
                            g = aux_in.grad if isinstance(aux_in, torch.Tensor) and aux_in.grad is not None else \
                                torch.zeros(1, dtype=torch.float32, device=hidden_in.device)
                            send.append(g)
                        produced[(B, a.stage, a.microbatch)] = [t.contiguous() for t in send]
            self._exchange(tick, produced, inbox, keep)
        assert not inbox and not saved and not produced, "pipeline step ended with undelivered work"
        return totals or None


# ---------------------------------------------------------------------------------------------------- wiring
def build_pipeline_schedule(args, model_container) -> PipelineSchedule:
    d = args.distributed_args
    tp = args.training_parameters
    from ..utils import string_to_torch_dtype

    dtype_name = args.mixed_precision_args.dtype
    dtype = torch.bfloat16 if dtype_name == "fp8" else string_to_torch_dtype(dtype_name)
    w = model_container[0]
    has_aux = any(b.mlp_type == "MoE" for b in w.config.mlp_blocks)
    seq = args.datasets[0].class_args.get("sequence_length")
    name = d.pipeline_parallel_schedule
    if name in ("1F1B", "Schedule1F1B"):
        assert tp.gradient_accumulation_steps % d.num_pipeline_stages == 0, (
            "1F1B needs gradient_accumulation_steps to be a multiple of num_pipeline_stages")
    return PipelineSchedule(model_container, name, d.num_pipeline_stages, tp.gradient_accumulation_steps,
                            tp.micro_batch_size, seq, dtype, has_aux)


def pipeline_train_step(model_container, pipeline_schedule: PipelineSchedule, optimizer_container,
                        lr_scheduler_container, train_dataloader, gradient_accumulation_steps: int,
                        gradient_clipping: float | None, micro_batch_size: int,
                        sequence_length: int) -> MetricsTrackingDict:
    """One optimizer step through the pipeline (lm_engine/train.py:49-132)."""
    from ..parallel.tensor_parallel import broadcast_tensor_parallel_input
    from ..train_utils import all_reduce_metrics_tracker

    optimizer_container.zero_grad()
    batch = next(train_dataloader) if ProcessGroupManager.is_tensor_parallel_first_rank() else None
    tokens = batch["text"] if isinstance(batch, dict) else batch
    tokens = broadcast_tensor_parallel_input(tokens, (micro_batch_size * gradient_accumulation_steps,
                                                      sequence_length + 1))
    totals = pipeline_schedule.step(tokens)

    # global gradient norm: local chunks -> pipeline group -> every chunk steps with the same clip coefficient
    engines = [w.engine for w in model_container]
    total = None
    for e in engines:
        s = e.local_sumsq()
        total = s.clone() if total is None else total + s
    group = ProcessGroupManager.get_pipeline_parallel_group()
    if group is not None:
        dist.all_reduce(total, group=group)
    grad_norm = None
    for opt in optimizer_container:
        opt.max_grad_norm = gradient_clipping
        grad_norm = opt.step(total_sumsq=total)
    lr_scheduler_container.step()

    metrics = MetricsTrackingDict({})
    if totals is not None:
        with torch.no_grad():
            metrics = metrics + totals
            metrics["grad_norm"] = grad_norm.reshape(()) if gradient_clipping is not None else 0.0
            metrics = all_reduce_metrics_tracker(metrics)
    return metrics
