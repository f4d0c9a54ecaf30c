"""Process-group manager: one NCCL(+gloo) world, one communicator per axis of :class:`Topology`.

Static getters mirror the reference's ``ProcessGroupManager`` (lm_engine/parallel/manager.py:105-508) including the
``set_dummy_*`` context managers that let a single process pretend to be a given rank (used to build an unsharded
model inside a distributed job and by the tests).  Without ``torchrun`` variables it runs as a 1-rank job with no
process group at all.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from datetime import timedelta
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..accelerator import Accelerator
from ..enums import ContextParallelLoadBalancerMethod
from .topology import Topology

_AXES = ("tp", "pp", "dp", "fsdp", "ddp", "cp", "batch", "ep", "edp")


class _State:
    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self.topology: Topology | None = None
        self.rank = 0
        self.local_rank = 0
        self.groups: dict[str, Any] = {}
        self.cpu_group = None
        self.cp_lb: ContextParallelLoadBalancerMethod | None = None
        self.cp_attention: str = "auto"
        self.async_tp = False
        self.dummy_rank: dict[str, int] = {}
        self.dummy_size: dict[str, int] = {}
        self.meshes: dict[str, Any] = {}
        self.owns_pg = False


_S = _State()


class ProcessGroupManager:
    def __init__(
        self,
        tensor_parallel_world_size: int = 1,
        pipeline_parallel_world_size: int = 1,
        data_parallel_replication_world_size: int | None = None,
        data_parallel_sharding_world_size: int | None = None,
        context_parallel_world_size: int = 1,
        context_parallel_load_balancing_method: ContextParallelLoadBalancerMethod | None = None,
        zero_stage: int = 3,
        timeout_minutes: int | None = None,
        use_async_tensor_parallel: bool = False,
        expert_parallel_world_size: int = 1,
        context_parallel_attention: str = "auto",
    ) -> None:
        _S.reset()
        rank = int(os.environ.get("RANK", "0"))
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        _S.rank, _S.local_rank = rank, local_rank
        _S.cp_lb = context_parallel_load_balancing_method
        # "gathered": K / V exchange inside the attention kernel; "ring": blocks around a ring; "ulysses": head
        # exchange; "auto": ulysses when the heads divide, else gathered when the kernel takes the shapes, else ring
        assert context_parallel_attention in ("auto", "ring", "ulysses", "gathered")
        _S.cp_attention = context_parallel_attention
        _S.async_tp = use_async_tensor_parallel
        Accelerator.set_device(local_rank)
        # optional cap on the SMs NCCL may take while its collectives overlap the persistent GEMM kernels (the GEMMs
        # then leave as many free): LME_COMM_SMS=<n>
        if int(os.environ.get("LME_COMM_SMS", "0")) > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", os.environ["LME_COMM_SMS"])
        if "MASTER_ADDR" in os.environ and not dist.is_initialized():
            backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
            kwargs = {}
            if timeout_minutes is not None:
                kwargs["timeout"] = timedelta(minutes=timeout_minutes)
            if torch.cuda.is_available():
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
            _S.owns_pg = True
        elif dist.is_initialized():
            rank, world = dist.get_rank(), dist.get_world_size()
            _S.rank = rank
        _S.topology = Topology.build(world, tp=tensor_parallel_world_size, pp=pipeline_parallel_world_size,
                                     cp=context_parallel_world_size, ddp=data_parallel_replication_world_size,
                                     fsdp=data_parallel_sharding_world_size, zero_stage=zero_stage,
                                     ep=expert_parallel_world_size)
        if dist.is_initialized() and world > 1:
            # every rank creates every group in the same order (new_group is collective)
            for axis in _AXES:
                for ranks in _S.topology.all_groups(axis):
                    if len(ranks) == 1:
                        continue
                    g = dist.new_group(ranks=ranks)
                    if rank in ranks:
                        _S.groups[axis] = g

    # ------------------------------------------------------------------ generic accessors
    @staticmethod
    def is_initialized() -> bool:
        return _S.topology is not None

    @staticmethod
    def topology() -> Topology:
        if _S.topology is None:
            _S.topology = Topology.build(1)
        return _S.topology

    @staticmethod
    def _size(axis: str) -> int:
        if axis in _S.dummy_size:
            return _S.dummy_size[axis]
        t = ProcessGroupManager.topology()
        return {"tp": t.tp, "pp": t.pp, "dp": t.dp, "fsdp": t.fsdp, "ddp": t.ddp, "cp": t.cp, "batch": t.batch,
                "ep": t.ep, "edp": t.dp // t.ep}[axis]

    @staticmethod
    def _rank(axis: str) -> int:
        if axis in _S.dummy_rank:
            return _S.dummy_rank[axis]
        return ProcessGroupManager.topology().coords(_S.rank)[axis]

    @staticmethod
    def get_group(axis: str):
        """The communicator of ``axis`` for this rank (None when that axis has size 1)."""
        return _S.groups.get(axis)

    @staticmethod
    def get_group_ranks(axis: str) -> list[int]:
        return ProcessGroupManager.topology().group(axis, _S.rank)

    @staticmethod
    @contextmanager
    def _dummy(table: dict[str, int], axis: str, value: int):
        had, old = axis in table, table.get(axis)
        table[axis] = value
        try:
            yield
        finally:
            if had:
                table[axis] = old
            else:
                del table[axis]

    @staticmethod
    def get_global_rank() -> int:
        return _S.rank

    @staticmethod
    def get_local_rank() -> int:
        return _S.local_rank

    @staticmethod
    def get_world_size() -> int:
        return ProcessGroupManager.topology().world_size

    # ------------------------------------------------------------------ tensor parallel
    @staticmethod
    def get_tensor_parallel_group():
        return _S.groups.get("tp")

    @staticmethod
    def get_tensor_parallel_rank() -> int:
        return ProcessGroupManager._rank("tp")

    @staticmethod
    def get_tensor_parallel_world_size() -> int:
        return ProcessGroupManager._size("tp")

    @staticmethod
    def set_dummy_tensor_parallel_rank(rank: int):
        return ProcessGroupManager._dummy(_S.dummy_rank, "tp", rank)

    @staticmethod
    def set_dummy_tensor_parallel_world_size(world_size: int):
        return ProcessGroupManager._dummy(_S.dummy_size, "tp", world_size)

    @staticmethod
    def get_tensor_parallel_first_rank() -> int:
        return ProcessGroupManager.get_group_ranks("tp")[0]

    @staticmethod
    def is_tensor_parallel_enabled() -> bool:
        return ProcessGroupManager.get_tensor_parallel_world_size() > 1

    @staticmethod
    def is_tensor_parallel_first_rank() -> bool:
        return ProcessGroupManager.get_tensor_parallel_rank() == 0

    @staticmethod
    def use_async_tensor_parallel() -> bool:
        return _S.async_tp

    # ------------------------------------------------------------------ pipeline parallel
    @staticmethod
    def get_pipeline_parallel_group():
        return _S.groups.get("pp")

    @staticmethod
    def get_pipeline_parallel_rank() -> int:
        return ProcessGroupManager._rank("pp")

    @staticmethod
    def get_pipeline_parallel_world_size() -> int:
        return ProcessGroupManager._size("pp")

    @staticmethod
    def set_dummy_pipeline_parallel_rank(rank: int):
        return ProcessGroupManager._dummy(_S.dummy_rank, "pp", rank)

    @staticmethod
    def set_dummy_pipeline_parallel_world_size(world_size: int):
        return ProcessGroupManager._dummy(_S.dummy_size, "pp", world_size)

    # ------------------------------------------------------------------ data parallel (ddp x fsdp == batch x cp)
    @staticmethod
    def get_data_parallel_group():
        return _S.groups.get("dp")

    @staticmethod
    def get_data_parallel_rank() -> int:
        return ProcessGroupManager._rank("dp")

    @staticmethod
    def get_data_parallel_world_size() -> int:
        return ProcessGroupManager._size("dp")

    @staticmethod
    def set_dummy_data_parallel_rank(rank: int):
        return ProcessGroupManager._dummy(_S.dummy_rank, "dp", rank)

    @staticmethod
    def set_dummy_data_parallel_world_size(world_size: int):
        return ProcessGroupManager._dummy(_S.dummy_size, "dp", world_size)

    @staticmethod
    def get_data_parallel_replication_world_size() -> int:
        return ProcessGroupManager._size("ddp")

    @staticmethod
    def get_data_parallel_sharding_world_size() -> int:
        return ProcessGroupManager._size("fsdp")

    @staticmethod
    def get_sharding_group():
        return _S.groups.get("fsdp")

    @staticmethod
    def get_replication_group():
        return _S.groups.get("ddp")

    @staticmethod
    def get_data_loading_rank() -> int:
        return ProcessGroupManager._rank("batch")

    @staticmethod
    def get_data_loading_world_size() -> int:
        return ProcessGroupManager._size("batch")

    # ------------------------------------------------------------------ context parallel
    @staticmethod
    def get_context_parallel_group():
        return _S.groups.get("cp")

    @staticmethod
    def get_context_parallel_rank() -> int:
        return ProcessGroupManager._rank("cp")

    @staticmethod
    def get_context_parallel_world_size() -> int:
        return ProcessGroupManager._size("cp")

    @staticmethod
    def set_dummy_context_parallel_rank(rank: int):
        return ProcessGroupManager._dummy(_S.dummy_rank, "cp", rank)

    @staticmethod
    def set_dummy_context_parallel_world_size(world_size: int):
        return ProcessGroupManager._dummy(_S.dummy_size, "cp", world_size)

    @staticmethod
    def is_context_parallel_enabled() -> bool:
        return ProcessGroupManager.get_context_parallel_world_size() > 1

    @staticmethod
    def is_context_parallel_first_rank() -> bool:
        return ProcessGroupManager.get_context_parallel_rank() == 0

    @staticmethod
    def get_context_parallel_load_balancing_method() -> ContextParallelLoadBalancerMethod | None:
        return _S.cp_lb

    @staticmethod
    def get_context_parallel_attention() -> str:
        return _S.cp_attention

    # ------------------------------------------------------------------ expert parallel (extension)
    @staticmethod
    def get_expert_parallel_group():
        return _S.groups.get("ep")

    @staticmethod
    def get_expert_parallel_rank() -> int:
        return ProcessGroupManager._rank("ep")

    @staticmethod
    def get_expert_parallel_world_size() -> int:
        return ProcessGroupManager._size("ep")

    @staticmethod
    def get_expert_data_parallel_group():
        return _S.groups.get("edp")

    # ------------------------------------------------------------------ device meshes (DTensor / DCP interop)
    @staticmethod
    def get_device_mesh(axis: str):
        """1-D ``DeviceMesh`` over the ranks of ``axis`` that contain this rank (built on first use)."""
        from torch.distributed.device_mesh import DeviceMesh

        if axis not in _S.meshes:
            ranks = ProcessGroupManager.get_group_ranks(axis)
            device = "cuda" if torch.cuda.is_available() else "cpu"
            group = _S.groups.get(axis)
            if group is not None:
                _S.meshes[axis] = DeviceMesh.from_group(group, device, mesh=ranks, mesh_dim_names=(axis,))
            else:
                _S.meshes[axis] = DeviceMesh(device, ranks, mesh_dim_names=(axis,))
        return _S.meshes[axis]

    @staticmethod
    def reject_context_parallel(what: str) -> None:
        """For layers whose recurrence has no context-parallel form here (the reference runs them on each rank's
        shard as if it were the whole sequence, which is silently wrong): fail at construction."""
        if ProcessGroupManager.is_context_parallel_enabled():
            raise NotImplementedError(f"{what}: context parallelism is implemented for softmax attention, Mamba-2 "
                                      "and M2RNN only")

    @staticmethod
    def get_device_mesh_2d(outer: str, inner: str):
        """2-D ``DeviceMesh`` ``[outer, inner]`` over the ranks that share this rank's other coordinates, on the
        existing process groups of the two axes (entry ``[i][j]``: the rank with index ``i`` on ``outer`` inside the
        ``inner`` group of ...): row ``i`` is the ``inner`` group of the ``i``-th member of this rank's ``outer``
        group."""
        from torch.distributed.device_mesh import DeviceMesh

        key = f"{outer}x{inner}"
        if key not in _S.meshes:
            topo = ProcessGroupManager.topology()
            grid = [topo.group(inner, r) for r in topo.group(outer, _S.rank)]
            device = "cuda" if torch.cuda.is_available() else "cpu"
            groups = [_S.groups.get(outer), _S.groups.get(inner)]
            assert all(g is not None for g in groups), f"no process group for {outer} / {inner}"
            _S.meshes[key] = DeviceMesh.from_group(groups, device, mesh=grid, mesh_dim_names=(outer, inner))
        return _S.meshes[key]

    # ------------------------------------------------------------------ misc
    @staticmethod
    def is_tracking_rank() -> bool:
        """first dp / cp / tp rank of the last pipeline stage (lm_engine/logging_utils/tracking.py:30-60)."""
        P = ProcessGroupManager
        return (P.get_data_parallel_rank() == 0 and P.get_tensor_parallel_rank() == 0
                and P.get_pipeline_parallel_rank() == P.get_pipeline_parallel_world_size() - 1)

    @staticmethod
    def broadcast_object(obj: Any, src: int = 0, group=None) -> Any:
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=group)
        return box[0]

    @staticmethod
    def barrier() -> None:
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    @staticmethod
    def destroy_process_groups() -> None:
        import sys

        if dist.is_initialized() and _S.owns_pg:
            dist.barrier()
        # symmetric-memory contexts are keyed by their group: none may outlive it (freed behind the barrier, when no
        # peer kernel can still be reading them)
        for name in ("expert_exchange", "gathered_attention"):
            mod = sys.modules.get(f"{__package__}.{name}")
            if mod is not None and mod._CONTEXTS:
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                mod._CONTEXTS.clear()
        if dist.is_initialized() and _S.owns_pg:
            dist.destroy_process_group()
        _S.reset()

    def __str__(self) -> str:
        t = ProcessGroupManager.topology()
        return (f"ProcessGroupManager(world={t.world_size}, pp={t.pp}, ddp={t.ddp}, fsdp={t.fsdp}, tp={t.tp}, "
                f"cp={t.cp}, ep={t.ep}, batch={t.batch})")


def run_rank_n(func: Callable, rank: int = 0, barrier: bool = False) -> Callable:
    """Wraps ``func`` so that only global rank ``rank`` executes it (others return None); optional barrier after."""

    def wrapper(*args, **kwargs):
        out = func(*args, **kwargs) if ProcessGroupManager.get_global_rank() == rank else None
        if barrier:
            ProcessGroupManager.barrier()
        return out

    return wrapper
