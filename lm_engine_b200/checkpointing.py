"""Checkpoint save / resume / unshard with the reference's on-disk layout
(lm_engine/checkpointing/__init__.py:49-446, model.py, optimizer.py, model_optimizer.py, lr_scheduler.py)::

    <save_path>/latest_checkpointed_iteration.json
    <save_path>/global_step{N}/model/            torch DCP directory, root key "state", keys "model.<parameter fqn>"
                               optimizer/        torch DCP directory, flattened optimizer state
                               model_optimizer/  async mode: {"state": {"model": ..., "optimizer": ...}}
                               lr_scheduler/lr_scheduler-{global_rank}.pt
                               rng_state/rng_state-{global_rank}.pt
                               dataloader/dataloader-{data_loading_rank}.pt
                               experiments_tracker.json, metadata.json, training_config.yml

The runtime keeps parameters as flat per-unit shards; at save time every parameter is re-cut into the standard
DTensor layout (``Shard(0)`` over the sharding group, ``Shard(tp_dim)`` over the tensor-parallel group), so the
files are ordinary DCP checkpoints that reshard on load to any topology and that plain ``dcp.load`` / the
reference's unshard path can read.  Works on CPU (gloo) as well as CUDA.  A checkpoint directory is written under a
temporary name and renamed when complete; ``latest_checkpointed_iteration.json`` is replaced atomically afterwards.
A file named ``KILLSWITCH`` in ``save_path`` makes the job exit cleanly after the next checkpoint.
"""

from __future__ import annotations

import json
import logging
import os
import random
import shutil
import subprocess

import numpy as np
import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import yaml
from torch.distributed.tensor import DTensor, Replicate, Shard

from .accelerator import Accelerator
from .arguments import DistillationArgs, TrainingArgs, UnshardingArgs
from .containers import LRSchedulerContainer, ModelContainer, OptimizerContainer
from .logging_utils import log_rank_0
from .parallel.manager import ProcessGroupManager
from .utils import load_yaml, string_to_torch_dtype

_KILLSWITCH = "KILLSWITCH"
_FUTURE = None
_PENDING_PUBLISH = None


def _tag(iteration: int) -> str:
    return f"global_step{iteration}"


def _base(path: str, iteration: int) -> str:
    return os.path.join(path, _tag(iteration))


def _latest_file(path: str) -> str:
    return os.path.join(path, "latest_checkpointed_iteration.json")


def _rank_file(base: str, kind: str, rank: int) -> str:
    return os.path.join(base, kind, f"{kind}-{rank}.pt")


def _commit_id() -> str | None:
    try:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        r = subprocess.run(["git", "-C", root, "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5)
        return r.stdout.strip() or None
    except Exception:  # noqa: BLE001
        return None


def ensure_last_checkpoint_is_saved() -> None:
    global _FUTURE, _PENDING_PUBLISH
    if _FUTURE is not None:
        _FUTURE.result()
        _FUTURE = None
    if _PENDING_PUBLISH is not None:
        _PENDING_PUBLISH()
        _PENDING_PUBLISH = None


# ---------------------------------------------------------------------------------------------- state dicts
def _to_dtensor(engine, local_full: torch.Tensor, param: torch.nn.Parameter) -> torch.Tensor:
    """Full (per-TP-rank) tensor -> DTensor in the standard layout, or the tensor itself on a single rank."""
    tp_dim = getattr(param, "tp_shard_dim", None)
    tp_group = ProcessGroupManager.get_tensor_parallel_group()
    if engine.shard_group is not None and tp_group is None and engine.stage >= 1 and local_full.dim() >= 1:
        mesh = ProcessGroupManager.get_device_mesh("fsdp")
        n, world, rank = local_full.size(0), engine.world, engine.rank
        per = -(-n // world)
        lo, hi = min(rank * per, n), min((rank + 1) * per, n)
        chunk = local_full[lo:hi].clone()
        return DTensor.from_local(chunk, mesh, [Shard(0)], run_check=False, shape=local_full.shape,
                                  stride=local_full.stride())
    if tp_group is not None:
        tp_placement = Shard(tp_dim) if tp_dim is not None else Replicate()
        if engine.shard_group is not None and engine.stage >= 1 and engine.world > 1 and local_full.dim() >= 1:
            # tensor parallel x sharded data parallel: every rank offers only its block of rows of the TP-local
            # tensor.  Mesh order (tp, fsdp): a dimension split by both is split tp-major, as the model lays it out.
            mesh = ProcessGroupManager.get_device_mesh_2d("tp", "fsdp")
            n, world, rank = local_full.size(0), engine.world, engine.rank
            per = -(-n // world)
            lo, hi = min(rank * per, n), min((rank + 1) * per, n)
            shape = list(local_full.shape)
            if tp_dim is not None:
                shape[tp_dim] *= dist.get_world_size(tp_group)
            stride = torch.empty(shape, device="meta").stride()
            return DTensor.from_local(local_full[lo:hi].clone(), mesh, [tp_placement, Shard(0)], run_check=False,
                                      shape=torch.Size(shape), stride=stride)
        mesh = ProcessGroupManager.get_device_mesh("tp")
        return DTensor.from_local(local_full.clone(), mesh, [tp_placement], run_check=False)
    return local_full.clone()


def _chunk_dtensor(engine, chunk: torch.Tensor, param: torch.nn.Parameter, shape: torch.Size) -> torch.Tensor:
    """DTensor from this rank's block of rows (see ``FSDPEngine.row_chunks``): ``Shard(0)`` over the sharding group,
    or on the (tp, fsdp) mesh when the parameter is a tensor-parallel slice (``shape`` is the slice's shape)."""
    tp_group = ProcessGroupManager.get_tensor_parallel_group()
    if tp_group is None:
        mesh = ProcessGroupManager.get_device_mesh("fsdp")
        stride = torch.empty(shape, device="meta").stride()
        return DTensor.from_local(chunk.contiguous(), mesh, [Shard(0)], run_check=False, shape=shape, stride=stride)
    tp_dim = getattr(param, "tp_shard_dim", None)
    full = list(shape)
    if tp_dim is not None:
        full[tp_dim] *= dist.get_world_size(tp_group)
    stride = torch.empty(full, device="meta").stride()
    mesh = ProcessGroupManager.get_device_mesh_2d("tp", "fsdp")
    return DTensor.from_local(chunk.contiguous(), mesh, [Shard(tp_dim) if tp_dim is not None else Replicate(),
                                                         Shard(0)], run_check=False, shape=torch.Size(full),
                              stride=stride)


def _unit_state_tensors(eng, u, which) -> dict[str, torch.Tensor]:
    """Checkpoint-layout tensors (name -> DTensor / tensor) of one unit's state ``which``: row blocks exchanged
    point to point where the layout allows it, else cut from the gathered unit."""
    out = {}
    if eng.can_exchange_row_chunks(u) and all(len(s.shape) >= 1 for s in u.slots):
        chunks = eng.row_chunks(u, which)
        for s in u.slots:
            out[s.name] = _chunk_dtensor(eng, chunks[s.name], s.param, s.shape)
        return out
    full = eng.gather_full(u, which)
    for s in u.slots:
        out[s.name] = _to_dtensor(eng, eng._slot_full(s, full[s.offset:s.offset + s.numel].view(s.shape)), s.param)
    return out


def _from_saved(value: torch.Tensor, engine) -> torch.Tensor:
    """Inverse of :func:`_to_dtensor`: the full per-TP-rank tensor."""
    if isinstance(value, DTensor):
        tp = ProcessGroupManager.get_tensor_parallel_group()
        names = value.device_mesh.mesh_dim_names
        if tp is not None and names == ("tp",):
            return value.to_local()
        if tp is not None and names == ("tp", "fsdp"):
            # gather the row blocks over the sharding group, keep the tensor-parallel slice
            return value.redistribute(placements=[value.placements[0], Replicate()]).to_local()
        return value.full_tensor()
    return value


def model_state_dict(model_container: ModelContainer, which: str = "master") -> dict[str, torch.Tensor]:
    """Checkpoint-layout state of all local pipeline stages (keys ``model.<fqn>``, teacher weights excluded)."""
    out: dict[str, torch.Tensor] = {}
    for wrapper in model_container:
        eng = wrapper.engine
        if eng is None:
            for k, v in wrapper.model.state_dict().items():
                out[f"model.{k}"] = v
            continue
        for u in eng.all_units:
            for name, t in _unit_state_tensors(eng, u, which).items():
                out[f"model.{name}"] = t
    return out


def _is_row_block(value) -> bool:
    """A DTensor in the layout of :func:`_chunk_dtensor` (this rank holds a block of rows)."""
    if not isinstance(value, DTensor):
        return False
    names, pl = value.device_mesh.mesh_dim_names, value.placements
    return ((names == ("fsdp",) and pl[0] == Shard(0))
            or (names == ("tp", "fsdp") and pl[1] == Shard(0) and ProcessGroupManager.get_tensor_parallel_group()
                is not None))


def _load_engine_state(eng, values: dict[str, torch.Tensor], which: str) -> None:
    """``values``: slot name -> loaded value in the checkpoint layout.  Unit by unit, so that at most one unit is ever
    whole on a rank; units whose parameters all arrived as row blocks are re-cut with one all-to-all and no gather."""
    for u in eng.all_units:
        mine = {s.name: values[s.name] for s in u.slots if s.name in values}
        if not mine:
            continue
        if len(mine) == len(u.slots) and eng.can_exchange_row_chunks(u) and all(_is_row_block(v)
                                                                                for v in mine.values()):
            eng.load_row_chunks(u, {n: v.to_local() for n, v in mine.items()}, which)
        else:
            eng.load_full_state_dict({n: _from_saved(v, eng) for n, v in mine.items()}, which)


def load_model_state_dict(model_container: ModelContainer, state: dict[str, torch.Tensor],
                          which: str = "master") -> None:
    for wrapper in model_container:
        eng = wrapper.engine
        if eng is None:
            wrapper.model.load_state_dict({k[len("model."):]: _from_saved(v, None) for k, v in state.items()},
                                          strict=False)
            continue
        names = [s.name for u in eng.all_units for s in u.slots]
        _load_engine_state(eng, {n: state[f"model.{n}"] for n in names if f"model.{n}" in state}, which)


_GROUP_KEYS = ("lr", "betas", "eps", "weight_decay", "initial_lr")


def _optimizer_keeps_step(opt) -> bool:
    """Whether the wrapped torch optimizer class tracks a per-parameter ``step`` (SGD does not)."""
    return getattr(opt, "class_name", "") not in ("TorchSGD",)


def _saved_optimizer_state_names(checkpoint_id: str, prefix: str = "state.") -> tuple[set[str], set[str]]:
    """Names of the per-element and of the scalar optimizer-state entries in a saved checkpoint (a fresh torch
    optimizer has no state yet, so the template to load into is shaped after what was saved)."""
    from torch.distributed.checkpoint import FileSystemReader

    tensors, scalars = set(), set()
    for k, md in FileSystemReader(checkpoint_id).read_metadata().state_dict_metadata.items():
        if not k.startswith(prefix + "state.model."):
            continue
        which = k.rpartition(".")[2]
        size = getattr(md, "size", None)
        (scalars if size is not None and len(size) == 0 else tensors).add(which)
    return tensors, scalars


def optimizer_state_dict(model_container: ModelContainer, optimizer_container: OptimizerContainer,
                         saved_names: tuple[set[str], set[str]] | None = None) -> dict:
    """Flattened optimizer state in torch's ``flatten_optimizer_state_dict`` key scheme:
    ``state.<fqn>.{exp_avg,exp_avg_sq,step}`` and ``param_groups.<fqn>.<hyper-parameter>``.  ``saved_names``
    (per-element names, scalar names) adds entries that a checkpoint holds but this optimizer has not created yet."""
    out: dict = {}
    for wrapper, opt in zip(model_container, optimizer_container):
        eng = wrapper.engine
        groups = {g["name"]: g for g in opt.param_groups}
        a = opt.class_args
        # fused AdamW: the moments are the engine's own shards; any other optimizer class keeps its per-element
        # state (momentum_buffer, exp_avg, square_avg, max_exp_avg_sq, ...) inside the wrapped torch optimizer
        fused = getattr(opt, "fused", True)
        keys = ["exp_avg", "exp_avg_sq"] if fused else opt.tensor_state_keys()
        scalars = {"step": float(eng.step_count)} if fused else {"step": float(eng.step_count), **opt.scalar_state()}
        if saved_names is not None and not fused:
            keys = sorted(set(keys) | saved_names[0])
            scalars = {**{k: 0.0 for k in saved_names[1]}, **scalars}
        for u in eng.all_units:
            states = {k: _unit_state_tensors(eng, u, k if fused else opt.unit_state(u, k)) for k in keys}
            for s in u.slots:
                fqn = f"model.{s.name}"
                for k, by_name in states.items():
                    out[f"state.{fqn}.{k}"] = by_name[s.name]
                for k, v in scalars.items():
                    out[f"state.{fqn}.{k}"] = torch.tensor(v)
                g = groups.get(s.group, groups["normal"])
                hyper = {"lr": g["lr"], "betas": tuple(a.get("betas", (0.9, 0.999))), "eps": a.get("eps", 1e-8),
                         "weight_decay": 0.0 if s.group == "no_weight_decay" else a.get("weight_decay", 1e-2),
                         "initial_lr": g.get("initial_lr", g["lr"])}
                for k in _GROUP_KEYS:
                    out[f"param_groups.{fqn}.{k}"] = hyper[k]
    return out


def load_optimizer_state_dict(model_container, optimizer_container, state: dict) -> None:
    for wrapper, opt in zip(model_container, optimizer_container):
        eng = wrapper.engine
        fused = getattr(opt, "fused", True)
        names = {s.name for u in eng.all_units for s in u.slots}
        found: dict[str, dict[str, torch.Tensor]] = {}       # state key -> slot name -> saved value
        for k, v in state.items():
            if k.startswith("state.model."):
                name, _, which = k[len("state.model."):].rpartition(".")
                if name in names:
                    found.setdefault(which, {})[name] = v
        if fused:
            for which in ("exp_avg", "exp_avg_sq"):
                _load_engine_state(eng, found.get(which, {}), which)
        else:
            scalars = {}
            for which, by_slot in found.items():
                first = next(iter(by_slot.values()))
                if not isinstance(first, DTensor) and first.numel() == 1:
                    if which != "step" or which in opt.scalar_state() or _optimizer_keeps_step(opt):
                        scalars[which] = float(first)
                    continue
                plain = {n: _from_saved(v, eng) for n, v in by_slot.items()}
                for u in eng.all_units:
                    opt.set_unit_state(u, which, eng.local_piece_from_slots(u, plain, opt.unit_state(u, which)))
            opt.set_scalar_state(scalars)
        steps = [float(v) for k, v in state.items() if k.endswith(".step")]
        if steps:
            eng.step_count = int(max(steps))
        for g in opt.param_groups:
            for u in eng.all_units:
                for s in u.slots:
                    if s.group == g["name"] and f"param_groups.model.{s.name}.lr" in state:
                        g["lr"] = state[f"param_groups.model.{s.name}.lr"]
                        g["initial_lr"] = state.get(f"param_groups.model.{s.name}.initial_lr", g["lr"])
                        break
                else:
                    continue
                break


# ---------------------------------------------------------------------------------------------- save
def save_checkpoint(args: TrainingArgs, model_container: ModelContainer,
                    optimizer_container: OptimizerContainer | None, lr_scheduler_container: LRSchedulerContainer | None,
                    train_dataloader, experiments_tracker, iteration: int, metadata: dict | None = None) -> None:
    global _FUTURE, _PENDING_PUBLISH
    ensure_last_checkpoint_is_saved()
    root = args.save_args.save_path
    final = _base(root, iteration)
    tmp = final + ".tmp"
    rank = ProcessGroupManager.get_global_rank()
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        os.makedirs(tmp, exist_ok=True)
    ProcessGroupManager.barrier()
    if lr_scheduler_container is not None:
        os.makedirs(os.path.join(tmp, "lr_scheduler"), exist_ok=True)
        torch.save([s.state_dict() for s in lr_scheduler_container], _rank_file(tmp, "lr_scheduler", rank))
    os.makedirs(os.path.join(tmp, "rng_state"), exist_ok=True)
    torch.save({"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
                "torch_rng_state": torch.get_rng_state(),
                "accelerator_rng_state": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
               _rank_file(tmp, "rng_state", rank))
    if train_dataloader is not None and hasattr(train_dataloader, "state_dict"):
        os.makedirs(os.path.join(tmp, "dataloader"), exist_ok=True)
        torch.save(train_dataloader.state_dict(),
                   _rank_file(tmp, "dataloader", ProcessGroupManager.get_data_loading_rank()))
    if rank == 0:
        if experiments_tracker is not None:
            json.dump(experiments_tracker.state_dict(), open(os.path.join(tmp, "experiments_tracker.json"), "w"),
                      indent=4)
        meta = dict(metadata or {})
        meta.setdefault("commit_id", _commit_id())
        meta["accelerator"] = Accelerator.get_accelerator().value
        json.dump(meta, open(os.path.join(tmp, "metadata.json"), "w"), indent=4)
        yaml.dump(args.to_dict(), open(os.path.join(tmp, "training_config.yml"), "w"), indent=2)
    save_opt = args.save_args.save_optimizer and optimizer_container is not None

    def publish() -> None:
        ProcessGroupManager.barrier()
        if rank == 0:
            shutil.rmtree(final, ignore_errors=True)
            os.replace(tmp, final)
            latest_tmp = _latest_file(root) + ".tmp"
            with open(latest_tmp, "w") as f:
                json.dump({"latest_checkpointed_iteration": iteration}, f, indent=4)
                f.flush()
                os.fsync(f.fileno())
            os.replace(latest_tmp, _latest_file(root))
        ProcessGroupManager.barrier()
        log_rank_0(logging.INFO, f"checkpoint saved at {iteration}")
        if os.path.exists(os.path.join(root, _KILLSWITCH)):
            log_rank_0(logging.WARNING, "KILLSWITCH found: exiting after checkpoint")
            ProcessGroupManager.destroy_process_groups()
            raise SystemExit(0)

    if args.save_args.async_checkpointing:
        state = {"model": model_state_dict(model_container)}
        if save_opt:
            state["optimizer"] = optimizer_state_dict(model_container, optimizer_container)
        _FUTURE = dcp.async_save({"state": state}, checkpoint_id=os.path.join(tmp, "model_optimizer"))
        _PENDING_PUBLISH = publish
        return
    dcp.save({"state": model_state_dict(model_container)}, checkpoint_id=os.path.join(tmp, "model"))
    if save_opt:
        dcp.save({"state": optimizer_state_dict(model_container, optimizer_container)},
                 checkpoint_id=os.path.join(tmp, "optimizer"))
    publish()


# ---------------------------------------------------------------------------------------------- load
def _resolve_iteration(load_path: str, iteration: int | None) -> int:
    if iteration is not None:
        return iteration
    return json.load(open(_latest_file(load_path)))["latest_checkpointed_iteration"]


def load_checkpoint_for_training(args: TrainingArgs, args_class: type[TrainingArgs | DistillationArgs],
                                 model_container: ModelContainer, optimizer_container: OptimizerContainer,
                                 lr_scheduler_container: LRSchedulerContainer, train_dataloader):
    """Restores model (+ optimizer, LR schedule, RNG, dataloader) state; returns ``(iteration, metadata,
    experiments-tracker state)``."""
    la = args.load_args
    if la is None or la.load_path is None:
        return 0, None, None
    iteration = _resolve_iteration(la.load_path, la.iteration)
    base = _base(la.load_path, iteration)
    saved_args = args_class(**load_yaml(os.path.join(base, "training_config.yml")))
    log_rank_0(logging.INFO, f"loading checkpoint saved at {base}")
    rank = ProcessGroupManager.get_global_rank()
    if saved_args.save_args.async_checkpointing:
        state = {"model": model_state_dict(model_container)}
        if la.load_optimizer:
            state["optimizer"] = optimizer_state_dict(
                model_container, optimizer_container,
                _saved_optimizer_state_names(os.path.join(base, "model_optimizer"), "state.optimizer."))
        wrapped = {"state": state}
        dcp.load(wrapped, checkpoint_id=os.path.join(base, "model_optimizer"))
        load_model_state_dict(model_container, wrapped["state"]["model"])
        if la.load_optimizer:
            load_optimizer_state_dict(model_container, optimizer_container, wrapped["state"]["optimizer"])
    else:
        wrapped = {"state": model_state_dict(model_container)}
        dcp.load(wrapped, checkpoint_id=os.path.join(base, "model"))
        load_model_state_dict(model_container, wrapped["state"])
        if la.load_optimizer:
            wrapped = {"state": optimizer_state_dict(
                model_container, optimizer_container,
                _saved_optimizer_state_names(os.path.join(base, "optimizer"), "state."))}
            dcp.load(wrapped, checkpoint_id=os.path.join(base, "optimizer"))
            load_optimizer_state_dict(model_container, optimizer_container, wrapped["state"])
    if la.load_lr_scheduler:
        assert la.load_optimizer, "load_lr_scheduler requires loading of optimizer"
        f = _rank_file(base, "lr_scheduler", rank)
        if not os.path.exists(f):
            f = _rank_file(base, "lr_scheduler", 0)
        for sched, sd in zip(lr_scheduler_container, torch.load(f, weights_only=False)):
            sched.load_state_dict(sd)
    elif la.resume_learning_rate:
        # rebuild the schedule position from the iteration, starting from the configured base learning rate
        for sched in lr_scheduler_container:
            sched.last_epoch = (iteration if la.load_starting_iteration else 0) - 1
            sched.step()
    if la.load_rng_state:
        f = _rank_file(base, "rng_state", rank)
        if os.path.exists(f):
            st = torch.load(f, weights_only=False)
            random.setstate(st["random_rng_state"])
            np.random.set_state(st["np_rng_state"])
            torch.set_rng_state(st["torch_rng_state"])
            if torch.cuda.is_available() and st.get("accelerator_rng_state") is not None:
                torch.cuda.set_rng_state(st["accelerator_rng_state"])
    metadata = json.load(open(os.path.join(base, "metadata.json")))
    if la.load_dataloader_state and train_dataloader is not None and hasattr(train_dataloader, "load_state_dict"):
        f = _rank_file(base, "dataloader", ProcessGroupManager.get_data_loading_rank())
        if os.path.exists(f):
            train_dataloader.load_state_dict(torch.load(f, weights_only=False))
    tracker = None
    tf = os.path.join(base, "experiments_tracker.json")
    if la.load_experiments_tracker_state and os.path.exists(tf):
        tracker = json.load(open(tf))
    return (iteration if la.load_starting_iteration else 0), metadata, tracker


def read_full_model_state(load_path: str, iteration: int | None = None) -> tuple[dict[str, torch.Tensor], dict, int]:
    """Reads a (possibly sharded) checkpoint into full CPU tensors without any process group.  Returns
    ``(state with keys "model.<fqn>", saved training config dict, iteration)``."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict

    iteration = _resolve_iteration(load_path, iteration)
    base = _base(load_path, iteration)
    cfg = load_yaml(os.path.join(base, "training_config.yml"))
    state: dict = {}
    if cfg["save_args"].get("async_checkpointing"):
        _load_state_dict(state, storage_reader=FileSystemReader(os.path.join(base, "model_optimizer")),
                         planner=_EmptyStateDictLoadPlanner(), no_dist=True)
        state = state["state"]["model"]
    else:
        _load_state_dict(state, storage_reader=FileSystemReader(os.path.join(base, "model")),
                         planner=_EmptyStateDictLoadPlanner(), no_dist=True)
        state = state["state"]
    return state, cfg, iteration


def load_checkpoint_and_unshard(args: UnshardingArgs):
    """Rebuilds the unsharded single-process model from a training checkpoint.  Returns
    ``(model wrapper, training args of the checkpoint, full state dict)``."""
    from .model_wrapper import get_model_container

    state, cfg, iteration = read_full_model_state(args.load_args.load_path, args.load_args.iteration)
    log_rank_0(logging.INFO, f"loading checkpoint saved at {_base(args.load_args.load_path, iteration)}")
    if "teacher_args" in cfg:
        cfg["tuning_args"]["tuning_method"] = "pretraining"
        cfg.pop("teacher_args")
    saved = TrainingArgs(**cfg)
    if args.mixed_precision_args is not None:
        saved.mixed_precision_args = args.mixed_precision_args
    P = ProcessGroupManager
    with P.set_dummy_tensor_parallel_rank(0), P.set_dummy_tensor_parallel_world_size(1), \
            P.set_dummy_pipeline_parallel_rank(0), P.set_dummy_pipeline_parallel_world_size(1), \
            saved.distributed_args.temporary_argument_value("num_pipeline_stages", 1), \
            saved.model_args.temporary_argument_value("efficient_initialization", False):
        wrapper = get_model_container(saved, efficient_initialization=False, keep_in_fp32=False)[0]
    dtype_name = saved.mixed_precision_args.dtype
    dtype = torch.bfloat16 if dtype_name == "fp8" else string_to_torch_dtype(dtype_name)
    plain = {k[len("model."):]: v.to(dtype) for k, v in state.items() if k.startswith("model.")}
    wrapper.model.to(dtype)
    wrapper.model.load_state_dict(plain)
    return wrapper, saved, plain
