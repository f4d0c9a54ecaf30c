"""Wraps the model container for distributed training: flat-buffer ZeRO/FSDP units, block gradient checkpointing,
mixed precision, efficient (meta-device) initialisation, and the pipeline schedule
(role of lm_engine/distributed.py:138-514).

``distributed_args`` mapping:

* ``stage`` 0 / 1 / 2 / 3 -> replicate / shard optimizer state (+ gradients) / shard parameters too.
* ``fsdp_algorithm`` 1, 2, 3 all select the same sharded runtime of this engine (FSDP-1's flat parameters, FSDP-2's
  per-block units and SimpleFSDP's compile-time bucketing are one mechanism here); ``null`` = no data-parallel
  wrapping beyond a single unit layout.
* ``zero_topology`` -> HSDP (replication x sharding groups).
* ``gradient_checkpointing_method: block`` with ``gradient_checkpointing_args: {num_blocks: N}`` checkpoints the
  first N blocks (all when omitted); ``checkpoint_every: k`` (extension) checkpoints every k-th block.
* ``communication_dtype`` -> dtype of the gradient buffers / reductions.
* ``torch_compile`` is accepted and ignored: there is no tracing compiler on the hot path.
"""

from __future__ import annotations

import logging

import torch
import torch.nn as nn

from .arguments import DistillationArgs, TrainingArgs
from .containers import ModelContainer
from .enums import GradientCheckpointingMethod, ParamsGroupMethod
from .logging_utils import log_rank_0
from .parallel.fsdp import FSDPEngine
from .utils import string_to_torch_dtype


def _flatten_args(args: tuple):
    """Splits positional args into tensors (passed through autograd) and a rebuild recipe."""
    tensors: list[torch.Tensor] = []
    recipe = []
    for a in args:
        if isinstance(a, torch.Tensor):
            recipe.append(("t", len(tensors)))
            tensors.append(a)
        elif isinstance(a, tuple) and all(x is None or isinstance(x, torch.Tensor) for x in a):
            idx = []
            for x in a:
                if x is None:
                    idx.append(None)
                else:
                    idx.append(len(tensors))
                    tensors.append(x)
            recipe.append(("tuple", idx))
        else:
            recipe.append(("const", a))

    def rebuild(ts):
        out = []
        for kind, v in recipe:
            if kind == "t":
                out.append(ts[v])
            elif kind == "tuple":
                out.append(tuple(None if i is None else ts[i] for i in v))
            else:
                out.append(v)
        return out

    return tensors, rebuild


def _install_unit_forward(engine: FSDPEngine, module: nn.Module, unit_name: str) -> None:
    """Routes ``module.forward`` through the engine.  Auxiliary (router) losses produced inside the unit are returned
    as one more output of the unit and re-added to the accumulator outside: the accumulator must only ever hold
    tensors of the outer autograd graph, else the final loss would back-propagate into a unit's private graph behind
    the engine's back (and a checkpointed unit would lose the term altogether)."""
    from .models.aux_loss import add_aux_loss, swap_aux_loss

    inner = module.forward

    def forward(*args, **kwargs):
        tensors, rebuild = _flatten_args(args)
        info = {}

        def fn(*ts):
            outer = swap_aux_loss(0)
            try:
                out = inner(*rebuild(ts), **kwargs)
            finally:
                aux = swap_aux_loss(outer)
            info["tuple"] = isinstance(out, tuple)
            info["aux"] = isinstance(aux, torch.Tensor)
            if not info["aux"]:
                return out
            return (*out, aux) if info["tuple"] else (out, aux)

        out = engine.run_unit(unit_name, fn, *tensors)
        if info.get("aux"):
            add_aux_loss(out[-1])
            out = out[:-1] if info["tuple"] else out[0]
        return out

    module.forward = forward


def build_units(model: nn.Module) -> list[tuple[str, list[nn.Module], list[str]]]:
    """Execution-ordered sharding units of a ``CausalLM``: embedding(s), each block, final norm, LM head."""
    tr = model.transformer
    units = []
    if hasattr(tr, "wte"):
        units.append(("embed", [tr.wte], ["transformer.wte"]))
    if hasattr(tr, "wpe"):
        units.append(("wpe", [tr.wpe], ["transformer.wpe"]))
    for key, blk in tr.h.items():
        units.append((f"h.{key}", [blk], [f"transformer.h.{key}"]))
    if hasattr(tr, "ln_f") and any(True for _ in tr.ln_f.parameters()):
        units.append(("ln_f", [tr.ln_f], ["transformer.ln_f"]))
    if hasattr(model, "lm_head"):
        units.append(("lm_head", [model.lm_head], ["lm_head"]))
    extra = getattr(model, "extra_units", None)
    if extra is not None:
        units.extend(extra())
    return units


def _checkpointed_units(model: nn.Module, method, ckpt_args: dict) -> set[str]:
    if method is None:
        return set()
    assert method == GradientCheckpointingMethod.block
    keys = list(model.transformer.h.keys())
    every = ckpt_args.get("checkpoint_every", 1)
    n = ckpt_args.get("num_blocks", len(keys))
    return {f"h.{k}" for i, k in enumerate(keys) if i < n and i % every == 0}


def shard_model(wrapper, *, stage: int, dtype: torch.dtype, communication_dtype: torch.dtype | None,
                gradient_checkpointing_method=None, gradient_checkpointing_args: dict | None = None,
                use_mup_group: bool = False, seed: int = 0, device: torch.device | None = None,
                cpu_offload: bool = False) -> FSDPEngine:
    model = wrapper.model
    units = build_units(model)
    ckpt = _checkpointed_units(model, gradient_checkpointing_method, gradient_checkpointing_args or {})
    has_dropout = any(isinstance(m, nn.Dropout) and m.p > 0 for m in model.modules())
    engine = FSDPEngine(model, units, stage=stage, compute_dtype=dtype, grad_dtype=communication_dtype or dtype,
                        device=device, use_mup_group=use_mup_group, checkpoint_units=ckpt, preserve_rng=has_dropout,
                        seed=seed, cpu_offload=cpu_offload)
    tr = model.transformer
    for name, mods, _ in units:
        for m in mods:
            _install_unit_forward(engine, m, name)
    if getattr(model, "_tied_word_embeddings", False) and hasattr(tr, "wte"):
        engine.by_name["embed"].keep_unsharded = True
        inner = model.compute_logits

        def compute_logits(hidden):
            return engine.run_unit("embed", lambda h: inner(h), hidden)

        model.compute_logits = compute_logits
        inner_loss = model.compute_lm_loss

        def compute_lm_loss(hidden, labels, **kw):
            return engine.run_unit("embed", lambda h, l: inner_loss(h, l, **kw), hidden, labels)

        model.compute_lm_loss = compute_lm_loss
    wrapper.engine = engine
    if wrapper.has_teacher_model():
        wrapper.place_teacher(engine.device)
    return engine


def wrap_model_container_for_distributed_training(args: TrainingArgs | DistillationArgs,
                                                  model_container: ModelContainer):
    """Returns ``(model_container, pipeline_schedule)``; ``pipeline_schedule`` is None without pipeline parallel."""
    d = args.distributed_args
    assert d.stage in (0, 1, 2, 3)
    dtype_name = args.mixed_precision_args.dtype
    dtype = torch.bfloat16 if dtype_name == "fp8" else string_to_torch_dtype(dtype_name)
    comm = string_to_torch_dtype(d.communication_dtype) if d.communication_dtype is not None else None
    if d.torch_compile:
        log_rank_0(logging.WARNING, "torch_compile is ignored: kernels are hand-written, nothing is traced")
    if d.cpu_offload:
        log_rank_0(logging.WARNING, "cpu_offload: fp32 master weights and AdamW moments are kept in pinned host "
                   "memory and updated on the host (slow; a B200 holds the state of a 10B-parameter model in HBM)")
    for wrapper in model_container:
        shard_model(wrapper, stage=d.stage, dtype=dtype, communication_dtype=comm,
                    gradient_checkpointing_method=d.gradient_checkpointing_method,
                    gradient_checkpointing_args=d.gradient_checkpointing_args,
                    use_mup_group=args.optimizer_args.params_group_method == ParamsGroupMethod.mup,
                    seed=args.random_args.seed, cpu_offload=bool(d.cpu_offload))
        if dtype_name == "fp8":
            from .fp8 import convert_to_fp8_training

            convert_to_fp8_training(wrapper.model)
    schedule = None
    if d.num_pipeline_stages > 1:
        from .parallel.pipeline_parallel import build_pipeline_schedule

        schedule = build_pipeline_schedule(args, model_container)
    return model_container, schedule
