"""Optimizers over the flat shards of :class:`~lm_engine_b200.parallel.fsdp.FSDPEngine`.

``TorchAdamW`` (the default) runs the fused CUDA AdamW with device-side global-norm clipping.  The other names of
the reference's table (lm_engine/optimization/optimizer.py:25-39) run the corresponding ``torch.optim`` class on
1-D fp32 parameters that alias the master shards - every one of them is element-wise, so the flat layout is exact.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..containers import ModelContainer, OptimizerContainer
from ..enums import ParamsGroupMethod
from ..parallel.fsdp import FSDPEngine

_TORCH_OPTIMIZERS = {
    "TorchAdadelta": "Adadelta", "TorchAdagrad": "Adagrad", "TorchAdam": "Adam", "TorchAdamax": "Adamax",
    "TorchAdamW": "AdamW", "TorchASGD": "ASGD", "TorchLBFGS": "LBFGS", "TorchNAdam": "NAdam", "TorchRAdam": "RAdam",
    "TorchRMSprop": "RMSprop", "TorchRprop": "Rprop", "TorchSGD": "SGD",
}


class ShardedOptimizer:
    """Optimizer facade with ``param_groups`` (for LR schedulers), ``step``, ``zero_grad`` and state dicts."""

    def __init__(self, engine: FSDPEngine, class_name: str, class_args: dict, m_width: float | None,
                 use_mup: bool, max_grad_norm: float | None, step_in_backward: bool = False) -> None:
        if class_name not in _TORCH_OPTIMIZERS:
            raise ValueError(f"invalid class_name ({class_name}) for optimizer")
        self.engine, self.class_name, self.class_args = engine, class_name, dict(class_args)
        self.max_grad_norm = max_grad_norm
        self.step_in_backward = step_in_backward
        lr = class_args["lr"]
        self.param_groups = [{"name": "normal", "lr": lr}, {"name": "no_weight_decay", "lr": lr, "weight_decay": 0}]
        if use_mup:
            self.param_groups.append({"name": "mup", "lr": lr / m_width})
        self.fused = class_name == "TorchAdamW" and set(class_args) <= {"lr", "weight_decay", "betas", "eps"}
        self._torch_opt = None
        if getattr(engine, "cpu_offload", False) and (not self.fused or step_in_backward):
            raise NotImplementedError("cpu_offload is implemented for TorchAdamW (lr / weight_decay / betas / eps) "
                                      "stepping after the backward pass")
        if not self.fused:
            self._build_torch_optimizer()
        if step_in_backward:
            # The reference steps a per-parameter optimizer from a post-accumulate-grad hook
            # (lm_engine/optimization/optimizer.py:70-83): the update of a parameter overlaps the backward pass of
            # the layers in front of it, and there is no global gradient norm to clip by.  Here the update of a
            # unit's shard runs on the reduction stream right behind the unit's gradient reduction.
            if not self.fused:
                raise NotImplementedError("use_optimizer_with_backward_hook is implemented for TorchAdamW with "
                                          "lr / weight_decay / betas / eps only")
            engine.post_reduce_hook = self._step_unit

    def _build_torch_optimizer(self) -> None:
        groups: dict[str, list[nn.Parameter]] = {g["name"]: [] for g in self.param_groups}
        self._aliases: list[tuple[nn.Parameter, torch.Tensor, torch.Tensor]] = []
        for u in self.engine.all_units:
            for g in u.local_group_ranges():
                sl = slice(g.start, g.end)
                p = nn.Parameter(u.master[sl])
                groups[g.name if g.name in groups else "normal"].append(p)
                self._aliases.append((p, u, sl))
        cls = getattr(torch.optim, _TORCH_OPTIMIZERS[self.class_name])
        pgs = []
        for g in self.param_groups:
            if groups[g["name"]]:
                pgs.append({"params": groups[g["name"]], **{k: v for k, v in g.items() if k != "name"}})
        self._torch_opt = cls(pgs, **self.class_args)
        self._torch_group_names = [g["name"] for g in self.param_groups if groups[g["name"]]]

    def zero_grad(self) -> None:
        self.engine.zero_grad()
        if self.step_in_backward:
            self.engine.step_count += 1     # the units step during the backward pass that follows

    @torch.no_grad()
    def _step_unit(self, u) -> None:
        from .. import ops

        e, a = self.engine, self.class_args
        lrs = {g["name"]: g["lr"] for g in self.param_groups}
        if u.grad_post_scale != 1.0:
            u.grad_shard.mul_(u.grad_post_scale)
        for g in u.local_group_ranges():
            sl = slice(g.start, g.end)
            ops.adamw_step(u.master[sl], u.exp_avg[sl], u.exp_avg_sq[sl], u.grad_shard[sl], u.lp_shard[sl],
                           lr=lrs.get(g.name, lrs["normal"]), betas=tuple(a.get("betas", (0.9, 0.999))),
                           eps=a.get("eps", 1e-8),
                           weight_decay=0.0 if g.name == "no_weight_decay" else a.get("weight_decay", 1e-2),
                           step=e.step_count, gscale=None)
        u.grad_scaled = True
        if u.main_grad is None:
            u.grad_shard_fresh = True       # the next reduction of this unit starts a new gradient
        else:
            for s in u.slots:
                s.param.main_grad_stale = True

    @torch.no_grad()
    def step(self, total_sumsq: torch.Tensor | None = None) -> torch.Tensor:
        e = self.engine
        lrs = {g["name"]: g["lr"] for g in self.param_groups}
        a = self.class_args
        if self.step_in_backward:
            # every unit has stepped behind its reduction; join, republish the parameters, no norm to report
            e.finish_backward()
            if e.stage in (1, 2):
                import torch.distributed as dist

                for u in e.all_units:
                    if u.world > 1:
                        dist.all_gather_into_tensor(u.flat_param, u.lp_shard.clone(), group=u.group)
            e._cross_rank_fence()
            e.prefetch_first_units()
            e.grad_norm.zero_()
            return e.grad_norm
        if self.fused:
            return e.clip_and_step(lr=lrs["normal"], lr_by_group=lrs, betas=tuple(a.get("betas", (0.9, 0.999))),
                                   eps=a.get("eps", 1e-8), weight_decay=a.get("weight_decay", 1e-2),
                                   max_grad_norm=self.max_grad_norm, total_sumsq=total_sumsq)
        from .. import ops

        e.step_count += 1
        if total_sumsq is not None:
            e.sumsq.copy_(total_sumsq)
        else:
            e.local_sumsq(include_pipeline_group=True)
        ops.clip_coef_(e.sumsq, self.max_grad_norm, e.grad_norm, e.clip_coef)
        for p, u, sl in self._aliases:
            p.grad = u.grad_shard[sl].float() * e.clip_coef
        for g, name in zip(self._torch_opt.param_groups, self._torch_group_names):
            g["lr"] = lrs[name]
        self._torch_opt.step()
        for p, u, sl in self._aliases:
            u.lp_shard[sl].copy_(u.master[sl])
            p.grad = None
        if e.stage in (1, 2):
            import torch.distributed as dist

            for u in e.all_units:
                if u.world > 1:
                    dist.all_gather_into_tensor(u.flat_param, u.lp_shard.clone(), group=u.group)
        # the peers read this rank's parameter shard for the next step's gathers: order the update before them
        e._cross_rank_fence()
        return e.grad_norm

    # ------------------------------------------------------------------ state of the torch optimizers, per unit
    def tensor_state_keys(self) -> list[str]:
        """Names of the per-element state tensors that the wrapped ``torch.optim`` class keeps (``momentum_buffer``,
        ``exp_avg``, ``square_avg``, ...); empty before the first step of a fresh optimizer."""
        keys: list[str] = []
        if self._torch_opt is None:
            return keys
        for p, _, _ in self._aliases:
            for k, v in self._torch_opt.state.get(p, {}).items():
                if isinstance(v, torch.Tensor) and v.numel() == p.numel() and v.numel() > 1 and k not in keys:
                    keys.append(k)
        return sorted(keys)

    def scalar_state(self) -> dict[str, float]:
        """Scalar entries (``step`` and the like), the same for every parameter."""
        out: dict[str, float] = {}
        if self._torch_opt is None:
            return out
        for p, _, _ in self._aliases:
            for k, v in self._torch_opt.state.get(p, {}).items():
                if isinstance(v, (int, float)) or (isinstance(v, torch.Tensor) and v.numel() == 1 and p.numel() > 1):
                    out.setdefault(k, float(v))
        return out

    def unit_state(self, u, key: str) -> torch.Tensor:
        """Local fp32 slice (the unit's optimizer-state range of this rank) of state tensor ``key``."""
        flat = torch.zeros(u.state_hi - u.state_lo, dtype=torch.float32, device=u.master.device)
        for p, pu, sl in self._aliases:
            if pu is u:
                v = self._torch_opt.state.get(p, {}).get(key)
                if v is not None:
                    flat[sl].copy_(v.reshape(-1))
        return flat

    def set_unit_state(self, u, key: str, flat: torch.Tensor) -> None:
        for p, pu, sl in self._aliases:
            if pu is u:
                self._torch_opt.state[p][key] = flat[sl].clone().view_as(p)

    def set_scalar_state(self, scalars: dict[str, float]) -> None:
        for p, _, _ in self._aliases:
            for k, v in scalars.items():
                self._torch_opt.state[p][k] = torch.tensor(float(v), dtype=torch.float32)

    def state_dict(self) -> dict:
        sd = {"step": self.engine.step_count, "param_groups": [dict(g) for g in self.param_groups]}
        if self._torch_opt is not None:
            sd["torch"] = self._torch_opt.state_dict()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.engine.step_count = sd["step"]
        for g, s in zip(self.param_groups, sd["param_groups"]):
            g.update(s)
        if self._torch_opt is not None and "torch" in sd:
            self._torch_opt.load_state_dict(sd["torch"])


def get_optimizer_container(optimizer_class_name: str, optimizer_class_args: dict, model_container: ModelContainer,
                            params_group_method: ParamsGroupMethod | None,
                            use_optimizer_with_backward_hook: bool = False,
                            max_grad_norm: float | None = 1.0) -> OptimizerContainer:
    opts = []
    for wrapper in model_container:
        engine = wrapper.engine
        assert engine is not None, "wrap_model_container_for_distributed_training must run before the optimizer"
        opts.append(ShardedOptimizer(engine, optimizer_class_name, optimizer_class_args,
                                     getattr(wrapper.config, "m_width", None),
                                     params_group_method == ParamsGroupMethod.mup, max_grad_norm,
                                     step_in_backward=use_optimizer_with_backward_hook))
    return OptimizerContainer(opts)
