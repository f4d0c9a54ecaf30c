"""Optimizer parameter groups from parameter markers: ``normal``, ``no_weight_decay`` (weight decay 0) and, with
``params_group_method: mup``, ``mup`` (lr / m_width) - lm_engine/optimization/params_group.py:18-145."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch.nn as nn

from ..enums import ParamsGroupMethod
from ..parameter import is_parameter_with_mup_learning_rate, is_parameter_with_no_weight_decay


@dataclass
class ParamsGroup:
    name: str
    parameter_name_map: dict[str, nn.Parameter]
    params_group_kwargs: dict = field(default_factory=dict)

    def to_param_group(self) -> dict:
        return {"params": list(self.parameter_name_map.values()), **self.params_group_kwargs}

    def __len__(self) -> int:
        return len(self.parameter_name_map)


@dataclass
class ParamsGroupsList:
    params_groups: list[ParamsGroup]

    def add_params_group(self, g: ParamsGroup) -> None:
        self.params_groups.append(g)

    def to_torch_compatible_params_groups(self) -> list[dict]:
        return [g.to_param_group() for g in self.params_groups]

    def get_param_names(self) -> dict[str, list[str]]:
        return {g.name: sorted(g.parameter_name_map) for g in self.params_groups}


def group_name_of(p: nn.Parameter, method: ParamsGroupMethod | None) -> str:
    if is_parameter_with_no_weight_decay(p):
        return "no_weight_decay"
    if method == ParamsGroupMethod.mup and is_parameter_with_mup_learning_rate(p):
        return "mup"
    return "normal"


def get_param_groups(model: nn.Module, optimizer_class_args: dict, method: ParamsGroupMethod | None,
                     m_width: float | None = None, prefix: str = "") -> ParamsGroupsList:
    if method not in (None, ParamsGroupMethod.mup):
        raise ValueError(f"unexpected `params_group_method` {method}")
    buckets: dict[str, dict[str, nn.Parameter]] = {"normal": {}, "no_weight_decay": {}, "mup": {}}
    for name, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
        buckets[group_name_of(p, method)][prefix + name] = p
    out = ParamsGroupsList([])
    if buckets["normal"]:
        out.add_params_group(ParamsGroup("normal", buckets["normal"]))
    if buckets["no_weight_decay"]:
        out.add_params_group(ParamsGroup("no_weight_decay", buckets["no_weight_decay"], {"weight_decay": 0}))
    if buckets["mup"]:
        assert m_width is not None, "m_width is needed for the mup params group method"
        out.add_params_group(ParamsGroup("mup", buckets["mup"], {"lr": optimizer_class_args["lr"] / m_width}))
    return out


def get_param_groups_list(model_container, optimizer_class_args: dict,
                          method: ParamsGroupMethod | None) -> list[ParamsGroupsList]:
    out = []
    for wrapper in model_container:
        cfg = getattr(wrapper, "config", None)
        out.append(get_param_groups(wrapper, optimizer_class_args, method, getattr(cfg, "m_width", None)))
    return out
