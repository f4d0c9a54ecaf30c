"""Base class of every config section: pydantic model that rejects unknown keys (the YAML schema is closed, as in
the reference's ``BaseArgs``, lm_engine/arguments/base.py:16-94) plus dict export and pretty logging."""

from __future__ import annotations

import logging
from contextlib import contextmanager
from enum import Enum
from typing import Any

from pydantic import BaseModel, ConfigDict


def _plain(value: Any) -> Any:
    if isinstance(value, BaseArgs):
        return value.to_dict()
    if isinstance(value, Enum):
        return value.value
    if isinstance(value, type):
        return value.__name__
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if isinstance(value, dict):
        return {k: _plain(v) for k, v in value.items()}
    return value


class BaseArgs(BaseModel):
    model_config = ConfigDict(extra="forbid", protected_namespaces=(), validate_assignment=False)

    def to_dict(self) -> dict:
        return {name: _plain(getattr(self, name)) for name in type(self).model_fields}

    @contextmanager
    def temporary_argument_value(self, name: str, value: Any):
        old = getattr(self, name)
        setattr(self, name, value)
        try:
            yield
        finally:
            setattr(self, name, old)

    def _lines(self, indent: int = 0) -> list[str]:
        pad = " " * indent
        out: list[str] = []
        for name in sorted(type(self).model_fields, key=str.lower):
            value = getattr(self, name)
            dots = "." * max(2, 48 - len(name) - indent)
            if isinstance(value, BaseArgs):
                out.append(f"{pad}{name}:")
                out.extend(value._lines(indent + 4))
            elif isinstance(value, list) and value and all(isinstance(v, BaseArgs) for v in value):
                out.append(f"{pad}{name}:")
                for i, v in enumerate(value):
                    if i:
                        out.append(" " * (indent + 4) + "*" * (44 - indent))
                    out.extend(v._lines(indent + 4))
            else:
                out.append(f"{pad}{name} {dots} {_plain(value)}")
        return out

    def log_args(self) -> None:
        from ..logging_utils import log_rank_0

        log_rank_0(logging.INFO, "------------------------ arguments ------------------------")
        for line in self._lines():
            log_rank_0(logging.INFO, line)
        log_rank_0(logging.INFO, "-------------------- end of arguments ---------------------")
