"""Dictionary of running metrics with element-wise ``+`` and ``/`` (reference: logging_utils/loss_dict.py:8-59)."""

from __future__ import annotations

from typing import Any

import torch


class MetricsTrackingDict:
    def __init__(self, tracked: dict[str, Any] | None = None) -> None:
        self._d: dict[str, Any] = dict(tracked or {})

    def __getitem__(self, key: str) -> Any:
        return self._d[key]

    def __setitem__(self, key: str, value: Any) -> None:
        self._d[key] = value

    def __contains__(self, key: str) -> bool:
        return key in self._d

    def __len__(self) -> int:
        return len(self._d)

    def __iter__(self):
        return iter(self._d)

    def keys(self):
        return self._d.keys()

    def items(self):
        return self._d.items()

    def get_dict(self) -> dict[str, Any]:
        return self._d

    def __add__(self, other: "MetricsTrackingDict | dict") -> "MetricsTrackingDict":
        od = other._d if isinstance(other, MetricsTrackingDict) else other
        if not self._d:
            return MetricsTrackingDict(od)
        out = dict(self._d)
        for k, v in od.items():
            out[k] = out[k] + v if k in out else v
        return MetricsTrackingDict(out)

    def __truediv__(self, divisor: float) -> "MetricsTrackingDict":
        return MetricsTrackingDict({k: v / divisor for k, v in self._d.items()})

    def to_floats(self) -> dict[str, float]:
        return {k: (v.item() if isinstance(v, torch.Tensor) else float(v)) for k, v in self._d.items()}

    def __repr__(self) -> str:
        return f"MetricsTrackingDict({self._d})"
