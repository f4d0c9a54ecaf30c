"""Lazy reader / sharded writer for safetensors checkpoints (reference: lm_engine/utils/safetensors.py:20-121).

The reader opens files on demand and can hand out slices (``get_slice``) so tensor-parallel ranks read only their
shard of each tensor.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors import safe_open
from safetensors.torch import save_file

_INDEX = "model.safetensors.index.json"
_SINGLE = "model.safetensors"


class SafeTensorsWeightsManager:
    def __init__(self, model_path: str) -> None:
        self.model_path = model_path
        self._where: dict[str, str] = {}
        self._handles: dict[str, object] = {}
        index = os.path.join(model_path, _INDEX)
        if os.path.exists(index):
            self._where = dict(json.load(open(index))["weight_map"])
        else:
            files = [f for f in sorted(os.listdir(model_path)) if f.endswith(".safetensors")]
            for fname in files:
                with safe_open(os.path.join(model_path, fname), framework="pt") as f:
                    for k in f.keys():
                        self._where[k] = fname

    def _file(self, name: str):
        fname = self._where[name]
        if fname not in self._handles:
            self._handles[fname] = safe_open(os.path.join(self.model_path, fname), framework="pt")
        return self._handles[fname]

    def __len__(self) -> int:
        return len(self._where)

    def __iter__(self):
        return iter(self._where)

    def keys(self):
        return self._where.keys()

    def has_tensor(self, name: str) -> bool:
        return name in self._where

    def get_slice(self, name: str):
        return self._file(name).get_slice(name)

    def get_shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.get_slice(name).get_shape())

    def get_tensor(self, name: str, dtype: torch.dtype | None = None, device: torch.device | None = None):
        t = self._file(name).get_tensor(name)
        if dtype is not None or device is not None:
            t = t.to(dtype=dtype, device=device)
        return t

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {k: self.get_tensor(k) for k in self._where}

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, SafeTensorsWeightsManager) or set(self.keys()) != set(other.keys()):
            return False
        return all(torch.equal(self.get_tensor(k), other.get_tensor(k)) for k in self.keys())

    @staticmethod
    def save_state_dict(state_dict: dict[str, torch.Tensor], save_path: str, max_shard_size: int = 5 * 2**30) -> None:
        """Writes ``model.safetensors`` or, above ``max_shard_size`` bytes, numbered shards plus an index json."""
        os.makedirs(save_path, exist_ok=True)
        shards: list[dict[str, torch.Tensor]] = [{}]
        size = 0
        for k, v in state_dict.items():
            nbytes = v.numel() * v.element_size()
            if shards[-1] and size + nbytes > max_shard_size:
                shards.append({})
                size = 0
            shards[-1][k] = v.detach().contiguous().cpu()
            size += nbytes
        if len(shards) == 1:
            save_file(shards[0], os.path.join(save_path, _SINGLE), metadata={"format": "pt"})
            return
        weight_map = {}
        total = 0
        for i, shard in enumerate(shards):
            fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(shard, os.path.join(save_path, fname), metadata={"format": "pt"})
            for k, v in shard.items():
                weight_map[k] = fname
                total += v.numel() * v.element_size()
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map},
                  open(os.path.join(save_path, _INDEX), "w"), indent=2)
