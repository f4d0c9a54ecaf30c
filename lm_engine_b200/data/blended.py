"""Composition of GPT datasets: weighted blends (greedy lowest-quota-first interleave built by the native helper),
plain concatenation, train/val/test splits of one prefix, and the top-level ``build`` that turns the YAML's
``data_path`` / ``*_data_path`` / ``split`` into three datasets
(lm_engine/data/megatron/{blended_dataset,concatenated_dataset,blended_megatron_dataset_builder}.py)."""

from __future__ import annotations

import hashlib
import json
import logging
import math
import os

import numpy as np
import torch

from ..logging_utils import log_rank_0
from ..parallel.manager import ProcessGroupManager
from .gpt_dataset import GPTDataset
from .helpers import build_blending_indices
from .indexed import IndexedDataset

SPLITS = ("train", "valid", "test")


def normalize(weights: list[float]) -> list[float]:
    w = np.asarray(weights, dtype=np.float64)
    return (w / w.sum()).tolist()


def parse_and_normalize_split(split: str) -> list[float]:
    """``"98,1,1"`` or ``"0.9/0.05/0.05"`` -> three fractions summing to 1."""
    parts = [float(x) for x in split.replace("/", ",").split(",")]
    parts += [0.0] * (len(SPLITS) - len(parts))
    assert len(parts) == len(SPLITS) and all(p >= 0 for p in parts)
    return normalize(parts)


def parse_blend(blend: list[str]) -> tuple[list[str], list[float] | None]:
    """``[w1, p1, w2, p2, ...]`` -> (prefixes, weights); a list that is not weight/prefix pairs -> (prefixes, None)."""
    if len(blend) % 2 == 1:
        return [p.strip() for p in blend], None
    try:
        weights = [float(blend[i]) for i in range(0, len(blend), 2)]
    except ValueError:
        return [p.strip() for p in blend], None
    return [blend[i].strip() for i in range(1, len(blend), 2)], weights


def split_bounds(split: list[float], num_elements: int) -> list[int]:
    """Cumulative element boundaries per split, e.g. [0, 900, 990, 1000]."""
    b = [0]
    for frac in split:
        b.append(b[-1] + int(round(frac * float(num_elements))))
    excess = b[-1] - num_elements
    b[1:] = [x - excess for x in b[1:]]
    assert b[-1] == num_elements
    return b


def sizes_for_blend(weights: list[float], targets: list[int]) -> list[list[int]]:
    """Samples to request from every member dataset per split (0.5 % head-room)."""
    return [[int(math.ceil(t * w * 1.005)) for t in targets] for w in weights]


class ConcatenatedDataset(torch.utils.data.ConcatDataset):
    def __init__(self, datasets: list, caching_allowed: bool = True) -> None:
        super().__init__(datasets)


class BlendedDataset(torch.utils.data.Dataset):
    def __init__(self, datasets: list, weights: list[float], size: int, path_to_cache: str | None = None,
                 caching_allowed: bool = True) -> None:
        assert len(datasets) == len(weights) < 32767
        self.datasets, self.weights, self.size = datasets, normalize(weights), size
        desc = {"class": type(self).__name__, "datasets": [d.unique_description for d in datasets],
                "weights": self.weights, "size": size}
        self.unique_description = json.dumps(desc, indent=4)
        self.unique_description_hash = hashlib.md5(self.unique_description.encode("utf-8")).hexdigest()
        self.dataset_index, self.dataset_sample_index = self._build(path_to_cache, caching_allowed)
        # every member must be able to serve the samples asked from it
        for i, d in enumerate(datasets):
            need = int(np.count_nonzero(self.dataset_index == i))
            assert need <= len(d), f"blend asks {need} samples from a dataset of {len(d)}"

    def _build(self, cache: str | None, caching_allowed: bool):
        files = None
        if cache is not None:
            base = os.path.join(cache, f"{self.unique_description_hash}-{type(self).__name__}-")
            files = [base + s for s in ("description.txt", "dataset_index.npy", "dataset_sample_index.npy")]
            if all(os.path.isfile(f) for f in files):
                return np.load(files[1], allow_pickle=True, mmap_mode="r"), \
                    np.load(files[2], allow_pickle=True, mmap_mode="r")
        di = np.zeros(self.size, dtype=np.int16)
        dsi = np.zeros(self.size, dtype=np.int64)
        build_blending_indices(di, dsi, np.asarray(self.weights), len(self.datasets), self.size)
        if files is not None and caching_allowed:
            os.makedirs(cache, exist_ok=True)
            with open(files[0], "wt") as f:
                f.write(self.unique_description)
            np.save(files[1], di, allow_pickle=True)
            np.save(files[2], dsi, allow_pickle=True)
        return di, dsi

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, idx: int) -> dict:
        d, i = int(self.dataset_index[idx]), int(self.dataset_sample_index[idx])
        return {"dataset_id": d, **self.datasets[d][i]}


def _rank0_first(make):
    """Builds on global rank 0 first (it writes the index caches), then everywhere else; only the first rank of every
    tensor-parallel group holds datasets."""
    if not ProcessGroupManager.is_initialized() or ProcessGroupManager.get_world_size() == 1:
        return make(True)
    first = ProcessGroupManager.get_global_rank() == 0
    holder = ProcessGroupManager.is_tensor_parallel_first_rank()
    ds = make(True) if (first and holder) else None
    ProcessGroupManager.barrier()
    if not first and holder:
        ds = make(False)
    return ds


def _splits_of_prefix(prefix: str, split: list[float], sizes: list[int], sequence_length: int, seed: int,
                      path_to_cache: str | None, fim_rate: float, fim_spm_rate: float, tokenizer) -> list:
    indexed = IndexedDataset(prefix)
    bounds = split_bounds(split, len(indexed.document_indices) - 1)
    out = []
    for i, name in enumerate(SPLITS):
        if split[i] == 0.0:
            out.append(None)
            continue
        docs = np.arange(bounds[i], bounds[i + 1], dtype=np.int32)
        out.append(_rank0_first(lambda allowed, docs=docs, name=name, n=sizes[i]: GPTDataset(
            indexed, docs, n, sequence_length, seed, split_name=name, path_to_cache=path_to_cache,
            fim_rate=fim_rate, fim_spm_rate=fim_spm_rate, tokenizer=tokenizer, caching_allowed=allowed)))
    return out


def _combine(members: list, weights: list[float] | None, size: int, path_to_cache: str | None):
    if any(m is None for m in members):
        assert all(m is None for m in members)
        return None
    if weights is None:
        return _rank0_first(lambda allowed: ConcatenatedDataset(members, caching_allowed=allowed))
    return _rank0_first(lambda allowed: BlendedDataset(members, weights, size, path_to_cache, allowed))


def build(sizes: list[int], sequence_length: int, tokenizer, random_seed: int, blend: list[str] | None = None,
          blend_per_split: list[list[str] | None] | None = None, split: str | None = None,
          path_to_cache: str | None = None, fim_rate: float = 0, fim_spm_rate: float = 0.5,
          node_uses_local_storage: bool = False, name: str | None = None) -> list:
    """Returns ``[train, valid, test]`` datasets (None where a split is empty)."""
    kw = dict(sequence_length=sequence_length, seed=random_seed, path_to_cache=path_to_cache, fim_rate=fim_rate,
              fim_spm_rate=fim_spm_rate, tokenizer=tokenizer)

    def from_blend(blend_list: list[str], split_vec: list[float], targets: list[int]) -> list:
        prefixes, weights = parse_blend(blend_list)
        if len(prefixes) == 1:
            return _splits_of_prefix(prefixes[0], split_vec, targets, **kw)
        concatenated = weights is None
        w = normalize([len(IndexedDataset(p)) for p in prefixes] if concatenated else weights)
        per_ds = sizes_for_blend(w, targets)
        totals = [sum(col) for col in zip(*per_ds)]
        members = [_splits_of_prefix(p, split_vec, per_ds[i], **kw) for i, p in enumerate(prefixes)]
        out = []
        for j in range(len(SPLITS)):
            col = [m[j] for m in members]
            out.append(None if split_vec[j] == 0.0 else _combine(col, None if concatenated else w, totals[j],
                                                                   path_to_cache))
        return out

    if blend_per_split is not None and any(blend_per_split):
        assert blend is None, "blend and blend_per_split are incompatible"
        assert len(blend_per_split) == len(SPLITS)
        out = []
        for i, b in enumerate(blend_per_split):
            if not b:
                out.append(None)
                continue
            vec = [0.0] * len(SPLITS)
            vec[i] = 1.0
            tg = [0] * len(SPLITS)
            tg[i] = sizes[i]
            out.append(from_blend(b, vec, tg)[i])
        return out
    assert blend is not None and split is not None, "both blend and split must be provided"
    vec = parse_and_normalize_split(split)
    log_rank_0(logging.INFO, f"split fractions = {vec}")
    return from_blend(blend, vec, sizes)
