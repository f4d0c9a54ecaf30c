"""numpy front-end of the native index builders in ``liblme_host.so`` (same results as the reference's pybind
``helpers`` module, lm_engine/data/megatron/utils/helpers.cpp)."""

from __future__ import annotations

import ctypes

import numpy as np

from ..ops._lib import host_lib


def _lib():
    lib = host_lib()
    lib.lme_num_samples.restype = ctypes.c_int64
    lib.lme_num_samples.argtypes = [ctypes.c_int64] * 3
    lib.lme_build_sample_idx.restype = ctypes.c_int
    lib.lme_build_sample_idx.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_int64, ctypes.c_void_p]
    lib.lme_build_blending_indices.restype = ctypes.c_int
    lib.lme_build_blending_indices.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                               ctypes.c_int64]
    return lib


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_epochs: int,
                     tokens_per_epoch: int) -> np.ndarray:
    """``[num_samples + 1, 2]`` array of (position in ``doc_idx``, token offset) marking where each sample of
    ``seq_length + 1`` tokens starts."""
    lib = _lib()
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    n = lib.lme_num_samples(num_epochs, int(tokens_per_epoch), seq_length)
    out = np.empty((n + 1, 2), dtype=np.int64)
    rc = lib.lme_build_sample_idx(sizes.ctypes.data, doc_idx.ctypes.data, doc_idx.size, seq_length, n,
                                  out.ctypes.data)
    if rc != 0:
        raise RuntimeError("document index exhausted while building the sample index")
    return out


def build_blending_indices(dataset_index: np.ndarray, dataset_sample_index: np.ndarray, weights: np.ndarray,
                           num_datasets: int, size: int, verbose: bool = False) -> None:
    assert dataset_index.dtype == np.int16 and dataset_sample_index.dtype == np.int64
    w = np.ascontiguousarray(weights, dtype=np.float64)
    rc = _lib().lme_build_blending_indices(dataset_index.ctypes.data, dataset_sample_index.ctypes.data,
                                           w.ctypes.data, num_datasets, size)
    if rc != 0:
        raise RuntimeError("build_blending_indices failed")


def compile_helpers() -> None:
    """Kept for API parity: the host library is built in-tree ahead of time, this only loads it."""
    host_lib()
