"""Small shared helpers (reference: lm_engine/utils/*.py)."""

from __future__ import annotations

import contextlib
import importlib
import importlib.util
import os
import re
from functools import lru_cache
from typing import Any

import torch
import yaml

from .safetensors import SafeTensorsWeightsManager

# ----------------------------------------------------------------------------- arithmetic


def divide_if_divisible(dividend: int, divisor: int, msg: str = "") -> int:
    if dividend % divisor != 0:
        raise AssertionError(msg or f"{dividend} is not divisible by {divisor}")
    return dividend // divisor


def ceil_divide(a: int, b: int) -> int:
    return -(-a // b)


# ----------------------------------------------------------------------------- dtype strings

_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "fp16": torch.float16, "float16": torch.float16,
           "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}
_DTYPE_NAMES = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}


def string_to_torch_dtype(name: str) -> torch.dtype:
    if name not in _DTYPES:
        raise AssertionError(f"{name} is not a supported torch dtype")
    return _DTYPES[name]


def torch_dtype_to_string(dtype: torch.dtype) -> str:
    if dtype not in _DTYPE_NAMES:
        raise AssertionError(f"{dtype} is not a supported torch dtype")
    return _DTYPE_NAMES[dtype]


def normalize_dtype_string(name: str) -> str:
    """'bfloat16' -> 'bf16' etc.; 'fp8' / 'float8' denote block-scaled e4m3 compute with bf16 storage."""
    if name in ("fp8", "float8"):
        return "fp8"
    return torch_dtype_to_string(string_to_torch_dtype(name))


# ----------------------------------------------------------------------------- YAML

_FLOAT_RE = re.compile(
    r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
        |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
        |\.[0-9_]+(?:[eE][-+][0-9]+)?
        |[-+]?\.(?:inf|Inf|INF)
        |\.(?:nan|NaN|NAN))$""",
    re.X,
)


class _Loader(yaml.SafeLoader):
    """SafeLoader that also reads ``1e-5`` (no dot) as a float, which YAML 1.1 treats as a string."""


_Loader.add_implicit_resolver("tag:yaml.org,2002:float", _FLOAT_RE, list("-+0123456789."))


def load_yaml(path: str) -> dict:
    with open(path) as f:
        return yaml.load(f, _Loader)


# ----------------------------------------------------------------------------- misc


@lru_cache(maxsize=None)
def is_package_available(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


@contextlib.contextmanager
def environment(**env: str):
    """Temporarily set environment variables."""
    old = {k: os.environ.get(k) for k in env}
    os.environ.update({k: str(v) for k, v in env.items()})
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def get_module_class_from_name(module: torch.nn.Module, name: str) -> type | None:
    for m in module.modules():
        if type(m).__name__ == name:
            return type(m)
    return None


def setup_tf32(enabled: bool = True) -> None:
    torch.backends.cuda.matmul.allow_tf32 = enabled
    torch.backends.cudnn.allow_tf32 = enabled


_GENERATION_CACHE_ENABLED = True


def is_generation_cache_enabled() -> bool:
    return _GENERATION_CACHE_ENABLED


@contextlib.contextmanager
def disable_generation_cache():
    global _GENERATION_CACHE_ENABLED
    old, _GENERATION_CACHE_ENABLED = _GENERATION_CACHE_ENABLED, False
    try:
        yield
    finally:
        _GENERATION_CACHE_ENABLED = old


def set_attr_path(obj: Any, dotted: str, value: Any) -> None:
    parts = dotted.split(".")
    for p in parts[:-1]:
        obj = getattr(obj, p) if not isinstance(obj, dict) else obj[p]
    if isinstance(obj, dict):
        obj[parts[-1]] = value
    else:
        setattr(obj, parts[-1], value)
