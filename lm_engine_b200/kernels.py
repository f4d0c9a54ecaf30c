"""Kernel switchboard (lm_engine/kernels.py:15-123).

In this engine the CUDA kernels are always the compute path on a GPU; the named switches of the reference are kept
for config compatibility and a few still change behaviour:

* ``fused_linear_cross_entropy`` / ``coda_linear_cross_entropy``: the model skips materialising full logits and the
  loss runs the LM head chunk by chunk;
* ``flash_attention_*_deterministic``: request the deterministic attention backward;
* ``rmsnorm_memory_efficient``: recompute the normalised activations in backward.

Environment: ``ENABLE_ALL_KERNELS=1`` or ``ENABLE_KERNELS=a,b``.
"""

from __future__ import annotations

import os
from contextlib import contextmanager

from .enums import Kernel

_ENABLED: set[Kernel] = set()
if os.environ.get("ENABLE_ALL_KERNELS", "").lower() in ("1", "true"):
    _ENABLED = set(Kernel)
elif os.environ.get("ENABLE_KERNELS"):
    _ENABLED = {Kernel(k.strip()) for k in os.environ["ENABLE_KERNELS"].split(",") if k.strip()}


def is_kernel_allowed(kernel: Kernel) -> bool:
    return kernel in _ENABLED


@contextmanager
def enable_kernels(kernels: list[Kernel]):
    global _ENABLED
    old = set(_ENABLED)
    _ENABLED = _ENABLED | {Kernel(k) if not isinstance(k, Kernel) else k for k in kernels}
    try:
        yield
    finally:
        _ENABLED = old


def is_fused_linear_cross_entropy_enabled() -> bool:
    return is_kernel_allowed(Kernel.fused_linear_cross_entropy) or is_kernel_allowed(Kernel.coda_linear_cross_entropy)


def is_flash_attention_enabled() -> bool:
    return any(is_kernel_allowed(k) for k in Kernel if k.value.startswith("flash_attention"))


def is_flash_attention_deterministic() -> bool:
    return any(is_kernel_allowed(k) for k in Kernel if k.value.endswith("_deterministic"))
