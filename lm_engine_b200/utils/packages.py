"""Probes for optional third-party packages (reference: lm_engine/utils/packages.py:8-245).

This engine carries its own kernels, so only the observability / data packages are optional.
"""

from __future__ import annotations

from . import is_package_available


def _probe(name: str):
    def f() -> bool:
        return is_package_available(name)

    f.__name__ = f"is_{name}_available"
    return f


is_wandb_available = _probe("wandb")
is_aim_available = _probe("aim")
is_colorlog_available = _probe("colorlog")
is_zstandard_available = _probe("zstandard")
is_ray_available = _probe("ray")
is_datasets_available = _probe("datasets")
is_multi_storage_client_available = _probe("multistorageclient")
is_transformers_available = _probe("transformers")
is_safetensors_available = _probe("safetensors")
is_pyarrow_available = _probe("pyarrow")
is_git_available = _probe("git")
