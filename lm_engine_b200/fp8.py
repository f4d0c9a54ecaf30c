"""``mixed_precision_args.dtype: fp8``: routes the linear layers of the transformer blocks through the 8-bit tensor
core path (tensor-wise dynamic scaling: e4m3 activations / weights, e5m2 output gradients; bf16 master-weight
copies, fp32 optimizer state).  Role of lm_engine/fp8.py:53-103, which delegates to torchao.

The LM head, embeddings, routers, norms and every layer whose sizes are not multiples of 16 stay in bf16.  Scaling
is *dynamic* (scale from the tensor being cast), so there is no amax history to synchronise between ranks and
nothing to pre-compute for the sharded all-gather: the two per-step hooks of the reference API are kept as no-ops.
"""

from __future__ import annotations

import logging

import torch.nn as nn

from .logging_utils import log_rank_0


def _is_block_linear(fqn: str, module: nn.Module) -> bool:
    from .models.layers.linear import ParameterizedLinear

    if not isinstance(module, ParameterizedLinear):
        return False
    if "lm_head" in fqn or fqn == "output" or "gate" in fqn.split(".")[-1:]:
        return False
    w = module.weight
    return w.dim() == 2 and w.size(0) % 16 == 0 and w.size(1) % 16 == 0


def convert_to_fp8_training(model: nn.Module, module_filter_fn=None, scaling: str | None = None) -> int:
    """Flags the weights of eligible linear layers; ``ops.linear`` / ``ops.linear_swiglu`` dispatch on the flag.
    Returns the number of converted layers.  ``scaling`` (default: ``LME_FP8_SCALING``, else ``tensor``):
    ``tensor`` = tensor-wise dynamic scales on the 8-bit tensor-core GEMM; ``block`` = the numerics of 1 x 128
    activation / 128 x 128 weight scales (``ops/fp8_block.py``: operands rounded to block-scaled e4m3, products still
    on the bf16 GEMM) for layers whose sizes are multiples of 128, tensor-wise for the rest."""
    import os

    scaling = scaling or os.environ.get("LME_FP8_SCALING", "tensor")
    assert scaling in ("tensor", "block"), scaling
    n = blocks = 0
    for fqn, m in model.named_modules():
        if not _is_block_linear(fqn, m):
            continue
        if module_filter_fn is not None and not module_filter_fn(m, fqn):
            continue
        w = m.weight
        if scaling == "block" and w.size(0) % 128 == 0 and w.size(1) % 128 == 0:
            w.fp8 = "block"
            blocks += 1
        else:
            w.fp8 = True
        n += 1
    log_rank_0(logging.INFO, f"fp8: {n} linear layers converted ({blocks} with block-scaled numerics, "
               f"{n - blocks} on the tensor-wise 8-bit tensor core path)")
    return n


class FP8Manager:
    """API-compatible holder of the reference's per-step FP8 hooks (lm_engine/fp8.py:53-103)."""

    def __init__(self, model_container, **_unused) -> None:
        for w in model_container:
            convert_to_fp8_training(w.model)

    @staticmethod
    def precompute_float8_dynamic_scale_for_fsdp(model_container) -> None:
        return None

    @staticmethod
    def sync_float8_amax_and_scale_history(model_container) -> None:
        return None
