"""String enums of the YAML schema (values are the public surface; reference: lm_engine/enums.py:8-110)."""

from __future__ import annotations

from enum import Enum


class _StrEnum(str, Enum):
    def __str__(self) -> str:  # pragma: no cover - cosmetic
        return self.value


ParamsGroupMethod = _StrEnum("ParamsGroupMethod", {"mup": "mup"})
GradientCheckpointingMethod = _StrEnum("GradientCheckpointingMethod", {"block": "block"})
LRDecaySchedule = _StrEnum("LRDecaySchedule", {k: k for k in ("constant", "cosine", "exponential", "linear", "power")})
DatasetSplit = _StrEnum("DatasetSplit", {k: k for k in ("train", "val", "test")})
TuningMethod = _StrEnum("TuningMethod", {k: k for k in ("pretraining", "full_finetuning", "distillation")})
LossMask = _StrEnum("LossMask", {k: k for k in ("output_only", "no_mask")})
KLDivergenceMethod = _StrEnum("KLDivergenceMethod", {k: k for k in ("forward", "backward")})
ExperimentsTrackerName = _StrEnum("ExperimentsTrackerName", {k: k for k in ("aim", "wandb")})
ContextParallelLoadBalancerMethod = _StrEnum("ContextParallelLoadBalancerMethod", {"headtail": "headtail"})

# Kernel names accepted in ``kernel_args.kernels`` / ENABLE_KERNELS.  In this engine every hot op already runs a
# hand-written sm_100a kernel on CUDA; the names are kept so existing YAML files validate, and a few of them still
# select behaviour (fused linear+CE, deterministic attention backward, memory-efficient RMSNorm).
_KERNEL_NAMES = (
    "causal_conv1d continuous_count cross_entropy fused_linear_cross_entropy gru linear_attention m2rnn "
    "pack_sequence rmsnorm rmsnorm_memory_efficient rnn scattermoe swiglu_packed unpack_sequence quack_gemm "
    "quack_gemm_act quack_gemm_gated quack_rmsnorm coda_linear_cross_entropy coda_linear_swiglu flash_attention_2 "
    "flash_attention_3 flash_attention_4 flash_attention_2_deterministic flash_attention_3_deterministic "
    "flash_attention_4_deterministic mamba2_ssm sonicmoe"
).split()


class Kernel(str, Enum):
    locals().update({k: k for k in _KERNEL_NAMES})

    @classmethod
    def validate_enabled(cls, kernels: list["Kernel"]) -> None:
        ks = set(kernels)
        rms = [k for k in (cls.quack_rmsnorm, cls.rmsnorm, cls.rmsnorm_memory_efficient) if k in ks]
        if cls.quack_rmsnorm in ks and len(rms) > 1:
            raise ValueError("quack_rmsnorm cannot be enabled with XMA RMSNorm kernels, got "
                             + ", ".join(k.value for k in rms))
        if cls.quack_gemm_act in ks and cls.quack_gemm_gated in ks:
            raise ValueError("quack_gemm_act cannot be enabled with quack_gemm_gated")
