"""lm-engine-b200: a Blackwell-native (sm_100a) engine for pretraining, finetuning and distillation of language
models with the public surface of open-lm-engine/lm-engine (YAML schema, model families, checkpoint formats)."""

import os as _os

__version__ = "0.1.0"

# The engine overlaps compute with kernels of its own that wait (bounded) for another GPU: the fused gradient
# reduce-scatter, the fused tensor-parallel GEMMs.  Such a kernel must never sit in front of unrelated work in one
# hardware queue, so every stream gets a queue of its own (the driver's default of 8 can alias the compute, gather,
# reduction and library streams).  Read by the driver when the CUDA context is created; an explicit setting wins.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
