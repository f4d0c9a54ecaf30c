"""lm-engine-b200: a Blackwell-native (sm_100a) engine for pretraining, finetuning and distillation of language
models with the public surface of open-lm-engine/lm-engine (YAML schema, model families, checkpoint formats)."""

__version__ = "0.1.0"
