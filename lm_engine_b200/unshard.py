"""``python -m lm_engine_b200.unshard --config unshard.yml``: converts a sharded training checkpoint into a single
HuggingFace-style directory (``config.json`` + safetensors + tokenizer) - lm_engine/unshard.py:10-18."""

from __future__ import annotations

from .arguments import UnshardingArgs, get_args
from .checkpointing import load_checkpoint_and_unshard
from .parallel.manager import ProcessGroupManager


def main() -> None:
    args = get_args(UnshardingArgs)
    wrapper, _, state = load_checkpoint_and_unshard(args)
    if ProcessGroupManager.get_global_rank() == 0:
        wrapper.save_pretrained(args.unsharded_path, state_dict=state)


if __name__ == "__main__":
    main()
