"""Dataloaders: ``ResumableDataLoader`` (state = dataset + sampler state) and the pretraining dataloader factory
(lm_engine/data/dataloader.py:10-16, lm_engine/data/pretraining.py:17-131)."""

from __future__ import annotations

import logging

import torch

from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ..logging_utils import log_rank_0
from ..parallel.manager import ProcessGroupManager
from .sampler import MegatronBatchSampler
from .synthetic import SyntheticBatchIterator


class ResumableDataLoader(torch.utils.data.DataLoader):
    def state_dict(self) -> dict:
        sd = {"dataset": self.dataset.state_dict() if hasattr(self.dataset, "state_dict") else {}}
        if hasattr(self.sampler, "state_dict"):
            sd["sampler"] = self.sampler.state_dict()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        if hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(sd.get("dataset", {}))
        if "sampler" in sd and hasattr(self.sampler, "load_state_dict"):
            self.sampler.load_state_dict(sd["sampler"])


def train_val_test_samples(num_training_steps: int, global_batch_size: int, eval_interval: int | None,
                           eval_steps: int | None) -> list[int]:
    eval_steps = eval_steps or 0
    n_val = 0 if not eval_interval else (num_training_steps // eval_interval + 1) * eval_steps * global_batch_size
    return [num_training_steps * global_batch_size, n_val, eval_steps * global_batch_size]


def _stack_collate(rows: list[dict]) -> dict:
    return {"text": torch.stack([torch.as_tensor(r["text"]) for r in rows])}


def _loader(ds, consumed_samples: int, micro_batch_size: int, gradient_accumulation_steps: int,
            num_pipeline_stages: int, num_workers: int):
    if ds is None:
        return None
    # a pipeline-parallel step consumes all of its micro-batches as one [mbs x accumulation, S + 1] batch
    rows = micro_batch_size if num_pipeline_stages == 1 else micro_batch_size * gradient_accumulation_steps
    sampler = MegatronBatchSampler(len(ds), consumed_samples, rows,
                                   ProcessGroupManager.get_data_loading_world_size(),
                                   ProcessGroupManager.get_data_loading_rank())
    loader = ResumableDataLoader(ds, batch_sampler=sampler, num_workers=num_workers,
                                 pin_memory=torch.cuda.is_available(), collate_fn=_stack_collate)
    return iter(loader)


def get_pretraining_dataloaders(args, tokenizer, consumed_samples: int):
    """``(train_iterator, [val_iterators], [test_iterators])``; iterators exist on the first rank of every
    tensor-parallel group only."""
    assert len(args.datasets) == 1
    dsa = args.datasets[0]
    ca = dsa.class_args
    assert dsa.max_input_tokens is None and dsa.max_output_tokens is None
    assert dsa.input_format == INPUT_FORMAT and dsa.output_format == OUTPUT_FORMAT
    tp = args.training_parameters
    n_stages = args.distributed_args.num_pipeline_stages
    if dsa.class_name == "SyntheticDataset":
        if not ProcessGroupManager.is_tensor_parallel_first_rank():
            return None, [], []
        cfg = args.model_args.pretrained_config or {}
        rows = tp.micro_batch_size if n_stages == 1 else tp.micro_batch_size * tp.gradient_accumulation_steps
        mk = lambda seed, consumed: SyntheticBatchIterator(  # noqa: E731
            ca.get("vocab_size", cfg.get("vocab_size")), ca["sequence_length"], rows,
            rank=ProcessGroupManager.get_data_loading_rank(), world=ProcessGroupManager.get_data_loading_world_size(),
            seed=seed, consumed_samples=consumed)
        seed = ca.get("seed", args.random_args.seed)
        return mk(seed, consumed_samples), [mk(seed + 1, 0)], [mk(seed + 2, 0)]
    if dsa.class_name != "MegatronDataset":
        raise ValueError(f"unexpected dataset class_name ({dsa.class_name}) for pretraining")
    from .blended import build
    from .helpers import compile_helpers

    compile_helpers()
    log_rank_0(logging.INFO, "> building train, validation, and test datasets for GPT ...")
    train_ds, val_ds, test_ds = build(
        sizes=train_val_test_samples(tp.num_training_steps, tp.global_batch_size, tp.eval_interval,
                                     ca.get("eval_steps")),
        sequence_length=ca.get("sequence_length"), blend=ca.get("data_path"),
        blend_per_split=[ca.get("train_data_path"), ca.get("val_data_path"), ca.get("test_data_path")],
        split=ca.get("split"), path_to_cache=ca.get("data_cache_path"), fim_rate=ca.get("fim_rate", 0),
        fim_spm_rate=ca.get("fim_spm_rate", 0.5), tokenizer=tokenizer,
        node_uses_local_storage=ca.get("node_uses_local_storage", False),
        random_seed=ca.get("seed", args.random_args.seed))
    log_rank_0(logging.INFO, "> finished creating GPT datasets ...")
    kw = dict(micro_batch_size=tp.micro_batch_size, gradient_accumulation_steps=tp.gradient_accumulation_steps,
              num_pipeline_stages=n_stages, num_workers=ca.get("num_workers", 2))
    val_list = val_ds if isinstance(val_ds, list) else [val_ds]
    test_list = test_ds if isinstance(test_ds, list) else [test_ds]
    return (_loader(train_ds, consumed_samples, **kw), [_loader(d, 0, **kw) for d in val_list if d is not None],
            [_loader(d, 0, **kw) for d in test_list if d is not None])
