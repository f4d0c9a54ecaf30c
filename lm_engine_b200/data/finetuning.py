"""Finetuning data: example datasets (``DebugDataset``, ``HuggingFaceDataset``), their concatenation, the collate
function (left padding with EOS, ``-100`` label masking, padding-free flattening) and the dataloader factory
(lm_engine/data/{base,debug,huggingface,finetuning,utils}.py)."""

from __future__ import annotations

import math
from functools import partial
from typing import Iterable

import torch

from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ..enums import DatasetSplit, LossMask
from ..parallel.manager import ProcessGroupManager
from .sampler import BlendedDistributedSampler

IGNORE = -100


class BaseDataset(torch.utils.data.Dataset):
    """An example is ``{"input": ids}`` (+ ``"output": ids`` ending in EOS when training; ``input`` then already
    contains the output tokens at its end)."""

    def __init__(self, class_args: dict, split: DatasetSplit, use_output: bool, tokenizer, data_name: str,
                 input_format: str = INPUT_FORMAT, output_format: str = OUTPUT_FORMAT,
                 max_input_tokens: int | None = None, max_output_tokens: int | None = None) -> None:
        super().__init__()
        self.class_args, self.split, self.use_output, self.tokenizer = class_args, split, use_output, tokenizer
        self.data_name, self.input_format, self.output_format = data_name, input_format, output_format
        self.do_format_input = input_format != INPUT_FORMAT
        self.do_format_output = output_format != OUTPUT_FORMAT
        self.max_input_tokens = max_input_tokens
        self.max_output_tokens = None if max_output_tokens is None else max_output_tokens - 1  # room for EOS
        self.examples: list[dict] = []

    def construct_input_from_format(self, text: str) -> str:
        return self.input_format.replace(INPUT_FORMAT, text, 1) if self.do_format_input else text

    def construct_output_from_format(self, text: str) -> str:
        return self.output_format.replace(OUTPUT_FORMAT, text, 1) if self.do_format_output else text

    def get_input_output_token_ids(self, input: str, output: str | None) -> dict:
        ids = list(self.tokenizer(input, add_special_tokens=False)["input_ids"])
        if self.max_input_tokens is not None:
            ids = ids[: self.max_input_tokens]
        if not self.use_output:
            return {"input": ids}
        out = list(self.tokenizer(output, add_special_tokens=False)["input_ids"])
        if self.max_output_tokens is not None:
            out = out[: self.max_output_tokens - 1]
        out.append(self.tokenizer.eos_token_id)
        return {"input": ids + out, "output": out}

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, sd: dict) -> None:
        return None

    def __getitem__(self, i: int) -> dict:
        return self.examples[i]

    def __len__(self) -> int:
        return len(self.examples)


class DebugDataset(BaseDataset):
    """``num_examples`` constant-token examples of the maximum lengths (timing / smoke tests)."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        if self.do_format_input or self.do_format_output:
            raise ValueError("DebugDataset does not support formatting")
        self._n = self.class_args.get("num_examples")
        assert isinstance(self._n, int) and self._n > 0
        self._token = self.class_args.get("token_id", getattr(self.tokenizer, "eos_token_id", 0))
        self._static = self.class_args.get("static_examples", True)
        self._example = self._make(self._token)

    def _make(self, token: int) -> dict:
        ex = {"input": [token] * self.max_input_tokens}
        if self.use_output:
            ex["output"] = [token] * (self.max_output_tokens + 1)
        return ex

    def __getitem__(self, i: int) -> dict:
        return self._example if self._static else self._make(i)

    def __len__(self) -> int:
        return self._n


class HuggingFaceDataset(BaseDataset):
    """Rows of a ``datasets`` dataset (hub name or local files) with ``input_key`` / ``output_key`` columns."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        from datasets import load_dataset

        a = self.class_args
        split = {"train": "train", "val": "validation", "test": "test"}[self.split.value]
        ds = load_dataset(a["data_path"], name=a.get("data_name"), data_files=a.get("data_files"),
                          split=a.get("split_map", {}).get(self.split.value, split))
        ik, ok = a.get("input_key", "input"), a.get("output_key", "output")
        for row in ds:
            text_in = self.construct_input_from_format(row[ik])
            text_out = self.construct_output_from_format(row[ok]) if self.use_output else None
            self.examples.append(self.get_input_output_token_ids(text_in, text_out))


_DATASET_CLASSES = {"DebugDataset": DebugDataset, "HuggingFaceDataset": HuggingFaceDataset}


class BlendedDatasets(torch.utils.data.Dataset):
    def __init__(self, datasets: list[BaseDataset], split: DatasetSplit) -> None:
        super().__init__()
        self.datasets, self.split = datasets, split
        self.index = [(d, i) for d, ds in enumerate(datasets) for i in range(len(ds))]

    def get_num_datasets(self) -> int:
        return len(self.datasets)

    def get_num_examples_in_each_dataset(self) -> list[int]:
        return [len(d) for d in self.datasets]

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, sd: dict) -> None:
        return None

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int) -> dict:
        d, j = self.index[i]
        return self.datasets[d][j]

    def __repr__(self) -> str:
        lines = [f"number of datasets = {len(self.datasets)}", f"total examples in the mixture = {len(self)}"]
        lines += [f"examples in {type(d).__name__} ({d.data_name}) = {len(d)}" for d in self.datasets]
        return "\n".join(lines)


def get_datasets_list(dataset_args_list, split: DatasetSplit, use_output: bool, tokenizer):
    datasets, ratios = [], []
    for a in dataset_args_list:
        if a.class_name not in _DATASET_CLASSES:
            raise ValueError(f"invalid class_name ({a.class_name}) for dataset")
        ds = _DATASET_CLASSES[a.class_name](a.class_args, split, use_output, tokenizer, a.data_name, a.input_format,
                                            a.output_format, a.max_input_tokens, a.max_output_tokens)
        if len(ds) > 0:
            datasets.append(ds)
            ratios.append(a.data_sampling_ratio)
    if any(r is None for r in ratios):
        ratios = None
    return datasets, ratios


def collate_fn(batch: list[dict], use_output: bool, loss_mask: LossMask, eos_token_id: int,
               use_padding_free_transformer: bool, labels_mask_value: int = IGNORE, pad_to_multiple_of: int = 1,
               device: torch.device | None = None) -> dict:
    inputs = [list(b["input"]) for b in batch]
    outputs = [list(b["output"]) for b in batch] if use_output else None
    if use_padding_free_transformer:
        if outputs is None:
            labels = None
        elif loss_mask == LossMask.output_only:
            labels = [[labels_mask_value] * (len(i) - len(o)) + o for i, o in zip(inputs, outputs)]
        elif loss_mask == LossMask.no_mask:
            labels = [list(i) for i in inputs]
        else:
            raise ValueError(f"unexpected loss_mask ({loss_mask})")
        if pad_to_multiple_of > 1:
            total = sum(len(i) for i in inputs)
            extra = math.ceil(total / pad_to_multiple_of) * pad_to_multiple_of - total
            inputs[-1] = inputs[-1] + [eos_token_id] * extra      # right padding is safe under a causal mask
            if labels is not None:
                labels[-1] = labels[-1] + [labels_mask_value] * extra
        lens = torch.tensor([0] + [len(i) for i in inputs])
        out = {"input_ids": torch.tensor([t for i in inputs for t in i], device=device),
               "position_ids": torch.tensor([p for i in inputs for p in range(len(i))], device=device),
               "cu_seqlens": lens.cumsum(0).to(torch.int32).to(device), "max_seqlen": int(lens.max())}
        if labels is not None:
            out["labels"] = torch.tensor([t for l in labels for t in l], device=device)
        return out
    width = max(len(i) for i in inputs)
    if pad_to_multiple_of > 1:
        width = math.ceil(width / pad_to_multiple_of) * pad_to_multiple_of
    out = {"input_ids": torch.tensor([[eos_token_id] * (width - len(i)) + i for i in inputs], device=device),
           "attention_mask": torch.tensor([[0] * (width - len(i)) + [1] * len(i) for i in inputs], device=device)}
    if outputs is not None:
        if loss_mask == LossMask.output_only:
            lab = [[labels_mask_value] * (width - len(o)) + o for o in outputs]
        elif loss_mask == LossMask.no_mask:
            lab = [[labels_mask_value] * (width - len(i)) + i for i in inputs]
        else:
            raise ValueError(f"unexpected loss_mask ({loss_mask})")
        out["labels"] = torch.tensor(lab, device=device)
    return out


class _LoaderIterator:
    """Iterator over a dataloader (endless when ``infinite``) that still exposes the loader's ``state_dict`` /
    ``load_state_dict``, so that a checkpoint can record and restore the sampler position.  Restoring takes effect
    on the first ``next`` (the underlying iterator is created lazily)."""

    def __init__(self, loader, infinite: bool) -> None:
        self.loader, self.infinite = loader, infinite
        self._it = None

    def __iter__(self):
        return self

    def __next__(self):
        if self._it is None:
            self._it = iter(self.loader)
        try:
            return next(self._it)
        except StopIteration:
            if not self.infinite:
                raise
            self._it = iter(self.loader)
            return next(self._it)

    def state_dict(self) -> dict:
        return self.loader.state_dict() if hasattr(self.loader, "state_dict") else {}

    def load_state_dict(self, sd: dict) -> None:
        if hasattr(self.loader, "load_state_dict"):
            self.loader.load_state_dict(sd)
        self._it = None


def custom_iterator(x: Iterable | None, infinite: bool):
    if x is None:
        return None
    return _LoaderIterator(x, infinite)


def get_finetuning_dataloader(args, tokenizer, split: str | DatasetSplit = "train"):
    """Infinite iterator over collated batches on the first rank of every tensor-parallel group, else None."""
    from .dataloader import ResumableDataLoader

    split = DatasetSplit(split) if not isinstance(split, DatasetSplit) else split
    if not ProcessGroupManager.is_tensor_parallel_first_rank():
        return None
    datasets, ratios = get_datasets_list(args.datasets, split, use_output=True, tokenizer=tokenizer)
    if not datasets:
        return None
    blended = BlendedDatasets(datasets, split)
    sampler = BlendedDistributedSampler(
        blended, ratios, num_replicas=ProcessGroupManager.get_data_loading_world_size(),
        rank=ProcessGroupManager.get_data_loading_rank(),
        ignore_sampling_proportion_for_validation=args.training_parameters.ignore_sampling_proportion_for_validation,
        is_train=split == DatasetSplit.train, shuffle=split == DatasetSplit.train, seed=args.random_args.seed)
    tp = ProcessGroupManager.get_tensor_parallel_world_size()
    loader = ResumableDataLoader(
        blended, batch_size=args.training_parameters.micro_batch_size, sampler=sampler,
        collate_fn=partial(collate_fn, use_output=True, loss_mask=args.training_parameters.loss_mask,
                           eos_token_id=getattr(tokenizer, "eos_token_id", 0),
                           use_padding_free_transformer=args.model_args.use_padding_free_transformer,
                           pad_to_multiple_of=tp if args.distributed_args.sequence_parallel else 1,
                           device=torch.device("cpu")))
    return custom_iterator(loader, infinite=split == DatasetSplit.train)
