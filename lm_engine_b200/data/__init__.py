"""Data pipeline: Megatron indexed datasets and blends for pretraining, example datasets for finetuning, a seeded
synthetic token stream, samplers and resumable dataloaders."""

from .blended import BlendedDataset, ConcatenatedDataset, build
from .dataloader import ResumableDataLoader, get_pretraining_dataloaders
from .finetuning import (
    BaseDataset,
    BlendedDatasets,
    DebugDataset,
    HuggingFaceDataset,
    collate_fn,
    custom_iterator,
    get_datasets_list,
    get_finetuning_dataloader,
)
from .gpt_dataset import GPTDataset
from .indexed import IndexedDataset, IndexedDatasetBuilder, MMapIndexedDataset, MMapIndexedDatasetBuilder
from .sampler import BlendedDistributedSampler, MegatronBatchSampler
from .synthetic import SyntheticBatchIterator, SyntheticDataset


def get_next_batch(x):
    return None if x is None else next(x)
