"""Seeded synthetic token data for pretraining benchmarks and tests.

``class_name: SyntheticDataset`` in the ``datasets`` section (an extension: the reference's pretraining path accepts
only Megatron ``.bin/.idx`` data, lm_engine/data/pretraining.py:78-111).  Every sample is ``sequence_length + 1``
uniform-random int64 ids in ``[0, vocab_size)`` drawn from a counter-based generator, so sample ``i`` is the same
whatever the rank layout and resuming is exact by sample index.
"""

from __future__ import annotations

import torch


class SyntheticDataset(torch.utils.data.Dataset):
    def __init__(self, vocab_size: int, sequence_length: int, num_samples: int, seed: int = 1234) -> None:
        self.vocab_size, self.sequence_length, self.num_samples, self.seed = (vocab_size, sequence_length,
                                                                              num_samples, seed)

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, i: int) -> dict:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        return {"text": torch.randint(0, self.vocab_size, (self.sequence_length + 1,), generator=g)}


class SyntheticBatchIterator:
    """Yields pinned ``[micro_batch, sequence_length + 1]`` batches for data-loading rank ``rank`` of ``world``;
    ``consumed_samples`` (global) positions the stream for resume."""

    def __init__(self, vocab_size: int, sequence_length: int, micro_batch_size: int, rank: int = 0, world: int = 1,
                 seed: int = 1234, consumed_samples: int = 0, pin_memory: bool = True) -> None:
        self.ds = SyntheticDataset(vocab_size, sequence_length, 1 << 62, seed)
        self.mbs, self.rank, self.world = micro_batch_size, rank, world
        self.cursor = consumed_samples
        self.pin = pin_memory and torch.cuda.is_available()
        # one generator per stream position keeps batches reproducible but avoids per-sample generator set-up
        self.vocab_size, self.sequence_length, self.seed = vocab_size, sequence_length, seed

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        start = self.cursor + self.rank * self.mbs
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + start)
        t = torch.randint(0, self.vocab_size, (self.mbs, self.sequence_length + 1), generator=g)
        if self.pin:
            t = t.pin_memory()
        self.cursor += self.mbs * self.world
        return {"text": t}
