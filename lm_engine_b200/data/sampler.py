"""Samplers: the resumable pretraining batch sampler (position = globally consumed samples) and the ratio-based
distributed sampler over several finetuning datasets (lm_engine/data/megatron/sampler.py:8-54,
lm_engine/data/sampler.py)."""

from __future__ import annotations

import math

import torch


class MegatronBatchSampler:
    """Yields this rank's ``micro_batch_size`` indices out of every global slab of ``micro_batch_size x
    num_replicas`` consecutive samples, starting at ``consumed_samples``."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, num_replicas: int,
                 rank: int, drop_last: bool = True) -> None:
        assert total_samples > 0, f"no sample to consume: {total_samples}"
        assert consumed_samples < total_samples, f"no samples left to consume: {consumed_samples}, {total_samples}"
        assert micro_batch_size > 0
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.num_replicas, self.rank, self.drop_last = (micro_batch_size, num_replicas, rank,
                                                                               drop_last)

    def __len__(self) -> int:
        return self.total_samples

    def __iter__(self):
        slab = self.micro_batch_size * self.num_replicas
        lo = self.rank * self.micro_batch_size
        pos = self.consumed_samples
        while pos + slab <= self.total_samples:
            yield list(range(pos + lo, pos + lo + self.micro_batch_size))
            pos += slab
        if pos < self.total_samples and not self.drop_last:
            tail = list(range(pos, self.total_samples))
            yield tail[lo:lo + self.micro_batch_size]


class BlendedDistributedSampler(torch.utils.data.DistributedSampler):
    """Infinite-epoch sampler over a concatenation of datasets in which dataset ``i`` contributes in proportion to
    ``data_sampling_ratios[i]`` (or to its size); every rank draws a disjoint strided slice; resumable."""

    def __init__(self, dataset, data_sampling_ratios: list[int] | None, num_replicas: int, rank: int,
                 ignore_sampling_proportion_for_validation: bool = True, is_train: bool = True, shuffle: bool = True,
                 seed: int = 0, drop_last: bool = False) -> None:
        super().__init__(dataset, num_replicas=num_replicas, rank=rank, shuffle=shuffle, seed=seed,
                         drop_last=drop_last)
        self.sizes = dataset.get_num_examples_in_each_dataset()
        self.starts = [0]
        for n in self.sizes[:-1]:
            self.starts.append(self.starts[-1] + n)
        self.total = sum(self.sizes)
        use_ratio = data_sampling_ratios is not None and (is_train or not ignore_sampling_proportion_for_validation)
        if use_ratio:
            r = [float(x) for x in data_sampling_ratios]
            s = sum(r)
            self.per_dataset = [max(1, int(self.total * x / s)) for x in r]
        else:
            self.per_dataset = list(self.sizes)
        self.num_samples_total = sum(self.per_dataset)
        self.index = 0
        self.generator = torch.Generator()
        self.generator.manual_seed(seed)

    def _epoch_indices(self) -> list[int]:
        picks = []
        for start, size, want in zip(self.starts, self.sizes, self.per_dataset):
            if self.shuffle:
                reps = math.ceil(want / size)
                perm = torch.cat([torch.randperm(size, generator=self.generator) for _ in range(reps)])[:want]
            else:
                perm = torch.arange(want) % size
            picks.append(perm + start)
        allidx = torch.cat(picks)
        if self.shuffle:
            allidx = allidx[torch.randperm(len(allidx), generator=self.generator)]
        return allidx.tolist()

    def __iter__(self):
        while True:
            # the permutation of this epoch is drawn from here: a resume inside the epoch must redraw the same one
            self._epoch_generator_state = self.generator.get_state()
            idx = self._epoch_indices()
            mine = idx[self.rank::self.num_replicas]
            for i in mine[self.index:]:
                self.index += 1
                yield i
            self.index = 0
            self.epoch += 1

    def __len__(self) -> int:
        return self.num_samples_total // self.num_replicas

    def state_dict(self) -> dict:
        state = getattr(self, "_epoch_generator_state", None)
        return {"epoch": self.epoch, "index": self.index,
                "generator": state if state is not None else self.generator.get_state()}

    def load_state_dict(self, sd: dict) -> None:
        self.epoch, self.index = sd["epoch"], sd["index"]
        self.generator.set_state(sd["generator"])
