"""GPT pretraining dataset over an indexed token file: every sample is ``sequence_length + 1`` consecutive tokens of
the (epoch-wise shuffled) document stream, samples are visited in shuffled order, and the three index arrays are
cached as ``.npy`` keyed by an md5 of the dataset description (lm_engine/data/megatron/gpt_dataset.py:29-525).
Optional fill-in-the-middle transformation (PSM / SPM)."""

from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from .helpers import build_sample_idx
from .indexed import IndexedDataset


def _num_epochs(tokens_per_epoch: int, seq_length: int, num_samples: int) -> int:
    epochs, tokens = 0, 0
    while True:
        epochs += 1
        tokens += tokens_per_epoch
        if (tokens - 1) // seq_length >= num_samples:
            return epochs


def _document_index(documents: np.ndarray, num_epochs: int, rng: np.random.RandomState,
                    separate_final_epoch: bool) -> np.ndarray:
    if not separate_final_epoch or num_epochs == 1:
        idx = np.tile(documents, num_epochs).astype(documents.dtype)
        rng.shuffle(idx)
        return idx
    return np.concatenate((_document_index(documents, num_epochs - 1, rng, False),
                           _document_index(documents, 1, rng, False)))


def _shuffle_index(num_samples: int, total_size: int, rng: np.random.RandomState) -> np.ndarray:
    dt = np.int64 if total_size >= np.iinfo(np.uint32).max - 1 else np.uint32
    first = np.arange(num_samples, dtype=dt)
    rng.shuffle(first)
    if num_samples == total_size:
        return first
    last = np.arange(num_samples, total_size, dtype=dt)
    rng.shuffle(last)
    return np.concatenate((first, last))


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, indexed_dataset: IndexedDataset, indexed_indices: np.ndarray, num_samples: int,
                 sequence_length: int, random_seed: int, split_name: str = "train", path_to_cache: str | None = None,
                 fim_rate: float = 0, fim_spm_rate: float = 0.5, tokenizer=None, caching_allowed: bool = True) -> None:
        self.indexed_dataset, self.indexed_indices = indexed_dataset, np.asarray(indexed_indices, dtype=np.int32)
        self.num_samples, self.sequence_length, self.random_seed = num_samples, sequence_length, random_seed
        self.split_name, self.path_to_cache = split_name, path_to_cache
        self.fim_rate, self.fim_spm_rate, self.tokenizer = fim_rate, fim_spm_rate, tokenizer
        self.caching_allowed = caching_allowed
        desc = {"class": type(self).__name__, "path_prefix": indexed_dataset.path_prefix,
                "num_samples": num_samples, "index_split": split_name, "random_seed": random_seed,
                "sequence_length": sequence_length,
                "split_range": [int(self.indexed_indices[0]), int(self.indexed_indices[-1])]}
        self.unique_description = json.dumps(desc, indent=4)
        self.unique_description_hash = hashlib.md5(self.unique_description.encode("utf-8")).hexdigest()
        self.document_index, self.sample_index, self.shuffle_index = self._build_indices()
        if fim_rate > 0:
            assert tokenizer is not None, "fill-in-the-middle needs a tokenizer"
            self._fim_rng = np.random.RandomState(random_seed)
            ids = {t: tokenizer.convert_tokens_to_ids(t) for t in ("<fim_prefix>", "<fim_middle>", "<fim_suffix>",
                                                                    "<fim_pad>")}
            self._fim_ids = ids

    # ------------------------------------------------------------------ indices
    def _build_indices(self):
        cache = self.path_to_cache or os.path.join(os.path.dirname(self.indexed_dataset.path_prefix) or ".", "cache",
                                                   f"{type(self).__name__}_indices")
        base = os.path.join(cache, f"{self.unique_description_hash}-{type(self).__name__}-")
        files = [base + s for s in ("description.txt", "document_index.npy", "sample_index.npy", "shuffle_index.npy")]
        tokens_per_epoch = int(np.sum(self.indexed_dataset.sequence_lengths[self.indexed_indices]))
        epochs = _num_epochs(tokens_per_epoch, self.sequence_length, self.num_samples)
        if not all(os.path.isfile(f) for f in files):
            separate, sans_final = False, 0
            if epochs > 1:
                sans_final = ((epochs - 1) * tokens_per_epoch - 1) // self.sequence_length
                from_final = self.num_samples - sans_final
                per_epoch = (tokens_per_epoch - 1) // self.sequence_length
                assert 0 <= from_final <= per_epoch + 1
                separate = from_final < int(0.80 * per_epoch)
            rng = np.random.RandomState(self.random_seed)
            doc_index = _document_index(self.indexed_indices, epochs, rng, separate)
            sample_index = build_sample_idx(self.indexed_dataset.sequence_lengths, doc_index, self.sequence_length,
                                            epochs, tokens_per_epoch)
            total = sample_index.shape[0] - 1
            shuffle_index = _shuffle_index(sans_final if separate else total, total, rng)
            if not self.caching_allowed:
                return doc_index, sample_index, shuffle_index
            os.makedirs(cache, exist_ok=True)
            with open(files[0], "wt") as f:
                f.write(self.unique_description)
            np.save(files[1], doc_index, allow_pickle=True)
            np.save(files[2], sample_index, allow_pickle=True)
            np.save(files[3], shuffle_index, allow_pickle=True)
        return tuple(np.load(f, allow_pickle=True, mmap_mode="r") for f in files[1:])

    # ------------------------------------------------------------------ access
    def __len__(self) -> int:
        return self.sample_index.shape[0] - 1

    def _tokens(self, idx: int) -> np.ndarray:
        idx = int(self.shuffle_index[idx])
        d0, o0 = (int(x) for x in self.sample_index[idx])
        d1, o1 = (int(x) for x in self.sample_index[idx + 1])
        if d0 == d1:
            return np.asarray(self.indexed_dataset.get(int(self.document_index[d0]), o0, o1 - o0 + 1), dtype=np.int64)
        parts = [self.indexed_dataset.get(int(self.document_index[d0]), o0)]
        parts += [self.indexed_dataset.get(int(self.document_index[d])) for d in range(d0 + 1, d1)]
        parts.append(self.indexed_dataset.get(int(self.document_index[d1]), 0, o1 + 1))
        return np.concatenate(parts).astype(np.int64)

    def __getitem__(self, idx: int) -> dict[str, np.ndarray]:
        text = self._tokens(idx)
        if self.fim_rate > 0:
            text = self._apply_fim(text)
        return {"text": text}

    # ------------------------------------------------------------------ fill in the middle
    def _apply_fim(self, sample: np.ndarray) -> np.ndarray:
        eod = self.tokenizer.eos_token_id
        pieces, out = np.split(sample, np.where(sample == eod)[0] + 1), []
        for piece in pieces:
            body = piece[:-1] if len(piece) and piece[-1] == eod else piece
            if len(body) > 0 and self._fim_rng.binomial(1, self.fim_rate):
                body = self._permute(body)
            out.append(np.concatenate((body, piece[len(piece) - 1:])) if len(piece) and piece[-1] == eod else body)
        res = np.concatenate(out) if out else sample
        n = len(sample)
        if len(res) < n:
            res = np.concatenate((res, np.full(n - len(res), self._fim_ids["<fim_pad>"])))
        return res[:n].astype(np.int64)

    def _permute(self, tokens: np.ndarray) -> np.ndarray:
        text = self.tokenizer.decode(tokens)
        a, b = sorted(self._fim_rng.randint(0, len(text) + 1, size=2))
        enc = lambda s: np.asarray(self.tokenizer.encode(s), dtype=np.int64)  # noqa: E731
        prefix, middle, suffix = enc(text[:a]), enc(text[a:b]), enc(text[b:])
        extra = len(prefix) + len(middle) + len(suffix) + 3 - len(tokens)
        if extra > 0:
            if len(suffix) <= extra:
                return tokens
            suffix = suffix[:len(suffix) - extra]
        elif extra < 0:
            suffix = np.concatenate((suffix, np.full(-extra, self._fim_ids["<fim_pad>"])))
        p, m, s = self._fim_ids["<fim_prefix>"], self._fim_ids["<fim_middle>"], self._fim_ids["<fim_suffix>"]
        if self._fim_rng.binomial(1, self.fim_spm_rate):
            return np.concatenate(([p, s], suffix, [m], prefix, middle))
        return np.concatenate(([p], prefix, [s], suffix, [m], middle))
