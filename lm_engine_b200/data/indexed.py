"""Megatron ``.bin`` / ``.idx`` indexed token datasets: memory-mapped reader and streaming writer.

On-disk format (bit-compatible with the reference, lm_engine/data/megatron/indexed_dataset/*.py and dtype.py):
``.idx`` = magic ``MMIDIDX\\0\\0`` | u64 version (1) | u8 dtype code | u64 #sequences | u64 #document-boundaries |
int32 sequence lengths | int64 byte offsets | int64 document boundaries [| int8 modes]; ``.bin`` = raw tokens.
"""

from __future__ import annotations

import os
import shutil
import struct

import numpy as np

_MAGIC = b"MMIDIDX\x00\x00"
_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODE_OF = {np.dtype(v).name: k for k, v in _CODES.items()}


def optimal_dtype(cardinality: int | None) -> type:
    """uint16 when the vocabulary fits, else int32."""
    return np.uint16 if cardinality is not None and cardinality < 65500 else np.int32


def idx_path(prefix: str) -> str:
    return prefix + ".idx"


def bin_path(prefix: str) -> str:
    return prefix + ".bin"


class IndexedDataset:
    """Random access to the sequences of one ``prefix.{bin,idx}`` pair through ``np.memmap``."""

    def __init__(self, path_prefix: str, multimodal: bool = False) -> None:
        self.path_prefix, self.multimodal = path_prefix, multimodal
        self._open()

    def _open(self) -> None:
        with open(idx_path(self.path_prefix), "rb") as f:
            assert f.read(9) == _MAGIC, "bad magic in .idx file"
            (version,) = struct.unpack("<Q", f.read(8))
            assert version == 1
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = _CODES[code]
            (n_seq,) = struct.unpack("<Q", f.read(8))
            (n_doc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._idx = np.memmap(idx_path(self.path_prefix), mode="r", order="C")
        self.sequence_lengths = np.frombuffer(self._idx, dtype=np.int32, count=n_seq, offset=offset)
        offset += self.sequence_lengths.nbytes
        self.sequence_pointers = np.frombuffer(self._idx, dtype=np.int64, count=n_seq, offset=offset)
        offset += self.sequence_pointers.nbytes
        self.document_indices = np.frombuffer(self._idx, dtype=np.int64, count=n_doc, offset=offset)
        offset += self.document_indices.nbytes
        self.sequence_modes = None
        if self.multimodal:
            self.sequence_modes = np.frombuffer(self._idx, dtype=np.int8, count=n_seq, offset=offset)
        self._bin = np.memmap(bin_path(self.path_prefix), mode="r", order="C")

    def __getstate__(self):
        return self.path_prefix, self.multimodal

    def __setstate__(self, state) -> None:
        self.path_prefix, self.multimodal = state
        self._open()

    def __len__(self) -> int:
        return len(self.sequence_lengths)

    def get(self, idx: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        n = int(self.sequence_lengths[idx]) - offset if length is None else length
        start = int(self.sequence_pointers[idx]) + offset * np.dtype(self.dtype).itemsize
        return np.frombuffer(self._bin, dtype=self.dtype, count=n, offset=start)

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            seq = self.get(int(idx))
            return (seq, self.sequence_modes[idx]) if self.multimodal else seq
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            assert step == 1, "slices into the dataset must be contiguous"
            lens = self.sequence_lengths[idx]
            flat = np.frombuffer(self._bin, dtype=self.dtype, count=int(lens.sum()),
                                 offset=int(self.sequence_pointers[start]))
            return np.split(flat, np.cumsum(lens)[:-1])
        raise TypeError(f"unexpected index type {type(idx)}")

    @staticmethod
    def exists(path_prefix: str) -> bool:
        return os.path.exists(idx_path(path_prefix)) and os.path.exists(bin_path(path_prefix))


class IndexedDatasetBuilder:
    """Streams tokens into ``bin_file`` and writes the matching index in :meth:`finalize`."""

    def __init__(self, bin_file: str, dtype=np.int32, multimodal: bool = False) -> None:
        self._f = open(bin_file, "wb")
        self.dtype, self.multimodal = dtype, multimodal
        self.sequence_lengths: list[int] = []
        self.document_indices: list[int] = [0]
        self.sequence_modes: list[int] | None = [] if multimodal else None

    def add_item(self, tokens, mode: int = 0) -> None:
        arr = np.asarray(tokens.numpy() if hasattr(tokens, "numpy") else tokens, dtype=self.dtype)
        self._f.write(arr.tobytes(order="C"))
        self.sequence_lengths.append(arr.size)
        if self.multimodal:
            self.sequence_modes.append(mode)

    def add_document(self, tokens, lengths: list[int], modes: list[int] | None = None) -> None:
        arr = np.asarray(tokens.numpy() if hasattr(tokens, "numpy") else tokens, dtype=self.dtype)
        self._f.write(arr.tobytes(order="C"))
        self.sequence_lengths.extend(lengths)
        self.document_indices.append(len(self.sequence_lengths))
        if self.multimodal:
            self.sequence_modes.extend(modes if modes is not None else [0] * len(lengths))

    def end_document(self) -> None:
        self.document_indices.append(len(self.sequence_lengths))

    def add_index(self, path_prefix: str) -> None:
        """Appends another dataset (merge)."""
        other = IndexedDataset(path_prefix, self.multimodal)
        assert other.dtype == self.dtype
        base = len(self.sequence_lengths)
        self.sequence_lengths.extend(other.sequence_lengths.tolist())
        self.document_indices.extend((base + other.document_indices[1:]).tolist())
        if self.multimodal:
            self.sequence_modes.extend(other.sequence_modes.tolist())
        with open(bin_path(path_prefix), "rb") as f:
            shutil.copyfileobj(f, self._f)

    def finalize(self, idx_file: str) -> None:
        self._f.close()
        lens = np.asarray(self.sequence_lengths, dtype=np.int32)
        item = np.dtype(self.dtype).itemsize
        ptrs = np.zeros(len(lens), dtype=np.int64)
        if len(lens) > 1:
            np.cumsum(lens[:-1].astype(np.int64) * item, out=ptrs[1:])
        with open(idx_file, "wb") as f:
            f.write(_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", _CODE_OF[np.dtype(self.dtype).name]))
            f.write(struct.pack("<Q", len(lens)))
            f.write(struct.pack("<Q", len(self.document_indices)))
            f.write(lens.tobytes(order="C"))
            f.write(ptrs.tobytes(order="C"))
            f.write(np.asarray(self.document_indices, dtype=np.int64).tobytes(order="C"))
            if self.multimodal:
                f.write(np.asarray(self.sequence_modes, dtype=np.int8).tobytes(order="C"))


# names used by the reference
MMapIndexedDataset = IndexedDataset
MMapIndexedDatasetBuilder = IndexedDatasetBuilder
