"""``python -m lm_engine_b200.data.preprocess``: tokenises raw text corpora into the Megatron ``.bin`` / ``.idx`` pair
read by :class:`~lm_engine_b200.data.indexed.IndexedDataset` (role of tools/data/preprocess_data.py:60-421).

Inputs: a file or a directory of ``.jsonl``, ``.jsonl.zst`` (when ``zstandard`` is importable), ``.json.gz``,
``.parquet`` or pre-tokenised ``.arrow`` files (column ``tokens``).  One output pair is written per input file and per
``--json-keys`` entry (``<prefix>_<key>.bin/.idx``); files are spread over ``--workers`` processes.  Unparseable lines
are counted and skipped instead of aborting a long run.  Remote object stores (MSC) and Ray are deployment services
this offline package does not talk to: ``--use-ray`` / ``--msc-base-path`` are accepted and rejected with a message.
"""

from __future__ import annotations

import argparse
import gzip
import io
import json
import logging
import os
from concurrent.futures import ProcessPoolExecutor
from typing import Iterator

import numpy as np

from .indexed import IndexedDatasetBuilder, bin_path, idx_path, optimal_dtype

_SUFFIXES = (".jsonl", ".jsonl.zst", ".json.gz", ".parquet", ".arrow")
log = logging.getLogger("lm_engine_b200.preprocess")


def _load_tokenizer(name: str):
    from ..tokenizers import get_tokenizer

    return get_tokenizer(name)


class Encoder:
    def __init__(self, tokenizer, json_keys: list[str], append_eod: bool) -> None:
        self.tokenizer = _load_tokenizer(tokenizer) if isinstance(tokenizer, str) else tokenizer
        self.json_keys, self.append_eod = json_keys, append_eod

    def encode_record(self, record: dict) -> dict[str, list[int]]:
        out = {}
        for key in self.json_keys:
            ids = list(self.tokenizer.encode(record[key]))
            if ids:
                if self.append_eod:
                    ids.append(self.tokenizer.eos_token_id)
                out[key] = ids
        return out

    def encode_line(self, line: str | bytes) -> dict[str, list[int]]:
        try:
            if isinstance(line, bytes):
                line = line.decode("utf-8")
            return self.encode_record(json.loads(line))
        except (json.JSONDecodeError, KeyError, TypeError, UnicodeDecodeError):
            return {}

    def encode_tokens(self, tokens: list[int]) -> dict[str, list[int]]:
        tokens = list(tokens)
        if tokens and self.append_eod:
            tokens.append(self.tokenizer.eos_token_id)
        return {self.json_keys[0]: tokens} if tokens else {}


def _documents(path: str, enc: Encoder) -> Iterator[dict[str, list[int]]]:
    if path.endswith(".jsonl"):
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield enc.encode_line(line)
    elif path.endswith(".jsonl.zst"):
        try:
            from zstandard import ZstdDecompressor
        except ImportError as e:
            raise RuntimeError("reading .jsonl.zst needs the zstandard package") from e
        with open(path, "rb") as raw, ZstdDecompressor().stream_reader(raw) as reader:
            for line in io.BufferedReader(reader, buffer_size=64 << 20):
                yield enc.encode_line(line)
    elif path.endswith(".json.gz"):
        with gzip.open(path, "rt", encoding="utf-8") as f:
            for line in f:
                yield enc.encode_line(line)
    elif path.endswith(".parquet"):
        import pyarrow.parquet as pq

        for batch in pq.ParquetFile(path).iter_batches(columns=enc.json_keys, batch_size=10000):
            for row in batch.to_pylist():
                try:
                    yield enc.encode_record(row)
                except (KeyError, TypeError):
                    yield {}
    elif path.endswith(".arrow"):
        import pyarrow as pa

        reader = pa.ipc.open_file(path)
        for i in range(reader.num_record_batches):
            yield enc.encode_tokens(reader.get_batch(i)["tokens"].to_numpy().tolist())
    else:
        raise ValueError(f"unsupported input {path}; known suffixes: {_SUFFIXES}")


def convert_file(tokenizer, input_file: str, output_prefix: str, json_keys: list[str] | None = None,
                 append_eos_token: bool = True) -> int:
    """Tokenises one file.  Returns the number of skipped (unparseable / empty) records."""
    json_keys = json_keys or ["text"]
    enc = Encoder(tokenizer, json_keys, append_eos_token)
    vocab = getattr(enc.tokenizer, "vocab_size", None) or len(enc.tokenizer)
    dtype = optimal_dtype(vocab)
    os.makedirs(os.path.dirname(os.path.abspath(output_prefix)), exist_ok=True)
    builders = {k: IndexedDatasetBuilder(bin_path(f"{output_prefix}_{k}"), dtype=dtype) for k in json_keys}
    skipped = 0
    for doc in _documents(input_file, enc):
        if not doc:
            skipped += 1
            continue
        for key, ids in doc.items():
            builders[key].add_item(np.asarray(ids, dtype=dtype))
            builders[key].end_document()
    for k in json_keys:
        builders[k].finalize(idx_path(f"{output_prefix}_{k}"))
    return skipped


def _job(a) -> tuple[str, int, str | None]:
    tokenizer, src, dst, keys, eod = a
    try:
        return src, convert_file(tokenizer, src, dst, keys, eod), None
    except Exception as e:  # noqa: BLE001 - a bad shard must not stop the others
        return src, 0, f"{type(e).__name__}: {e}"


def collect_inputs(path: str) -> list[str]:
    if os.path.isfile(path):
        return [path]
    found = []
    for root, _, files in os.walk(path):
        found += [os.path.join(root, f) for f in files if f.endswith(_SUFFIXES)]
    return sorted(found)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m lm_engine_b200.data.preprocess")
    ap.add_argument("--input", required=True, help="file or directory of jsonl / jsonl.zst / json.gz / parquet / arrow")
    ap.add_argument("--json-keys", nargs="+", default=["text"])
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--append-eod", action="store_true")
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--use-ray", action="store_true")
    ap.add_argument("--msc-base-path", default=None)
    a = ap.parse_args(argv)
    if a.use_ray or a.msc_base_path:
        ap.error("Ray clusters and MSC object stores are not reachable from this package; run with --workers on "
                 "local files")
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s")
    inputs = collect_inputs(a.input)
    assert inputs, f"no input files under {a.input}"
    single = os.path.isfile(a.input)
    jobs = []
    for src in inputs:
        if single:
            dst = a.output_prefix
        else:
            rel = os.path.relpath(src, a.input)
            for suf in sorted(_SUFFIXES, key=len, reverse=True):
                if rel.endswith(suf):
                    rel = rel[: -len(suf)]
                    break
            dst = os.path.join(a.output_prefix, rel)
        jobs.append((a.tokenizer, src, dst, a.json_keys, a.append_eod))
    failed = 0
    if a.workers <= 1 or len(jobs) == 1:
        results = map(_job, jobs)
    else:
        pool = ProcessPoolExecutor(max_workers=a.workers)
        results = pool.map(_job, jobs)
    for src, skipped, err in results:
        if err is not None:
            failed += 1
            log.error("FAILED %s: %s", src, err)
        else:
            log.info("done %s (skipped %d records)", src, skipped)
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
