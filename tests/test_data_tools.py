"""Corpus tools: jsonl / parquet -> .bin/.idx, merge, and reading the result back through the dataset classes."""

import json
import os

import numpy as np


class _Tok:
    vocab_size = 300
    eos_token_id = 299

    def encode(self, text):
        return [ord(c) % 256 for c in text]

    def decode(self, ids):
        return "".join(chr(i) for i in ids if i < 256)


def _write_jsonl(path, docs, bad_line=False):
    with open(path, "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")
        if bad_line:
            f.write("{not json\n")


def test_preprocess_and_merge_roundtrip(tmp_path):
    from lm_engine_b200.data.indexed import IndexedDataset
    from lm_engine_b200.data.merge import groups_by_size, main as merge_main, merge_files
    from lm_engine_b200.data.preprocess import convert_file

    docs_a, docs_b = ["hello world", "abc", "x" * 50], ["second file", "zz"]
    _write_jsonl(tmp_path / "a.jsonl", docs_a, bad_line=True)
    _write_jsonl(tmp_path / "b.jsonl", docs_b)
    skipped = convert_file(_Tok(), str(tmp_path / "a.jsonl"), str(tmp_path / "out" / "a"), ["text"], True)
    assert skipped == 1
    assert convert_file(_Tok(), str(tmp_path / "b.jsonl"), str(tmp_path / "out" / "b"), ["text"], True) == 0
    a = IndexedDataset(str(tmp_path / "out" / "a_text"))
    assert len(a) == 3 and a.dtype == np.uint16
    assert a[0].tolist() == [ord(c) for c in "hello world"] + [299]
    merge_files([str(tmp_path / "out" / "a_text"), str(tmp_path / "out" / "b_text")], str(tmp_path / "m" / "all"))
    m = IndexedDataset(str(tmp_path / "m" / "all"))
    assert len(m) == 5
    for i, d in enumerate(docs_a + docs_b):
        assert _Tok().decode(m[i].tolist()[:-1]) == d
    assert m.document_indices.tolist() == [0, 1, 2, 3, 4, 5]
    # directory mode with a size cap that forces one shard per group
    groups = groups_by_size(str(tmp_path / "out"), max_size_gb=1e-9)
    assert [len(g) for _, gs in groups for g in gs] == [1, 1]
    assert merge_main(["merge", "--input-directory", str(tmp_path / "out"), "--output-prefix",
                       str(tmp_path / "dir")]) == 0
    assert len(IndexedDataset(str(tmp_path / "dir" / "0"))) == 5
    assert os.path.isfile(tmp_path / "dir" / "file_map-0.json")


def test_preprocess_parquet_and_multiple_keys(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq

    from lm_engine_b200.data.indexed import IndexedDataset
    from lm_engine_b200.data.preprocess import convert_file

    pq.write_table(pa.table({"text": ["one", "two", ""], "code": ["x=1", "y=2", "z=3"]}), tmp_path / "d.parquet")
    convert_file(_Tok(), str(tmp_path / "d.parquet"), str(tmp_path / "o"), ["text", "code"], False)
    assert len(IndexedDataset(str(tmp_path / "o_text"))) == 2      # the empty document is dropped
    c = IndexedDataset(str(tmp_path / "o_code"))
    assert len(c) == 3 and c[2].tolist() == [ord(ch) for ch in "z=3"]
