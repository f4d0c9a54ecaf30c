"""``python -m lm_engine_b200.data.merge``: concatenates ``.bin`` / ``.idx`` shards into larger ones, and small
inspection commands (role of tools/data/{merge_data,list_bin_files,iterate_preprocessed_data}.py).

* ``merge --input-prefixes a b c --output-prefix out``: one merged pair.
* ``merge --input-directory dir --output-prefix out [--max-size GB]``: every sub-directory is merged on its own, split
  into groups of at most ``--max-size`` GB; a ``file_map-<group>.json`` records which shards went where.
* ``list --input-directory dir``: shard prefixes with sequence / token counts.
* ``show --prefix p [--tokenizer t] [-n N]``: prints the first documents (decoded when a tokenizer is given).
"""

from __future__ import annotations

import argparse
import json
import os
from concurrent.futures import ProcessPoolExecutor

import numpy as np

from .indexed import IndexedDataset, IndexedDatasetBuilder, bin_path, idx_path


def merge_files(input_prefixes: list[str], output_prefix: str) -> None:
    assert input_prefixes, "nothing to merge"
    first = IndexedDataset(input_prefixes[0])
    os.makedirs(os.path.dirname(os.path.abspath(output_prefix)), exist_ok=True)
    builder = IndexedDatasetBuilder(bin_path(output_prefix), dtype=first.dtype)
    del first
    for p in input_prefixes:
        builder.add_index(p)
    builder.finalize(idx_path(output_prefix))


def groups_by_size(path: str, max_size_gb: float | None = None) -> list[tuple[str, list[list[str]]]]:
    """Per sub-directory, the lists of shard prefixes to merge together."""
    out = []
    for root, _, files in sorted(os.walk(path)):
        prefixes = sorted(os.path.join(root, f[:-4]) for f in files if f.endswith(".bin"))
        if not prefixes:
            continue
        if max_size_gb is None:
            out.append((root, [prefixes]))
            continue
        limit, groups, cur, size = max_size_gb * 1024**3, [], [], 0
        for p in prefixes:
            cur.append(p)
            size += os.path.getsize(p + ".bin")
            if size > limit:
                groups.append(cur)
                cur, size = [], 0
        if cur:
            groups.append(cur)
        out.append((root, groups))
    return out


def _merge_job(a) -> str:
    prefixes, dst = a
    merge_files(prefixes, dst)
    return dst


def _cmd_merge(a) -> int:
    if a.input_prefixes:
        assert a.max_size is None
        merge_files(a.input_prefixes, a.output_prefix)
        return 0
    assert a.input_directory, "give --input-prefixes or --input-directory"
    jobs = []
    for root, groups in groups_by_size(a.input_directory, a.max_size):
        rel = os.path.relpath(root, a.input_directory)
        dst_dir = os.path.normpath(os.path.join(a.output_prefix, rel))
        os.makedirs(dst_dir, exist_ok=True)
        for gid, group in enumerate(groups):
            if a.specific_group is not None and gid != a.specific_group:
                continue
            with open(os.path.join(dst_dir, f"file_map-{gid}.json"), "w") as f:
                json.dump({"subdir": root, "grp_id": gid, "group": group}, f, indent=4)
            jobs.append((group, os.path.join(dst_dir, str(gid))))
    if a.workers > 1 and len(jobs) > 1:
        with ProcessPoolExecutor(max_workers=a.workers) as pool:
            for dst in pool.map(_merge_job, jobs):
                print("merged", dst)
    else:
        for j in jobs:
            print("merged", _merge_job(j))
    return 0


def _cmd_list(a) -> int:
    total = 0
    for root, groups in groups_by_size(a.input_directory):
        for p in groups[0]:
            ds = IndexedDataset(p)
            n = int(np.asarray(ds.sequence_lengths, dtype=np.int64).sum())
            total += n
            print(f"{p}\tsequences={len(ds)}\ttokens={n}\tdtype={np.dtype(ds.dtype).name}")
    print(f"total tokens: {total}")
    return 0


def _cmd_show(a) -> int:
    ds = IndexedDataset(a.prefix)
    tok = None
    if a.tokenizer:
        from ..tokenizers import get_tokenizer

        tok = get_tokenizer(a.tokenizer)
    for i in range(min(a.n, len(ds))):
        ids = ds[i]
        print(f"--- document {i} ({len(ids)} tokens)")
        print(tok.decode(ids.tolist()) if tok is not None else ids.tolist())
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m lm_engine_b200.data.merge")
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("merge")
    m.add_argument("--input-prefixes", nargs="+", default=None)
    m.add_argument("--input-directory", default=None)
    m.add_argument("--output-prefix", required=True)
    m.add_argument("--max-size", type=float, default=None, help="GB per merged shard")
    m.add_argument("--specific-group", type=int, default=None)
    m.add_argument("--workers", type=int, default=1)
    m.set_defaults(fn=_cmd_merge)
    l = sub.add_parser("list")
    l.add_argument("--input-directory", required=True)
    l.set_defaults(fn=_cmd_list)
    s = sub.add_parser("show")
    s.add_argument("--prefix", required=True)
    s.add_argument("--tokenizer", default=None)
    s.add_argument("-n", type=int, default=3)
    s.set_defaults(fn=_cmd_show)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    raise SystemExit(main())
