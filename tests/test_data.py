"""Indexed dataset format, native index builders, GPT dataset coverage, blends, samplers, tokenizer (CPU)."""

import os

import numpy as np
import pytest
import torch

from lm_engine_b200.data import (
    BlendedDataset,
    GPTDataset,
    IndexedDataset,
    IndexedDatasetBuilder,
    MegatronBatchSampler,
    build,
)
from lm_engine_b200.data.helpers import build_blending_indices, build_sample_idx


def _write(prefix, docs, dtype=np.int32):
    b = IndexedDatasetBuilder(prefix + ".bin", dtype=dtype)
    for d in docs:
        b.add_item(np.asarray(d))
        b.end_document()
    b.finalize(prefix + ".idx")


def _docs(n, seed, vocab=1000):
    rng = np.random.RandomState(seed)
    return [rng.randint(0, vocab, size=rng.randint(5, 60)).tolist() for _ in range(n)]


def test_indexed_roundtrip_and_merge(tmp_path):
    a, b = _docs(20, 0), _docs(7, 1)
    pa, pb, pm = (str(tmp_path / x) for x in ("a", "b", "m"))
    _write(pa, a, np.uint16)
    _write(pb, b, np.uint16)
    ds = IndexedDataset(pa)
    assert len(ds) == 20 and ds.dtype == np.uint16
    for i, d in enumerate(a):
        assert ds[i].tolist() == d
        assert ds.get(i, 2, 3).tolist() == d[2:5]
    assert [x.tolist() for x in ds[3:6]] == a[3:6]
    m = IndexedDatasetBuilder(pm + ".bin", dtype=np.uint16)
    m.add_index(pa)
    m.add_index(pb)
    m.finalize(pm + ".idx")
    merged = IndexedDataset(pm)
    assert [merged[i].tolist() for i in range(len(merged))] == a + b
    assert merged.document_indices.tolist() == list(range(28))


def test_sample_index_matches_python_walk():
    rng = np.random.RandomState(0)
    sizes = rng.randint(3, 40, size=50).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(50) for _ in range(3)]).astype(np.int32)
    S = 16
    tokens = int(sizes.sum())
    out = build_sample_idx(sizes, doc_idx, S, 3, tokens)
    n = (3 * tokens - 1) // S
    assert out.shape == (n + 1, 2)
    stream = np.concatenate([np.full(sizes[d], d) for d in doc_idx])
    # sample s starts at global token s * S (consecutive samples overlap by one token)
    starts = np.concatenate(([0], np.cumsum(sizes[doc_idx])))
    for s in (0, 1, 5, n // 2, n):
        di, off = out[s]
        assert starts[di] + off == s * S
        assert stream[s * S] == doc_idx[di]


def test_gpt_dataset_samples_are_contiguous_token_windows(tmp_path):
    docs = _docs(40, 3)
    p = str(tmp_path / "d")
    _write(p, docs)
    ds = GPTDataset(IndexedDataset(p), np.arange(40, dtype=np.int32), num_samples=60, sequence_length=32,
                    random_seed=7, path_to_cache=str(tmp_path / "cache"))
    assert len(ds) >= 60
    flat = {tuple(d) for d in docs}
    seen = set()
    for i in range(len(ds)):
        t = ds[i]["text"]
        assert t.shape == (33,) and t.dtype == np.int64
        seen.add(tuple(t.tolist()))
    assert len(seen) == len(ds)
    # a second construction hits the cache and yields identical samples
    ds2 = GPTDataset(IndexedDataset(p), np.arange(40, dtype=np.int32), num_samples=60, sequence_length=32,
                     random_seed=7, path_to_cache=str(tmp_path / "cache"))
    assert all((ds[i]["text"] == ds2[i]["text"]).all() for i in range(0, len(ds), 7))
    assert flat


def test_blending_indices_follow_weights():
    n = 10000
    di = np.zeros(n, dtype=np.int16)
    dsi = np.zeros(n, dtype=np.int64)
    w = np.array([0.5, 0.3, 0.2])
    build_blending_indices(di, dsi, w, 3, n)
    counts = np.bincount(di, minlength=3) / n
    assert np.abs(counts - w).max() < 1e-3
    for d in range(3):
        assert (dsi[di == d] == np.arange((di == d).sum())).all()


def test_build_blend_and_splits(tmp_path):
    pa, pb = str(tmp_path / "a"), str(tmp_path / "b")
    _write(pa, _docs(200, 0))
    _write(pb, _docs(100, 1))
    train, val, test = build(sizes=[100, 20, 10], sequence_length=16, tokenizer=None, random_seed=1,
                             blend=["0.7", pa, "0.3", pb], split="90,5,5", path_to_cache=str(tmp_path / "c"))
    assert isinstance(train, BlendedDataset) and len(train) >= 100
    ids = [train[i]["dataset_id"] for i in range(100)]
    assert 0.6 < ids.count(0) / 100 < 0.8
    assert val is not None and test is not None
    single = build(sizes=[50, 0, 0], sequence_length=16, tokenizer=None, random_seed=1, blend=[pa], split="100,0,0",
                   path_to_cache=str(tmp_path / "c"))
    assert isinstance(single[0], GPTDataset) and single[1] is None


def test_batch_sampler_partitions_and_resumes():
    total, mbs, world = 1000, 4, 8
    seen = []
    for r in range(world):
        seen += [i for b in MegatronBatchSampler(total, 0, mbs, world, r) for i in b]
    assert sorted(seen) == list(range(total - total % (mbs * world)))
    resumed = [i for b in MegatronBatchSampler(total, 320, mbs, world, 2) for i in b]
    full = [i for b in MegatronBatchSampler(total, 0, mbs, world, 2) for i in b]
    assert resumed == [i for i in full if i >= 320]


def test_alpha_numeric_tokenizer():
    from lm_engine_b200.tokenizers import get_tokenizer

    t = get_tokenizer("alpha_numeric")
    ids = t.encode("aZ09", add_special_tokens=True)
    assert ids == [10, 61, 0, 9, 62]
    assert t.decode(ids, skip_special_tokens=True) == "aZ09"
    batch = t(["a", "abc"], padding=True)
    assert batch["input_ids"] == [[62, 62, 10], [10, 11, 12]] and batch["attention_mask"][0] == [0, 0, 1]
    with pytest.raises(ValueError):
        t.encode("a b")


def test_collate_left_pads_and_masks():
    from lm_engine_b200.data import collate_fn
    from lm_engine_b200.enums import LossMask

    batch = [{"input": [5, 6, 7, 8], "output": [7, 8]}, {"input": [1, 2], "output": [2]}]
    out = collate_fn(batch, True, LossMask.output_only, eos_token_id=0, use_padding_free_transformer=False)
    assert out["input_ids"].tolist() == [[5, 6, 7, 8], [0, 0, 1, 2]]
    assert out["attention_mask"].tolist() == [[1, 1, 1, 1], [0, 0, 1, 1]]
    assert out["labels"].tolist() == [[-100, -100, 7, 8], [-100, -100, -100, 2]]
    pf = collate_fn([dict(b) for b in batch], True, LossMask.output_only, 0, True)
    assert pf["cu_seqlens"].tolist() == [0, 4, 6] and pf["max_seqlen"] == 4
    assert pf["labels"].tolist() == [-100, -100, 7, 8, -100, 2]


def test_finetuning_dataloader_resumes_inside_an_epoch(tmp_path):
    """Save in the middle of an epoch, build a fresh dataloader, restore: the next batches are the ones the first
    loader goes on to produce (also across the epoch boundary, where a new permutation is drawn)."""
    import torch

    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.data import get_finetuning_dataloader
    from lm_engine_b200.models import dense_config
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.train import resumed_consumed_samples

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager()
    cfg = dense_config(vocab_size=512, hidden_size=64, num_layers=1, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=128, max_position_embeddings=32).to_dict()
    args = TrainingArgs(
        model_args={"pretrained_config": cfg}, tuning_args={"tuning_method": "full_finetuning"},
        optimizer_args={"class_args": {"lr": 1e-3}}, lr_scheduler_args={"lr_decay_style": "cosine"},
        datasets=[{"class_name": "DebugDataset", "data_name": "debug", "max_input_tokens": 4, "max_output_tokens": 4,
                   "class_args": {"num_examples": 37, "static_examples": False, "token_id": 5}}],
        save_args={"save_path": str(tmp_path), "save_interval": 100},
        training_parameters={"num_training_steps": 20, "micro_batch_size": 4, "gradient_accumulation_steps": 1,
                             "eval_during_training": False},
        load_args={"load_path": str(tmp_path)})

    class _Tok:
        eos_token_id = 1
        pad_token_id = 2

    def first_tokens(batch):
        return batch["input_ids"][:, 0].tolist()

    a = get_finetuning_dataloader(args, _Tok(), split="train")
    seen = [first_tokens(next(a)) for _ in range(5)]
    torch.save(a.state_dict(), tmp_path / "dl.pt")
    cont = [first_tokens(next(a)) for _ in range(12)]           # runs over the end of the epoch (37 examples / 4)
    b = get_finetuning_dataloader(args, _Tok(), split="train")
    b.load_state_dict(torch.load(tmp_path / "dl.pt", weights_only=False))
    resumed = [first_tokens(next(b)) for _ in range(12)]
    assert resumed == cont
    assert len({x for row in seen + cont[:4] for x in row}) == 36      # 9 batches of one epoch: no repeats
    # load_dataloader_state: false drops the checkpoint's data position for the pretraining loaders too
    assert resumed_consumed_samples(args, {"consumed_samples": 96}) == 96
    args.load_args.load_dataloader_state = False
    assert resumed_consumed_samples(args, {"consumed_samples": 96}) == 0
    ProcessGroupManager.destroy_process_groups()
