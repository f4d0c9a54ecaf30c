"""Checkpoint layout, bit-exact resume, unshard, and resharding of a 2-rank checkpoint into one process (CPU)."""

import json
import os

import numpy as np
import torch

from .dist_utils import run_distributed

VOCAB, SEQ, MBS = 512, 32, 2


def _args(save_path, load_path=None, stage=3):
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.models import dense_config

    cfg = dense_config(vocab_size=VOCAB, hidden_size=64, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=128, max_position_embeddings=SEQ).to_dict()
    d = dict(
        model_args={"pretrained_config": cfg, "efficient_initialization": True},
        tuning_args={"tuning_method": "pretraining"},
        optimizer_args={"class_args": {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10}},
        lr_scheduler_args={"num_warmup_steps": 2, "lr_decay_style": "cosine"},
        datasets=[{"class_name": "SyntheticDataset", "data_name": "syn", "class_args": {"sequence_length": SEQ}}],
        save_args={"save_path": save_path, "save_interval": 100},
        training_parameters={"num_training_steps": 20, "micro_batch_size": MBS, "gradient_accumulation_steps": 1,
                             "eval_during_training": False},
        distributed_args={"stage": stage, "gradient_checkpointing_method": "block"})
    if load_path is not None:
        d["load_args"] = {"load_path": load_path}
    return TrainingArgs(**d)


def _build(args, optimizer="TorchAdamW", optimizer_args=None, init_groups=True):
    from lm_engine_b200.distributed import wrap_model_container_for_distributed_training
    from lm_engine_b200.model_wrapper import get_model_container
    from lm_engine_b200.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    if init_groups:
        ProcessGroupManager(zero_stage=args.distributed_args.stage)
    args.training_parameters.reset_training_parameters(ProcessGroupManager.get_data_loading_world_size())
    models = get_model_container(args)
    models, _ = wrap_model_container_for_distributed_training(args, models)
    opts = get_optimizer_container(optimizer, optimizer_args or args.optimizer_args.class_args, models, None,
                                   max_grad_norm=1.0)
    ls = args.lr_scheduler_args
    scheds = get_scheduler_container(models, opts, ls.num_warmup_steps, 0, None, 20, ls.lr_decay_style,
                                     ls.lr_decay_factor, {})
    return models, opts, scheds


def _steps(models, opts, scheds, batches):
    from lm_engine_b200.train import train_step_without_pipeline_parallel

    out = []
    it = iter([{"text": b} for b in batches])
    for _ in batches:
        m = train_step_without_pipeline_parallel(models, opts, scheds, it, 1, 1.0)
        out.append((float(m["loss"]), float(m["grad_norm"])))
    return out


def _data(n, rank=0, world=1):
    g = torch.Generator().manual_seed(3)
    d = torch.randint(0, VOCAB, (n, world * MBS, SEQ + 1), generator=g)
    return [d[i, rank * MBS:(rank + 1) * MBS] for i in range(n)]


def test_layout_and_bit_exact_resume(tmp_path):
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.checkpointing import load_checkpoint_for_training, save_checkpoint

    path = str(tmp_path / "ckpt")
    args = _args(path)
    models, opts, scheds = _build(args)
    data = _data(6)
    _steps(models, opts, scheds, data[:3])
    save_checkpoint(args, models, opts, scheds, None, None, 3, {"consumed_samples": 3 * MBS})
    base = os.path.join(path, "global_step3")
    for sub in ("model/.metadata", "optimizer/.metadata", "lr_scheduler/lr_scheduler-0.pt",
                "rng_state/rng_state-0.pt", "metadata.json", "training_config.yml"):
        assert os.path.exists(os.path.join(base, sub)), sub
    assert json.load(open(os.path.join(path, "latest_checkpointed_iteration.json"))) == {
        "latest_checkpointed_iteration": 3}
    assert json.load(open(os.path.join(base, "metadata.json")))["consumed_samples"] == 3 * MBS
    cont = _steps(models, opts, scheds, data[3:])
    # fresh objects, different seed, then resume
    args2 = _args(path, load_path=path)
    args2.random_args.seed = 999
    models2, opts2, scheds2 = _build(args2)
    it, meta, _ = load_checkpoint_for_training(args2, TrainingArgs, models2, opts2, scheds2, None)
    assert it == 3 and meta["consumed_samples"] == 3 * MBS
    resumed = _steps(models2, opts2, scheds2, data[3:])
    assert resumed == cont, (resumed, cont)


def test_unshard_roundtrip(tmp_path):
    from lm_engine_b200.arguments import UnshardingArgs
    from lm_engine_b200.checkpointing import load_checkpoint_and_unshard, read_full_model_state, save_checkpoint
    from lm_engine_b200.utils import SafeTensorsWeightsManager

    path = str(tmp_path / "ckpt")
    args = _args(path)
    models, opts, scheds = _build(args)
    _steps(models, opts, scheds, _data(2))
    save_checkpoint(args, models, opts, scheds, None, None, 2, {})
    state, cfg, it = read_full_model_state(path)
    want = models[0].engine.full_state_dict()
    assert it == 2 and set(state) == {f"model.{k}" for k in want}
    for k, v in want.items():
        assert torch.equal(state[f"model.{k}"], v)
    wrapper, saved, plain = load_checkpoint_and_unshard(
        UnshardingArgs(load_args={"load_path": path}, unsharded_path=str(tmp_path / "hf")))
    wrapper.save_pretrained(str(tmp_path / "hf"), state_dict=plain)
    mgr = SafeTensorsWeightsManager(str(tmp_path / "hf"))
    for k, v in want.items():
        assert torch.equal(mgr.get_tensor(k), v)
    assert os.path.exists(tmp_path / "hf" / "config.json")


def _save_two_ranks(rank, world, path):
    from lm_engine_b200.checkpointing import save_checkpoint

    args = _args(path)
    models, opts, scheds = _build(args)
    _steps(models, opts, scheds, _data(2, rank, world))
    save_checkpoint(args, models, opts, scheds, None, None, 2, {})
    return {k: v.numpy().copy() for k, v in models[0].engine.full_state_dict().items()}


def test_two_rank_checkpoint_reshards_to_one(tmp_path):
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.checkpointing import load_checkpoint_for_training, read_full_model_state
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    path = str(tmp_path / "ckpt")
    outs = run_distributed(_save_two_ranks, 2, path)
    state, _, _ = read_full_model_state(path)
    for k, v in outs[0].items():
        assert np.array_equal(state[f"model.{k}"].numpy(), v), k
    ProcessGroupManager.destroy_process_groups()
    args = _args(path, load_path=path)
    models, opts, scheds = _build(args)
    load_checkpoint_for_training(args, TrainingArgs, models, opts, scheds, None)
    got = models[0].engine.full_state_dict()
    for k, v in outs[0].items():
        assert np.array_equal(got[k].numpy(), v), k
    assert models[0].engine.step_count == 2


def _resume_with_torch_optimizer(rank, world, path, optimizer, optimizer_args):
    """3 steps, save, 3 more steps; then fresh objects, load, the same 3 steps: identical losses and norms."""
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.checkpointing import load_checkpoint_for_training, save_checkpoint

    args = _args(path)
    models, opts, scheds = _build(args, optimizer, optimizer_args)
    assert not opts[0].fused
    data = _data(6, rank, world)
    _steps(models, opts, scheds, data[:3])
    save_checkpoint(args, models, opts, scheds, None, None, 3, {})
    cont = _steps(models, opts, scheds, data[3:])
    args2 = _args(path, load_path=path)
    args2.random_args.seed = 999
    models2, opts2, scheds2 = _build(args2, optimizer, optimizer_args, init_groups=False)
    load_checkpoint_for_training(args2, TrainingArgs, models2, opts2, scheds2, None)
    resumed = _steps(models2, opts2, scheds2, data[3:])
    return cont, resumed


def test_resume_keeps_momentum_of_sgd_on_two_ranks(tmp_path):
    """The optimizers other than the fused AdamW keep their state inside a wrapped torch optimizer; a checkpoint
    must carry it (SGD's momentum buffer here), otherwise the first steps after a resume differ."""
    outs = run_distributed(_resume_with_torch_optimizer, 2, str(tmp_path / "ckpt"), "TorchSGD",
                           {"lr": 1e-2, "momentum": 0.9, "weight_decay": 0.0})
    for cont, resumed in outs:
        assert resumed == cont, (resumed, cont)


def test_resume_keeps_amsgrad_state(tmp_path):
    cont, resumed = _resume_with_torch_optimizer(0, 1, str(tmp_path / "ckpt"), "TorchAdamW",
                                                 {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                  "eps": 1e-10, "amsgrad": True})
    assert resumed == cont, (resumed, cont)
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()


def _tp2_dp2(rank, world, path, phase):
    """Tensor parallel 2 x ZeRO-3 over 2.  ``save``: two steps, checkpoint, return the local state and what each rank
    offers to the checkpoint writer.  ``load``: fresh model of the same topology, load, return the local state."""
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.checkpointing import load_checkpoint_for_training, model_state_dict, save_checkpoint
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    args = _args(path, load_path=path if phase == "load" else None)
    args.distributed_args.tensor_parallel_world_size = 2
    ProcessGroupManager(zero_stage=3, tensor_parallel_world_size=2)
    models, opts, scheds = _build(args, init_groups=False)
    dp_rank, dp_world = ProcessGroupManager.get_data_parallel_rank(), ProcessGroupManager.get_data_parallel_world_size()
    if phase == "save":
        _steps(models, opts, scheds, _data(2, dp_rank, dp_world))
        save_checkpoint(args, models, opts, scheds, None, None, 2, {})
        offered = {k: (tuple(v.to_local().shape), tuple(v.shape), v.device_mesh.mesh_dim_names)
                   for k, v in model_state_dict(models).items() if hasattr(v, "to_local")}
    else:
        from lm_engine_b200.parallel.fsdp import FSDPEngine

        calls, gathers = [], []
        inner, inner_full = FSDPEngine.load_row_chunks, FSDPEngine.load_full_state_dict
        FSDPEngine.load_row_chunks = lambda self, u, chunks, which="master": (calls.append(u.name),
                                                                               inner(self, u, chunks, which))[1]
        FSDPEngine.load_full_state_dict = lambda self, sd, which="master": (gathers.append(len(sd)),
                                                                             inner_full(self, sd, which))[1]
        try:
            load_checkpoint_for_training(args, TrainingArgs, models, opts, scheds, None)
        finally:
            FSDPEngine.load_row_chunks, FSDPEngine.load_full_state_dict = inner, inner_full
        offered = {"row_block_loads": len(calls), "gather_loads": len(gathers)}
    eng = models[0].engine
    local = {k: v.numpy().copy() for k, v in eng.full_state_dict().items()}
    moments = {k: v.numpy().copy() for k, v in eng.full_state_dict("exp_avg").items()}
    return local, moments, offered, ProcessGroupManager.get_tensor_parallel_rank(), eng.step_count


def test_tensor_parallel_times_sharded_checkpoint_is_two_dimensional(tmp_path):
    """Under TP 2 x ZeRO-3 over 2 every rank offers only its block of rows of its tensor-parallel slice (a DTensor on
    the (tp, fsdp) mesh), the checkpoint holds the global tensors, and it loads back bit-exactly."""
    from lm_engine_b200.checkpointing import read_full_model_state

    path = str(tmp_path / "ckpt")
    saved = run_distributed(_tp2_dp2, 4, path, "save", timeout=600)
    state, _, _ = read_full_model_state(path)
    for local, _, offered, tp_rank, _ in saved:
        assert offered and all(names == ("tp", "fsdp") for _, _, names in offered.values())
        for key, (local_shape, global_shape, _) in offered.items():
            # a rank's piece is at most half (rounded up) of the rows of its tensor-parallel slice
            name = key[len("model."):]
            tp_local_rows = local[name].shape[0]
            assert local_shape[0] <= -(-tp_local_rows // 2), (key, local_shape, tp_local_rows)
            assert tuple(state[key].shape) == global_shape
        for name, v in local.items():                      # the global tensor contains this rank's slice
            g = state[f"model.{name}"].numpy()
            if g.shape == v.shape:
                assert np.array_equal(g, v), name
            else:
                dim = [i for i, (a, b) in enumerate(zip(g.shape, v.shape)) if a != b][0]
                n = v.shape[dim]
                assert np.array_equal(np.take(g, range(tp_rank * n, (tp_rank + 1) * n), axis=dim), v), name
    loaded = run_distributed(_tp2_dp2, 4, path, "load", timeout=600)
    for (a, ma, _, _, _), (b, mb, info, _, step) in zip(saved, loaded):
        assert step == 2
        # weights and both moments of every unit came in as row blocks and were re-cut without a gather
        assert info["row_block_loads"] > 0 and info["gather_loads"] == 0, info
        for k in a:
            assert np.array_equal(a[k], b[k]), k
            assert np.array_equal(ma[k], mb[k]), k


def _row_block_round_trip(rank, world):
    """``row_chunks`` followed by ``load_row_chunks`` is the identity on every unit's state, on a group size that
    divides neither the rows nor the flat sizes (empty and partial blocks occur)."""
    args = _args("/nonexistent")
    models, opts, scheds = _build(args)
    _steps(models, opts, scheds, _data(1, rank, world))
    eng = models[0].engine
    ok = True
    for which in ("master", "exp_avg"):
        for u in eng.all_units:
            if not eng.can_exchange_row_chunks(u) or any(len(s.shape) == 0 for s in u.slots):
                continue
            state = {"master": u.master, "exp_avg": u.exp_avg}[which]
            before = state.clone()
            chunks = eng.row_chunks(u, which)
            for s in u.slots:                                   # the block sizes of an even split of the rows
                per = -(-s.shape[0] // world)
                rows = max(min((rank + 1) * per, s.shape[0]) - min(rank * per, s.shape[0]), 0)
                ok &= chunks[s.name].shape[0] == rows
            state.zero_()
            eng.load_row_chunks(u, chunks, which)
            ok &= bool(torch.equal(state, before))
    return ok


def test_row_block_exchange_round_trip_on_three_ranks():
    assert all(run_distributed(_row_block_round_trip, 3, timeout=600))
