"""The tiny dense configuration trained for 20 AdamW steps on CPU in fp32, step by step against the unmodified
reference package: vocab 2048, 4 layers, hidden 256, 4 query / 2 key-value heads of 64, RoPE 10000, RMSNorm 1e-5,
SwiGLU 1024, untied embeddings, weights from seed 0; micro batch 4 x 512 uniform-random tokens from seed 1234;
AdamW lr 3e-4, betas 0.9 / 0.95, weight decay 0.1, clipping at 1.0, cosine schedule with 5 warm-up steps.

Checked: the loss and the gradient norm of every step; a checkpoint written at step 10 by this repository resumes
into the same tail; a DCP payload written at step 10 by the reference's own saver classes loads into this
repository's engine and continues like the reference does.
"""

import os

import pytest
import torch
import torch.distributed.checkpoint as dcp
import torch.nn as nn

from .refutil import build_reference_model, reference

VOCAB, SEQ, MBS, STEPS = 2048, 512, 4, 20
OPT = {"lr": 3e-4, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-8}


def _model_config():
    from lm_engine_b200.models import dense_config

    return dense_config(vocab_size=VOCAB, hidden_size=256, num_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, intermediate_size=1024, head_dim=64, max_position_embeddings=SEQ,
                        rope_theta=10000).to_dict()


def _data():
    g = torch.Generator().manual_seed(1234)
    return torch.randint(0, VOCAB, (STEPS, MBS, SEQ + 1), generator=g)


class _RefWrapper(nn.Module):
    """What the reference's optimizer / checkpoint helpers expect of a model wrapper: `.model`, no teacher."""

    def __init__(self, model):
        super().__init__()
        self.model = model

    def has_teacher_model(self):
        return False


def _reference_run(tmp_path, data, save_at):
    reference()
    from lm_engine.checkpointing.model import _ModelSaver
    from lm_engine.checkpointing.optimizer import _OptimizerSaver
    from lm_engine.optimization.lr_scheduler.cosine import CosineScheduler
    from lm_engine.optimization.params_group import get_normal_group_with_names

    torch.manual_seed(0)
    ref = build_reference_model(_model_config())
    init = {k: v.clone() for k, v in ref.state_dict().items()}
    wrap = _RefWrapper(ref)
    groups = get_normal_group_with_names(wrap, {}).to_torch_compatible_params_groups()
    opt = torch.optim.AdamW(groups, lr=OPT["lr"], betas=tuple(OPT["betas"]), eps=OPT["eps"],
                            weight_decay=OPT["weight_decay"])
    sched = CosineScheduler(opt, num_warmup_steps=5, num_constant_steps=0, num_decay_steps=None,
                            num_training_steps=STEPS, lr_decay_factor=0.1)
    trace = []
    for step in range(STEPS):
        if step == save_at:
            dcp.save({"state": _ModelSaver([wrap])}, checkpoint_id=str(tmp_path / "ref_ckpt" / "model"))
            dcp.save({"state": _OptimizerSaver([wrap], [opt])}, checkpoint_id=str(tmp_path / "ref_ckpt" / "optimizer"))
        x, y = data[step, :, :-1], data[step, :, 1:]
        logits = ref(input_ids=x).logits
        loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, VOCAB), y.reshape(-1),
                                                 reduction="sum") / (MBS * SEQ)
        loss.backward()
        norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        sched.step()
        opt.zero_grad()
        trace.append((float(loss), float(norm)))
    return init, trace


def _args(path, load_path=None):
    from lm_engine_b200.arguments import TrainingArgs

    d = dict(
        model_args={"pretrained_config": _model_config(), "efficient_initialization": True},
        tuning_args={"tuning_method": "pretraining"},
        optimizer_args={"class_name": "TorchAdamW", "class_args": dict(OPT)},
        lr_scheduler_args={"num_warmup_steps": 5, "lr_decay_style": "cosine"},
        datasets=[{"class_name": "SyntheticDataset", "data_name": "syn", "class_args": {"sequence_length": SEQ}}],
        save_args={"save_path": path, "save_interval": 100},
        training_parameters={"num_training_steps": STEPS, "micro_batch_size": MBS, "gradient_accumulation_steps": 1,
                             "eval_during_training": False, "gradient_clipping": 1.0},
        mixed_precision_args={"dtype": "fp32"},
        distributed_args={"stage": 3, "gradient_checkpointing_method": "block"})
    if load_path is not None:
        d["load_args"] = {"load_path": load_path}
    return TrainingArgs(**d)


def _build(args):
    from lm_engine_b200.distributed import wrap_model_container_for_distributed_training
    from lm_engine_b200.model_wrapper import get_model_container
    from lm_engine_b200.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=args.distributed_args.stage)
    args.training_parameters.reset_training_parameters(ProcessGroupManager.get_data_loading_world_size())
    models = get_model_container(args)
    models, _ = wrap_model_container_for_distributed_training(args, models)
    opts = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, models, None, max_grad_norm=1.0)
    ls = args.lr_scheduler_args
    scheds = get_scheduler_container(models, opts, ls.num_warmup_steps, 0, None, STEPS, ls.lr_decay_style,
                                     ls.lr_decay_factor, {})
    return models, opts, scheds


def _steps(models, opts, scheds, batches):
    from lm_engine_b200.train import train_step_without_pipeline_parallel

    it = iter([{"text": b} for b in batches])
    out = []
    for _ in range(len(batches)):
        m = train_step_without_pipeline_parallel(models, opts, scheds, it, 1, 1.0)
        out.append((float(m["loss"]), float(m["grad_norm"])))
    return out


def _close(a, b, tol):
    return all(abs(x - y) <= tol * max(abs(y), 1e-6) for p, q in zip(a, b) for x, y in zip(p, q))


def test_twenty_steps_resume_and_cross_load(tmp_path):
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.checkpointing import (load_checkpoint_for_training, load_model_state_dict,
                                              load_optimizer_state_dict, model_state_dict, optimizer_state_dict,
                                              save_checkpoint, _saved_optimizer_state_names)
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    data = _data()
    init, ref_trace = _reference_run(tmp_path, data, save_at=10)
    assert abs(ref_trace[0][0] - 7.676) < 0.05                # ~ ln(2048) at initialisation

    # ---- this repository, same initial weights, through the engine and the public step function
    path = str(tmp_path / "ckpt")
    args = _args(path)
    models, opts, scheds = _build(args)
    models[0].engine.load_full_state_dict(init)
    ours = _steps(models, opts, scheds, list(data[:10]))
    save_checkpoint(args, models, opts, scheds, None, None, 10, {"consumed_samples": 10 * MBS})
    ours += _steps(models, opts, scheds, list(data[10:]))
    assert _close(ours, ref_trace, 5e-4), list(zip(ours, ref_trace))

    # ---- resume from the checkpoint written at step 10: the tail repeats exactly
    args2 = _args(path, load_path=path)
    models2, opts2, scheds2 = _build(args2)
    it, meta, _ = load_checkpoint_for_training(args2, TrainingArgs, models2, opts2, scheds2, None)
    assert it == 10 and meta["consumed_samples"] == 10 * MBS
    assert _steps(models2, opts2, scheds2, list(data[10:])) == ours[10:]

    # ---- the payload written at step 10 by the reference's own saver classes loads into this engine
    models3, opts3, scheds3 = _build(_args(str(tmp_path / "unused")))
    ref_ckpt = str(tmp_path / "ref_ckpt")
    wrapped = {"state": model_state_dict(models3)}
    dcp.load(wrapped, checkpoint_id=os.path.join(ref_ckpt, "model"))
    load_model_state_dict(models3, wrapped["state"])
    wrapped = {"state": optimizer_state_dict(models3, opts3,
                                             _saved_optimizer_state_names(os.path.join(ref_ckpt, "optimizer")))}
    dcp.load(wrapped, checkpoint_id=os.path.join(ref_ckpt, "optimizer"))
    load_optimizer_state_dict(models3, opts3, wrapped["state"])
    assert models3[0].engine.step_count == 10
    for _ in range(10):
        scheds3.step()
    cross = _steps(models3, opts3, scheds3, list(data[10:]))
    assert _close(cross, ref_trace[10:], 5e-4), list(zip(cross, ref_trace[10:]))
    ProcessGroupManager.destroy_process_groups()
