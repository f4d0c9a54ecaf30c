"""ZeRO stages 0-3 (and HSDP) of the flat-buffer engine on gloo ranks against a single-process run on the
concatenated batch."""

import numpy as np
import pytest
import torch

from .dist_utils import run_distributed

VOCAB, SEQ = 512, 32


def _cfg():
    from lm_engine_b200.models import dense_config

    return dense_config(vocab_size=VOCAB, hidden_size=64, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        intermediate_size=128, max_position_embeddings=SEQ)


def _train(rank, world, stage, ddp, fsdp, steps, mbs):
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.enums import GradientCheckpointingMethod
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager(zero_stage=stage, data_parallel_replication_world_size=ddp,
                        data_parallel_sharding_world_size=fsdp)
    w = ModelWrapperForPretraining(pretrained_config=_cfg().to_dict(), micro_batch_size=mbs, sequence_length=SEQ,
                                   efficient_initialization=True)
    eng = shard_model(w, stage=stage, dtype=torch.float32, communication_dtype=None,
                      gradient_checkpointing_method=GradientCheckpointingMethod.block, seed=11)
    opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10},
                           None, False, 1.0)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, VOCAB, (steps, world * mbs, SEQ + 1), generator=g)
    losses, norms = [], []
    for s in range(steps):
        opt.zero_grad()
        out = w(data[s, rank * mbs:(rank + 1) * mbs], lm_loss_multiplier=1 / (mbs * SEQ))
        out["loss"].backward()
        norms.append(float(opt.step()))
        losses.append(float(out["loss"].detach()))
    params = eng.full_state_dict()
    return losses, norms, {k: v.detach().cpu().numpy().copy() for k, v in params.items()}


def _single(steps, total_mbs):
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()
    return _train(0, 1, 3, None, None, steps, total_mbs)


@pytest.mark.parametrize("stage,ddp,fsdp", [(3, None, None), (2, None, None), (0, None, None), (3, 2, 1), (3, 1, 2)])
def test_two_ranks_match_single_process(stage, ddp, fsdp):
    steps, mbs, world = 3, 2, 2
    ref_losses, ref_norms, ref_params = _single(steps, mbs * world)
    outs = run_distributed(_train, world, stage, ddp, fsdp, steps, mbs)
    mean_loss = [sum(o[0][s] for o in outs) / world for s in range(steps)]
    for a, b in zip(mean_loss, ref_losses):
        assert abs(a - b) < 2e-4, (mean_loss, ref_losses)
    for a, b in zip(outs[0][1], ref_norms):
        assert abs(a - b) / b < 2e-3, (outs[0][1], ref_norms)
    for k, v in ref_params.items():
        for o in outs:
            assert np.allclose(o[2][k], v, atol=2e-5, rtol=1e-4), k


def test_four_ranks_hsdp():
    steps, mbs, world = 2, 1, 4
    ref_losses, ref_norms, ref_params = _single(steps, mbs * world)
    outs = run_distributed(_train, world, 3, 2, 2, steps, mbs)
    for k, v in ref_params.items():
        assert np.allclose(outs[3][2][k], v, atol=2e-5, rtol=1e-4), k
    assert abs(outs[0][1][0] - ref_norms[0]) / ref_norms[0] < 2e-3


def _train_fused_ce(rank, world, tied):
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.kernels import enable_kernels
    from lm_engine_b200.enums import Kernel
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager(zero_stage=3)
    cfg = _cfg().to_dict()
    cfg["tie_word_embeddings"] = tied
    w = ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=2, sequence_length=SEQ,
                                   efficient_initialization=True)
    eng = shard_model(w, stage=3, dtype=torch.float32, communication_dtype=None, seed=11)
    opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10},
                           None, False, 1.0)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, VOCAB, (world * 2, SEQ + 1), generator=g)[rank * 2:(rank + 1) * 2]
    res = []
    for fused in (False, True):
        opt.zero_grad()
        kernels = [Kernel.fused_linear_cross_entropy] if fused else []
        with enable_kernels(kernels):
            out = w(data, lm_loss_multiplier=1 / (2 * SEQ))
            out["loss"].backward()
        eng.finish_backward()
        grads = eng.full_state_dict("grad")
        res.append((float(out["loss"].detach()), {k: v.numpy().copy() for k, v in grads.items()}))
    return res


@pytest.mark.parametrize("tied", [False, True])
def test_fused_linear_cross_entropy_under_zero3(tied):
    outs = run_distributed(_train_fused_ce, 2, tied)
    for (l0, g0), (l1, g1) in outs:
        assert abs(l0 - l1) < 1e-5
        for k in g0:
            assert np.allclose(g0[k], g1[k], atol=1e-6, rtol=1e-4), k


def _in_backward_run(rank, world, in_backward):
    import torch

    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.models import dense_config
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager(zero_stage=3)
    cfg = dense_config(vocab_size=128, hidden_size=32, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=64, max_position_embeddings=16).to_dict()
    w = ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=2, sequence_length=16,
                                   efficient_initialization=True)
    eng = shard_model(w, stage=3, dtype=torch.float32, communication_dtype=None, seed=1)
    opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-2, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-8},
                           None, False, None, step_in_backward=in_backward)
    data = torch.randint(0, 128, (4, 2 * world, 17), generator=torch.Generator().manual_seed(3))
    losses = []
    for s in range(4):
        opt.zero_grad()
        out = w(data[s, 2 * rank:2 * rank + 2], lm_loss_multiplier=1 / 32)
        out["loss"].backward()
        opt.step()
        losses.append(float(out["loss"].detach()))
    return losses, {k: v.cpu().numpy().copy() for k, v in eng.full_state_dict().items()}


@pytest.mark.parametrize("world", [1, 2])
def test_optimizer_in_backward_equals_step_after_backward(world):
    """Without clipping, stepping every unit right behind its gradient reduction (the reference's
    `use_optimizer_with_backward_hook`) gives the weights of the ordinary step after the whole backward pass."""
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    runs = []
    for mode in (False, True):
        if world == 1:
            ProcessGroupManager.destroy_process_groups()
            runs.append([_in_backward_run(0, 1, mode)])
            ProcessGroupManager.destroy_process_groups()
        else:
            runs.append(run_distributed(_in_backward_run, world, mode))
    for (la, pa), (lb, pb) in zip(*runs):
        assert la == lb
        for k in pa:
            assert np.array_equal(pa[k], pb[k]), k
