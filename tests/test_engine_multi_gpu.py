"""ZeRO-3 on 2 GPUs (copy-engine parameter all-gather over symmetric memory; gradient reduce-scatter by the fused
peer-load kernel, its in-switch variant, copy engines, or NCCL) against the same global batch on 1 GPU: per-step mean
loss and global gradient norm."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _moe_config():
    from lm_engine_b200.models import dense_config

    cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=1024, head_dim=64, max_position_embeddings=256).to_dict()
    cfg["mlp_blocks"] = [{"mlp_type": "MoE", "intermediate_size": 256, "num_experts": 4, "num_experts_per_tok": 2,
                          "activation_function": "swiglu", "shared_intermediate_size": None, "add_bias": False}
                         for _ in range(3)]
    cfg["router_aux_loss_coef"] = 0.01
    return cfg


def _hybrid_config():
    from lm_engine_b200.models import dense_config

    cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=1024, head_dim=64, max_position_embeddings=256).to_dict()
    cfg["position_embedding_type"] = "nope"
    cfg["sequence_mixer_blocks"] = [
        dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=512, num_heads=8, conv_kernel_size=4,
             activation_function="silu", num_groups=1, chunk_size=32, normalization_function="rmsnorm"),
        dict(sequence_mixer_type="m2rnn", k_head_dim=16, v_head_dim=16, num_q_heads=1, num_k_heads=1, num_v_heads=8,
             num_f_heads=8, num_g_heads=8, num_weight_heads=8, use_residual=True, kernel_size=4,
             activation_function="silu", add_bias=False, gradient_clipping=1.0, normalization_function="rmsnorm"),
        dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, head_dim=64)]
    return cfg


def _worker(rank, world, port, q, reduce_mode, total_mbs, steps, ep=1, weights_dir=None, cp=1, ep_exchange="peer"):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", LME_REDUCE_SCATTER=reduce_mode,
                      LME_EP_EXCHANGE=ep_exchange)
    try:
        import torch.distributed as dist

        from lm_engine_b200.distributed import shard_model
        from lm_engine_b200.enums import GradientCheckpointingMethod
        from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
        from lm_engine_b200.models import dense_config
        from lm_engine_b200.ops import _lib
        from lm_engine_b200.optimization.optimizer import ShardedOptimizer
        from lm_engine_b200.parallel.manager import ProcessGroupManager

        ProcessGroupManager(zero_stage=3, expert_parallel_world_size=ep if world > 1 else 1,
                            context_parallel_world_size=cp if world > 1 else 1)
        shards = cp if world > 1 else 1                  # context-parallel ranks share the batch and split the tokens
        mbs = total_mbs // (world // shards)
        cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=3, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=1024, head_dim=64,
                           max_position_embeddings=256).to_dict()
        if weights_dir is not None:     # the same saved weights on every topology (experts are sliced on load)
            w = ModelWrapperForPretraining(model_name=weights_dir, micro_batch_size=mbs, sequence_length=256,
                                           dtype="bf16")
        else:
            w = ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=mbs, sequence_length=256,
                                           efficient_initialization=True, dtype="bf16")
        eng = shard_model(w, stage=3, dtype=torch.bfloat16, communication_dtype=None,
                          gradient_checkpointing_method=GradientCheckpointingMethod.block, seed=5)
        opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                   "eps": 1e-10}, None, False, 1.0)
        g = torch.Generator().manual_seed(11)
        data = torch.randint(0, 2048, (steps, total_mbs, 257), generator=g)
        losses, norms = [], []
        for s in range(steps):
            opt.zero_grad()
            dl_rank = rank // shards
            out = w(data[s, dl_rank * mbs:(dl_rank + 1) * mbs].cuda(), lm_loss_multiplier=1 / (mbs * 256 / shards))
            out["loss"].backward()
            norms.append(float(opt.step()))
            losses.append(float(out["loss"]))
        torch.cuda.synchronize()
        info = {"ce_gather": eng.copy_engine_gather, "ce_reduce": eng.copy_engine_reduce,
                "reduce_mode": eng.reduce_mode,
                "multicast": any(getattr(eng, "_symm_grad_mc", {}).values())}
        q.put((rank, "ok", (losses, norms, _lib.read_status(), info)))
        if world > 1:
            dist.barrier()
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


def _run(world, reduce_mode, total_mbs=4, steps=4, ep=1, weights_dir=None, cp=1, ep_exchange="peer"):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, reduce_mode, total_mbs, steps, ep, weights_dir, cp,
                                                 ep_exchange))
             for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", payload
            res[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return [res[r] for r in range(world)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("reduce_mode", ["fused", "nvls", "nccl", "ce"])
def test_zero3_two_gpus_match_one_gpu(reduce_mode):
    (ref_losses, ref_norms, ref_status, _), = _run(1, "nccl")
    outs = _run(2, reduce_mode)
    for losses, norms, status, info in outs:
        assert status[0] == 0, status
        assert info["ce_gather"] and info["ce_reduce"] == (reduce_mode == "ce")
        assert info["reduce_mode"] == reduce_mode
        if reduce_mode == "nvls" and not info["multicast"]:
            pytest.skip("no multicast mapping on this machine: the kernel ran on plain peer loads")
    mean = [(outs[0][0][s] + outs[1][0][s]) / 2 for s in range(len(ref_losses))]
    for a, b in zip(mean, ref_losses):
        assert abs(a - b) < 1.5e-2 * abs(b), (mean, ref_losses)
    for o in outs:
        for a, b in zip(o[1], ref_norms):
            assert abs(a - b) < 3e-2 * abs(b), (o[1], ref_norms)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_expert_parallel_two_gpus_match_one_gpu(tmp_path, exchange):
    """Mixture of experts with the experts split over 2 GPUs (token rows exchanged by the peer-memory kernels or by
    NCCL all-to-all, grouped GEMM kernels, expert parameter units reduced over their replica group) against all
    experts on one GPU."""
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.utils import SafeTensorsWeightsManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=3)
    torch.manual_seed(5)
    cfg = config_from_dict(_moe_config())
    model = build_model(cfg)
    d = str(tmp_path / "weights")
    cfg.save_pretrained(d)
    SafeTensorsWeightsManager.save_state_dict(model.state_dict(), d)
    ProcessGroupManager.destroy_process_groups()
    (ref_losses, ref_norms, _, _), = _run(1, "nccl", ep=2, weights_dir=d)
    outs = _run(2, "nccl", ep=2, weights_dir=d, ep_exchange=exchange)
    mean = [(outs[0][0][s] + outs[1][0][s]) / 2 for s in range(len(ref_losses))]
    for a, b in zip(mean, ref_losses):
        assert abs(a - b) < 1.5e-2 * abs(b), (mean, ref_losses)
    for losses, norms, status, _ in outs:
        assert status[0] == 0, status
        for a, b in zip(norms, ref_norms):
            assert abs(a - b) < 4e-2 * abs(b), (norms, ref_norms)


def _save_weights(config: dict, path) -> str:
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.utils import SafeTensorsWeightsManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=3)
    torch.manual_seed(5)
    cfg = config_from_dict(config)
    model = build_model(cfg)
    cfg.save_pretrained(str(path))
    SafeTensorsWeightsManager.save_state_dict(model.state_dict(), str(path))
    ProcessGroupManager.destroy_process_groups()
    return str(path)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_hybrid_two_gpus_match_one_gpu(tmp_path):
    """Mamba-2, M2RNN and attention layers with the sequence split over 2 GPUs: the SSD prefix over ranks, the
    scan kernels' carried state and its gradient through the sequence pipeline, the convolution halo, and the
    head-exchange attention, against the whole sequence on one GPU."""
    d = _save_weights(_hybrid_config(), tmp_path / "weights")
    (ref_losses, ref_norms, _, _), = _run(1, "nccl", weights_dir=d, cp=2)
    outs = _run(2, "nccl", weights_dir=d, cp=2)
    mean = [(outs[0][0][s] + outs[1][0][s]) / 2 for s in range(len(ref_losses))]
    for a, b in zip(mean, ref_losses):
        assert abs(a - b) < 1.5e-2 * abs(b), (mean, ref_losses)
    for losses, norms, status, _ in outs:
        assert status[0] == 0, status
        for a, b in zip(norms, ref_norms):
            assert abs(a - b) < 4e-2 * abs(b), (norms, ref_norms)


def _cp_attention_worker(rank, world, port, q, method, algo):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        import torch.distributed as dist

        from lm_engine_b200.ops import attention
        from lm_engine_b200.parallel.context_parallel import shard_indices
        from lm_engine_b200.parallel.manager import ProcessGroupManager
        from lm_engine_b200.parallel.ring_attention import ring_attention
        from lm_engine_b200.parallel.ulysses import ulysses_attention

        ProcessGroupManager(context_parallel_world_size=world, context_parallel_load_balancing_method=method)
        g = torch.Generator().manual_seed(3)
        B, S, Hq, Hkv, D = 2, 512, 8, 2, 128
        q_, k_, v_, do = (torch.randn(B, S, h, D, generator=g).to(torch.bfloat16).cuda() for h in (Hq, Hkv, Hkv, Hq))
        full = [t.clone().requires_grad_() for t in (q_, k_, v_)]
        ref = attention(*full, causal=True)
        ref.backward(do)
        idx = shard_indices(S, world, rank, method, device="cuda")
        loc = [t[:, idx].clone().requires_grad_() for t in (q_, k_, v_)]
        if algo == "gathered":
            from lm_engine_b200.parallel.gathered_attention import eligible, gathered_kv_attention

            assert eligible(loc[0], loc[1], True, None, method)
            out = gathered_kv_attention(*loc)
            out.backward(do[:, idx])
            loc = [t.detach().clone().requires_grad_() for t in loc]      # a second call: slots and sequence numbers
            out = gathered_kv_attention(*loc)
        else:
            out = (ulysses_attention if algo == "ulysses" else ring_attention)(*loc, causal=True)
        out.backward(do[:, idx])
        torch.cuda.synchronize()
        def rel(a, b):
            return float((a.detach().float() - b.detach().float()).norm() / (b.detach().float().norm() + 1e-6))

        from lm_engine_b200.ops import _lib

        err = [rel(out, ref[:, idx])] + [rel(a.grad, b.grad[:, idx]) for a, b in zip(loc, full)]
        err.append(float(_lib.read_status()[0]))
        q.put((rank, "ok", err))
        dist.barrier()
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("method", [None, "headtail"])
@pytest.mark.parametrize("algo", ["ulysses", "ring", "gathered"])
def test_context_parallel_attention_two_gpus(method, algo):
    """Head-exchange, ring attention (on the tcgen05 block kernels: 512 tokens split 2 ways gives runs of 256 / 128
    rows) and the gathered form (K / V chunks arrive by copy engines while ONE attention launch per query run waits
    for their readiness words; dK / dV summed by the peer-load reduce-scatter kernel) against single-GPU attention,
    outputs and gradients."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_cp_attention_worker, args=(r, 2, port, q, method, algo)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", payload
            assert payload[-1] == 0, payload        # no bounded wait expired
            assert max(payload[:-1]) < 2e-2, payload     # relative error of the output and of dq, dk, dv
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()


def _pp_worker(rank, world, port, q, stages, schedule, M):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        import torch.distributed as dist

        from lm_engine_b200.containers import ModelContainer
        from lm_engine_b200.distributed import shard_model
        from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
        from lm_engine_b200.models import dense_config
        from lm_engine_b200.ops import _lib
        from lm_engine_b200.optimization.optimizer import ShardedOptimizer
        from lm_engine_b200.parallel.manager import ProcessGroupManager
        from lm_engine_b200.parallel.pipeline_parallel import PipelineSchedule

        mbs, seq, steps = 2, 256, 3
        ProcessGroupManager(zero_stage=3, pipeline_parallel_world_size=world)
        cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=1024, head_dim=64,
                           max_position_embeddings=seq).to_dict()
        if world > 1:
            ids = ProcessGroupManager.topology().pipeline_stage_ids(ProcessGroupManager.get_pipeline_parallel_rank(),
                                                                    stages)
            ws = [ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=mbs, sequence_length=seq,
                                             efficient_initialization=True, dtype="bf16",
                                             num_pipeline_stages=stages, pipeline_stage_id=i) for i in ids]
        else:
            ws = [ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=mbs, sequence_length=seq,
                                             efficient_initialization=True, dtype="bf16")]
        mc = ModelContainer(ws)
        opts = []
        for w in ws:
            e = shard_model(w, stage=3, dtype=torch.bfloat16, communication_dtype=None, seed=3)
            opts.append(ShardedOptimizer(e, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                           "eps": 1e-10}, None, False, 1.0))
        data = torch.randint(0, 2048, (steps, M * mbs, seq + 1), generator=torch.Generator().manual_seed(9)).cuda()
        losses, norms = [], []
        sched = PipelineSchedule(mc, schedule, stages, M, mbs, seq, torch.bfloat16, False) if world > 1 else None
        for s in range(steps):
            for o in opts:
                o.zero_grad()
            if sched is not None:
                totals = sched.step(data[s])
                total = sum(w.engine.local_sumsq().clone() for w in ws)
                dist.all_reduce(total, group=ProcessGroupManager.get_pipeline_parallel_group())
                for o in opts:
                    n = o.step(total_sumsq=total)
                losses.append(float(totals["loss"]) if totals is not None else None)
            else:
                acc = 0.0
                for mb in data[s].chunk(M):
                    out = ws[0](mb, lm_loss_multiplier=1 / (mbs * seq))
                    (out["loss"] / M).backward()
                    acc += float(out["loss"].detach()) / M
                n = opts[0].step()
                losses.append(acc)
            norms.append(float(n))
        torch.cuda.synchronize()
        q.put((rank, "ok", (losses, norms, _lib.read_status())))
        if world > 1:
            dist.barrier()
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


def _spawn(world, target, *args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=target, args=(r, world, port, q, *args)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", payload
            res[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return [res[r] for r in range(world)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("stages,schedule,M", [(2, "1F1B", 4), (4, "Interleaved1F1B", 4)])
def test_pipeline_parallel_two_gpus_match_one_gpu(stages, schedule, M):
    """Two pipeline ranks over NCCL (batched isend / irecv per tick) in bf16 against the same micro-batches on one
    GPU: loss of the last stage and the global gradient norm per step."""
    (ref_losses, ref_norms, _), = _spawn(1, _pp_worker, 1, None, M)
    outs = _spawn(2, _pp_worker, stages, schedule, M)
    last = outs[(stages - 1) % 2]
    for a, b in zip(last[0], ref_losses):
        assert abs(a - b) < 1.5e-2 * abs(b), (last[0], ref_losses)
    for losses, norms, status in outs:
        assert status[0] == 0, status
        for a, b in zip(norms, ref_norms):
            assert abs(a - b) < 3e-2 * abs(b), (norms, ref_norms)
