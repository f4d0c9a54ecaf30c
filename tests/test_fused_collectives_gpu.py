"""Fused all-gather -> GEMM over NVLink peer memory on 2 GPUs (child processes, NVLS off): results against a plain
all-gather followed by an fp32 matmul, over several calls so that both staging slots and the flag protocol cycle."""

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


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lm_engine_b200.ops import _lib
        from lm_engine_b200.parallel.symm import all_gather_matmul

        errs = []
        for (t, K, N), calls in (((512, 1024, 768), 5), ((4096, 4096, 6144), 3), ((384, 256, 264), 2)):
            w = (torch.randn(N, K, device="cuda", generator=torch.Generator("cuda").manual_seed(7)) * 0.05
                 ).to(torch.bfloat16)
            for c in range(2 * calls):
                g = torch.Generator("cuda").manual_seed(100 * rank + c)
                x = torch.randn(t, K, device="cuda", generator=g).to(torch.bfloat16)
                # even calls: copy engines deliver the peers' rows; odd calls: copy CTAs inside the GEMM grid
                y, xg = all_gather_matmul(x, w, dist.group.WORLD, n_copy=0 if c % 2 == 0 else 8)
                ref_x = torch.empty(world * t, K, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(ref_x, x)
                ref = ref_x.float() @ w.float().t()
                errs.append(float((xg != ref_x).sum()))
                errs.append(float((y.float() - ref).abs().max() / ref.abs().max()))
        # GEMM -> reduce-scatter in the epilogue
        from lm_engine_b200.parallel.symm import matmul_reduce_scatter

        for (M, Kl, N), calls in (((512, 256, 768), 5), ((8192, 2048, 4096), 3), ((256, 136, 264), 2)):
            w = (torch.randn(N, Kl, device="cuda", generator=torch.Generator("cuda").manual_seed(11 + rank)) * 0.05
                 ).to(torch.bfloat16)
            bias = torch.randn(N, device="cuda", generator=torch.Generator("cuda").manual_seed(5)).to(torch.bfloat16)
            for c in range(calls):
                g = torch.Generator("cuda").manual_seed(1000 * rank + c)
                x = torch.randn(M, Kl, device="cuda", generator=g).to(torch.bfloat16)
                res = torch.randn(M // world, N, device="cuda", generator=g).to(torch.bfloat16)
                y = matmul_reduce_scatter(x, w, dist.group.WORLD, bias=bias, residual=res)
                part = (x.float() @ w.float().t()).to(torch.bfloat16).float()   # partial products travel as bf16
                dist.all_reduce(part)
                ref = part[rank * (M // world):(rank + 1) * (M // world)] + bias.float() + res.float()
                errs.append(0.0)
                errs.append(float((y.float() - ref).abs().max() / ref.abs().max()))
        torch.cuda.synchronize()
        q.put((rank, "ok", (errs, _lib.read_status())))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_all_gather_matmul_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, status, payload = q.get(timeout=240)
            assert status == "ok", payload
            res[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, (errs, status) in res.items():
        assert status[0] == 0, status
        for i in range(0, len(errs), 2):
            assert errs[i] == 0, f"rank {rank}: gathered operand differs ({errs[i]} elements)"
            assert errs[i + 1] < 1e-2, f"rank {rank}: GEMM error {errs[i + 1]}"


def _tp_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", LME_FUSED_TP="always")
    try:
        import torch.distributed as dist

        from lm_engine_b200.distributed import shard_model
        from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
        from lm_engine_b200.models import dense_config
        from lm_engine_b200.ops import _lib
        from lm_engine_b200.optimization.optimizer import ShardedOptimizer
        from lm_engine_b200.parallel import manager
        from lm_engine_b200.parallel.manager import ProcessGroupManager

        ProcessGroupManager(tensor_parallel_world_size=2, zero_stage=3)
        cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=1024, head_dim=64, max_position_embeddings=512)
        g = torch.Generator().manual_seed(3)
        data = torch.randint(0, 2048, (1, 513), generator=g).cuda()
        out = {}
        for fused in (False, True):
            manager._S.async_tp = fused
            launches = _lib.launch_count
            w = ModelWrapperForPretraining(pretrained_config=cfg.to_dict(), micro_batch_size=1, sequence_length=512,
                                           efficient_initialization=True, dtype="bf16", sequence_parallel=True)
            eng = shard_model(w, stage=3, dtype=torch.bfloat16, communication_dtype=None, seed=3)
            opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                       "eps": 1e-10}, None, False, 1.0)
            losses, norms = [], []
            for _ in range(4):
                opt.zero_grad()
                o = w(data if ProcessGroupManager.is_tensor_parallel_first_rank() else None,
                      lm_loss_multiplier=1 / 512)
                o["loss"].backward()
                norms.append(float(opt.step()))
                losses.append(float(o["loss"]))
            out[fused] = (losses, norms)
        torch.cuda.synchronize()
        q.put((rank, "ok", (out, _lib.read_status())))
        dist.barrier()
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_parallel_training_with_fused_collectives_matches_two_step_path():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", payload
            res[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, (out, status) in res.items():
        assert status[0] == 0, status
        (l0, n0), (l1, n1) = out[False], out[True]
        assert l0[-1] < l0[0]
        for a, b in zip(l0 + n0, l1 + n1):
            assert abs(a - b) <= 2e-2 * abs(a) + 1e-3, (out[False], out[True])
