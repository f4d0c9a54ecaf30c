"""Times the fused all-gather -> GEMM kernel against its two-step equivalent (NCCL all-gather, then the same GEMM)
and against the GEMM alone on an already gathered operand (the floor).  One process per GPU::

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m benchmarks.symm_bench

Device time by CUDA events around ``iters`` back-to-back calls after warm-up, max over ranks; operands rotate through a
pool larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from lm_engine_b200.ops import _lib
from lm_engine_b200.ops.gemm import gemm
from lm_engine_b200.parallel.symm import all_gather_matmul


def _time(fn, iters: int, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="rows of the gathered operand (all ranks together)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--copy-ctas", type=int, default=16)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    T, rows = a.tokens, []
    for name, K, N_full in (("qkv", 4096, 6144), ("fc1", 4096, 28672)):
        N, t = N_full // world, T // world
        pool = 4
        xs = [torch.randn(t, K, device="cuda").to(torch.bfloat16) for _ in range(pool)]
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(pool)]
        full = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)

        def fused(i):
            all_gather_matmul(xs[i % pool], ws[i % pool], dist.group.WORLD, n_copy=0)

        def fused_ctas(i):
            all_gather_matmul(xs[i % pool], ws[i % pool], dist.group.WORLD, n_copy=a.copy_ctas)

        def two_step(i):
            dist.all_gather_into_tensor(full, xs[i % pool])
            gemm(full, ws[i % pool], out=out)

        def floor(i):
            gemm(full, ws[i % pool], out=out)

        # numerical check of both fused forms against the two-step result
        two_step(0)
        want = out.float().clone()
        errs = []
        for nc in (0, a.copy_ctas):
            y, xg = all_gather_matmul(xs[0], ws[0], dist.group.WORLD, n_copy=nc)
            errs.append(float((y.float() - want).abs().max() / want.abs().max()))
            errs.append(float((xg != full).sum()))
        r_err = max(errs)
        r = {"name": name, "world": world, "M": T, "N": N, "K": K, "max_err": r_err,
             "fused_ms": _time(fused, a.iters),
             "fused_copy_ctas_ms": _time(fused_ctas, a.iters), "copy_ctas": a.copy_ctas,
             "nccl_then_gemm_ms": _time(two_step, a.iters), "gemm_only_ms": _time(floor, a.iters)}
        r["nvlink_bytes_in"] = (world - 1) * t * K * 2
        r["fused_tflops"] = 2.0 * T * N * K / (r["fused_ms"] * 1e-3) / 1e12
        rows.append(r)
        if rank == 0:
            print(f"{name:4s} M={T} N={N} K={K} world={world}: fused (copy engines feed the GEMM) {r['fused_ms']:.3f} ms "
                  f"({r['fused_tflops']:.0f} TF) | fused ({a.copy_ctas} copy CTAs in the grid) "
                  f"{r['fused_copy_ctas_ms']:.3f} ms | NCCL all-gather + GEMM {r['nccl_then_gemm_ms']:.3f} ms | GEMM alone {r['gemm_only_ms']:.3f} ms"
                  f" | max err vs two-step {r['max_err']:.2e}",
                  flush=True)
    # GEMM -> reduce-scatter: row-parallel projections (contraction dim split over the ranks)
    from lm_engine_b200.parallel.symm import matmul_reduce_scatter

    for name, K_full, N in (("attn-out", 4096, 4096), ("fc2", 14336, 4096)):
        Kl, pool = K_full // world, 4
        xs = [torch.randn(T, Kl, device="cuda").to(torch.bfloat16) for _ in range(pool)]
        ws = [(torch.randn(N, Kl, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(pool)]
        full = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        shard = torch.empty(T // world, N, device="cuda", dtype=torch.bfloat16)

        def fused_rs(i):
            matmul_reduce_scatter(xs[i % pool], ws[i % pool], dist.group.WORLD)

        def two_step_rs(i):
            gemm(xs[i % pool], ws[i % pool], out=full)
            dist.reduce_scatter_tensor(shard, full)

        def floor_rs(i):
            gemm(xs[i % pool], ws[i % pool], out=full)

        two_step_rs(0)
        got = matmul_reduce_scatter(xs[0], ws[0], dist.group.WORLD)
        r_err = float((got.float() - shard.float()).abs().max() / shard.float().abs().max())
        r = {"name": name, "world": world, "M": T, "N": N, "K": Kl, "max_err": r_err,
             "fused_ms": _time(fused_rs, a.iters),
             "gemm_then_nccl_ms": _time(two_step_rs, a.iters), "gemm_only_ms": _time(floor_rs, a.iters)}
        r["nvlink_bytes_out"] = (world - 1) * (T // world) * N * 2
        r["fused_tflops"] = 2.0 * T * N * Kl / (r["fused_ms"] * 1e-3) / 1e12
        rows.append(r)
        if rank == 0:
            print(f"{name:8s} M={T} N={N} K={Kl} world={world}: fused GEMM+reduce-scatter {r['fused_ms']:.3f} ms "
                  f"({r['fused_tflops']:.0f} TF) | GEMM + NCCL reduce-scatter {r['gemm_then_nccl_ms']:.3f} ms | "
                  f"GEMM alone {r['gemm_only_ms']:.3f} ms | max err vs two-step {r['max_err']:.2e}", flush=True)
    st = _lib.read_status()
    if rank == 0:
        print("device status:", st)
        if a.json:
            json.dump({"rows": rows, "status": st}, open(a.json, "w"), indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
