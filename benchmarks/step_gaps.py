"""Where the compute stream of a training step waits: torch-profiler trace of ONE step of the headline model (fewer
layers, same shapes), per-stream kernel totals and the idle gaps of the busiest stream with the kernels around them.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m benchmarks.step_gaps --layers 8 --out /tmp/trace.json

Timings under the profiler are for shares and gaps only, never benchmark values; the unprofiled step time is printed
first (CUDA events, 2 steps after 3 warm-up steps).
"""

from __future__ import annotations

import argparse
import collections
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--out", default=os.path.join(os.environ.get("TMPDIR", "/tmp"), "lme_step_trace.json"))
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel group size (mixture-of-experts models)")
    ap.add_argument("--kernels", type=int, default=4, help="kernel names listed per stream, by total time")
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    import bench
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.data.synthetic import SyntheticBatchIterator
    from lm_engine_b200.distributed import wrap_model_container_for_distributed_training
    from lm_engine_b200.kernels import enable_kernels
    from lm_engine_b200.model_wrapper import get_model_container
    from lm_engine_b200.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.train import train_step_without_pipeline_parallel
    from lm_engine_b200.utils import disable_generation_cache

    bench.LAYERS_OVERRIDE = a.layers
    cfg = bench.training_config(a.model, a.seq, a.mbs, 1, ["fused_linear_cross_entropy"], None)
    cfg["distributed_args"]["expert_parallel_world_size"] = a.ep
    args = TrainingArgs(**cfg)
    ProcessGroupManager(zero_stage=3, expert_parallel_world_size=a.ep)
    rank, world = ProcessGroupManager.get_global_rank(), ProcessGroupManager.get_world_size()
    args.training_parameters.reset_training_parameters(ProcessGroupManager.get_data_loading_world_size())
    models = get_model_container(args)
    models, _ = wrap_model_container_for_distributed_training(args, models)
    opts = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, models, None, max_grad_norm=1.0)
    scheds = get_scheduler_container(models, opts, 5, 0, None, 10**6, args.lr_scheduler_args.lr_decay_style, 0.1, {})
    models.train()
    it = SyntheticBatchIterator(bench.MODELS[a.model][0], a.seq, a.mbs, rank=rank, world=world)

    def step():
        return train_step_without_pipeline_parallel(models, opts, scheds, it, 1, 1.0, reduce_metrics=True)

    with disable_generation_cache(), enable_kernels(args.kernel_args.kernels):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        step()
        e1.record()
        torch.cuda.synchronize()
        if rank == 0:
            print("unprofiled ms/step", e0.elapsed_time(e1) / 2, flush=True)
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            step()
            torch.cuda.synchronize()
    if rank == 0:
        prof.export_chrome_trace(a.out)
        events = [e for e in json.load(open(a.out))["traceEvents"]
                  if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
        os.remove(a.out)
        streams = collections.defaultdict(list)
        for e in events:
            streams[e["args"].get("stream")].append(e)
        busy = {s: sum(e["dur"] for e in v) for s, v in streams.items()}
        main_stream = max(busy, key=busy.get)
        t0 = min(e["ts"] for e in events)
        t1 = max(e["ts"] + e["dur"] for e in events)
        print("world", world, "layers", a.layers, "span_us", round(t1 - t0))
        for s, v in sorted(streams.items(), key=lambda kv: -busy[kv[0]]):
            names = collections.Counter()
            for e in v:
                names[e["name"].split("<")[0].split("(")[0][:60]] += e["dur"]
            print(f"stream {s}: n={len(v)} busy_us={busy[s]:.0f}", [(k, round(d)) for k, d in names.most_common(a.kernels)])
        v = sorted(streams[main_stream], key=lambda e: e["ts"])
        gaps = [(n["ts"] - (p["ts"] + p["dur"]), p["name"][:50], n["name"][:50], p["ts"] - t0)
                for p, n in zip(v, v[1:]) if n["ts"] - (p["ts"] + p["dur"]) > 3]
        print("busiest stream", main_stream, "busy_us", round(busy[main_stream]), "idle_us (gaps > 3 us)",
              round(sum(g[0] for g in gaps)), "gaps", len(gaps))
        for g in sorted(gaps, reverse=True)[:a.top]:
            print(f"  gap {g[0]:8.0f} us at {g[3]:9.0f}  after {g[1]}  before {g[2]}")
    if dist.is_initialized():
        dist.barrier()
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()
