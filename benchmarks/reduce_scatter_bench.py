"""Times the gradient reduce-scatter kernel (csrc/kernels/reduce_scatter.cu) by itself.

    python -m benchmarks.reduce_scatter_bench                      # 1 GPU: 8 local buffers stand in for the ranks
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        -m benchmarks.reduce_scatter_bench [--nvls]                # the real thing over NVLink

Per CTA count: device time (CUDA events, max over ranks, 3 warm-up + 10 timed launches), bytes that cross NVLink into
this GPU per launch ((world - 1) x shard) divided by that time, and the fraction of the measured 770 GB/s per
direction peer-copy rate.  On one GPU the figure is local HBM traffic ((world + 1) x shard) against the measured copy
bandwidth.  Every launch also waits for the peers' announcement of its sequence number, as in training.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=int, default=218_112_000, help="elements of the unreduced buffer (one 8B block)")
    ap.add_argument("--ctas", default="16,32,48,96,148,296")
    ap.add_argument("--nvls", action="store_true", help="read through the switch (multimem.ld_reduce)")
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()

    import torch
    import torch.distributed as dist

    from lm_engine_b200.ops import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lib = _lib.cuda_lib()
    dtype = torch.float32 if a.fp32 else torch.bfloat16
    esz = 4 if a.fp32 else 2
    if world > 1:
        import torch.distributed._symmetric_memory as symm_mem

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl")
        ranks = world
        numel = a.elements // (128 * ranks) * (128 * ranks)
        buf = symm_mem.empty(numel, dtype=dtype, device="cuda")
        buf.normal_()
        handle = symm_mem.rendezvous(buf, dist.group.WORLD)
        pad = symm_mem.empty(16, dtype=torch.int32, device="cuda")
        pad.zero_()
        pad_handle = symm_mem.rendezvous(pad, dist.group.WORLD)
        shard = numel // ranks
        srcs = [handle.get_buffer(r, (numel,), dtype, 0).data_ptr() + rank * shard * esz for r in range(ranks)]
        pads = [pad_handle.get_buffer(r, (16,), torch.int32, 0).data_ptr() for r in range(ranks)]
        mc = int(handle.multicast_ptr or 0) if a.nvls else 0
        mc_src = mc + rank * shard * esz if mc else None
        torch.cuda.synchronize()
        dist.barrier()
    else:
        ranks = 8
        numel = a.elements // (128 * ranks) * (128 * ranks)
        shard = numel // ranks
        bufs = [torch.randn(numel, device="cuda").to(dtype) for _ in range(ranks)]
        srcs = [b.data_ptr() for b in bufs]            # "rank 0" owns the first shard of every buffer
        pad_t = [torch.full((16,), 1 << 30, dtype=torch.int32, device="cuda") for _ in range(ranks)]
        pads = [p.data_ptr() for p in pad_t]
        mc_src = None
    src_arr = (ctypes.c_void_p * 8)(*(srcs + [None] * (8 - ranks)))
    pad_arr = (ctypes.c_void_p * 8)(*(pads + [None] * (8 - ranks)))
    out = torch.empty(shard, dtype=dtype, device="cuda")
    partials = torch.zeros(1184, dtype=torch.float32, device="cuda")
    seq = 0
    rows = []
    for ctas in [int(c) for c in a.ctas.split(",")]:
        times = []
        for i in range(13):
            seq += 1
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(lib.lme_reduce_scatter_peers(src_arr, pad_arr, mc_src, rank if world > 1 else 0, ranks, seq,
                                                    out.data_ptr(), shard, int(not a.fp32), 1.0 / ranks, 0,
                                                    partials.data_ptr(), ctas, _lib.stream_ptr()),
                       "lme_reduce_scatter_peers")
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor(sorted(times)[len(times) // 2], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
        moved = ((ranks - 1) if world > 1 else (ranks + 1)) * shard * esz
        rows.append({"ctas": ctas, "ms": ms, "gbs": moved / ms / 1e6, "bytes": moved})
        if rank == 0:
            what = "over NVLink into this GPU" if world > 1 else "of local HBM traffic"
            print(f"ctas {ctas:4d}  {ms:7.3f} ms  {moved / ms / 1e6:7.0f} GB/s {what}"
                  + (f"  ({moved / ms / 1e6 / 770:.2f} of the 770 GB/s peer-copy rate)" if world > 1 else ""),
                  flush=True)
    status = _lib.read_status()
    if rank == 0:
        print("device status:", status, "ranks", ranks, "shard MB", shard * esz / 1e6, "nvls", bool(mc_src))
        if a.json:
            json.dump({"world": world, "rows": rows, "status": status}, open(a.json, "w"), indent=1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
