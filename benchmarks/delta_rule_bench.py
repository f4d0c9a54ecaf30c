"""Gated delta rule layer core (``ops.recurrence.gated_delta_rule``): device time of the forward pass and of forward +
backward at one layout, CUDA events after warm-up.

    python -m benchmarks.delta_rule_bench --batch 2 --seq 4096 --heads 3 --k 256 --v 512

``--iters 1 --warmup 0`` makes a short run for a profiler capture of the chain kernels
(``-k regex:delta_chain``); numbers printed under a profiler are not benchmark values.
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=3)
    ap.add_argument("--k", type=int, default=256)
    ap.add_argument("--v", type=int, default=512)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()

    import torch

    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.recurrence import gated_delta_rule

    dev, bf = "cuda", torch.bfloat16
    B, S, N, K, V = a.batch, a.seq, a.heads, a.k, a.v
    g = torch.Generator(device=dev).manual_seed(0)
    args = [torch.randn(B, S, N, K, device=dev, generator=g).to(bf), torch.randn(B, S, N, K, device=dev, generator=g).to(bf),
            torch.randn(B, S, N, V, device=dev, generator=g).to(bf), -torch.rand(B, S, N, device=dev, generator=g) * 0.1,
            torch.rand(B, S, N, device=dev, generator=g)]
    for t in args:
        t.requires_grad_(True)

    def fwd():
        return gated_delta_rule(*args)[0]

    def both():
        y = fwd()
        y.backward(torch.ones_like(y))

    def timed(fn) -> float:
        for _ in range(a.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters

    with torch.no_grad():
        f = timed(fwd)
    fb = timed(both)
    print(f"gated delta rule B={B} S={S} heads={N} K={K} V={V}: fwd {f:.3f} ms  fwd+bwd {fb:.3f} ms  "
          f"status {_lib.read_status()[:2]}", flush=True)


if __name__ == "__main__":
    main()
