"""Grouped (per-expert) tcgen05 GEMM and the token movement kernels around it at the shapes of the MoE target config
(64 experts, hidden 2048, SwiGLU 1024, top-8, 16384 tokens): device time of each launch, CUDA events after warm-up,
operand sets rotated so that every launch reads memory that is not in L2.

    python -m benchmarks.grouped_gemm_bench [--skew 4]

``--skew s``: expert e receives a share proportional to ``1 + (s - 1) * e / (E - 1)`` of the rows (1 = uniform).
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=1024)
    ap.add_argument("--skew", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()

    import torch

    from lm_engine_b200.ops import _lib
    from lm_engine_b200.ops.moe import (GroupLayout, combine_tokens, dispatch_tokens, grouped_linear_padded,
                                        topk_softmax)

    dev, bf = "cuda", torch.bfloat16
    T, K, E, H, I = a.tokens, a.top_k, a.experts, a.hidden, a.intermediate
    g = torch.Generator(device=dev).manual_seed(0)
    bias = torch.log(1 + (a.skew - 1) * torch.arange(E, device=dev) / max(E - 1, 1))
    n_sets = 3
    logits = [(torch.randn(T, E, device=dev, generator=g) + bias).to(bf) for _ in range(n_sets)]
    xs = [torch.randn(T, H, device=dev, generator=g).to(bf).requires_grad_(True) for _ in range(n_sets)]
    w1 = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.02).to(bf).requires_grad_(True)
    w2 = (torch.randn(E, H, I, device=dev, generator=g) * 0.02).to(bf).requires_grad_(True)

    def timed(fn, iters=a.iters):
        for i in range(3):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    routed = [topk_softmax(l, K, True) for l in logits]
    layouts = [GroupLayout.from_selection(sel, E) for _, sel in routed]
    rows = T * K
    print(f"tokens {T} top-k {K} experts {E} hidden {H} intermediate {I} skew {a.skew}: {rows} routed rows, "
          f"capacity {layouts[0].capacity}, largest expert {int(layouts[0].freq.max())}, smallest "
          f"{int(layouts[0].freq.min())}")
    t = timed(lambda i: topk_softmax(logits[i % n_sets], K, True))
    print(f"router top-k + softmax            {t * 1e3:8.1f} us")
    t = timed(lambda i: GroupLayout.from_selection(routed[i % n_sets][1], E))
    print(f"row layout (3 kernels)            {t * 1e3:8.1f} us")
    with torch.no_grad():
        t = timed(lambda i: dispatch_tokens(xs[i % n_sets], layouts[i % n_sets]))
        print(f"dispatch (scatter rows)           {t * 1e3:8.1f} us  {rows * H * 2 * 2 / t / 1e6:7.0f} GB/s")
        xp = [dispatch_tokens(xs[i], layouts[i]) for i in range(n_sets)]
        t1 = timed(lambda i: grouped_linear_padded(xp[i % n_sets], w1, layouts[i % n_sets], swiglu=True))
        f1 = 2 * rows * H * 2 * I
        print(f"expert fc1 + SwiGLU (grouped)     {t1 * 1e3:8.1f} us  {f1 / t1 / 1e9:7.0f} TFLOP/s")
        hs = [grouped_linear_padded(xp[i], w1, layouts[i], swiglu=True) for i in range(n_sets)]
        t2 = timed(lambda i: grouped_linear_padded(hs[i % n_sets], w2, layouts[i % n_sets]))
        f2 = 2 * rows * I * H
        print(f"expert fc2 (grouped)              {t2 * 1e3:8.1f} us  {f2 / t2 / 1e9:7.0f} TFLOP/s")
        ys = [grouped_linear_padded(hs[i], w2, layouts[i]) for i in range(n_sets)]
        gates = [w for w, _ in routed]
        t = timed(lambda i: combine_tokens(ys[i % n_sets], gates[i % n_sets], layouts[i % n_sets]))
        print(f"combine (weighted gather-reduce)  {t * 1e3:8.1f} us  {(rows + T) * H * 2 / t / 1e6:7.0f} GB/s")

    def fwd_bwd(i):
        j = i % n_sets
        w, sel = topk_softmax(logits[j], K, True)
        lay = GroupLayout.from_selection(sel, E)
        h = grouped_linear_padded(dispatch_tokens(xs[j], lay), w1, lay, swiglu=True)
        y = combine_tokens(grouped_linear_padded(h, w2, lay), w, lay)
        y.backward(torch.ones_like(y))

    t = timed(fwd_bwd, iters=5)
    print(f"whole expert block fwd + bwd      {t * 1e3:8.1f} us  {3 * (f1 + f2) / t / 1e9:7.0f} TFLOP/s (model FLOPs)")
    print("device status", _lib.read_status()[:4])


if __name__ == "__main__":
    main()
