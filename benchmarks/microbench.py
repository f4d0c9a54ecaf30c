"""Micro-benchmarks of the hand-written kernels against their roofline.

    python -m benchmarks.microbench [--json out.json] [--quick]

Timing: CUDA events on the launching stream, >= 3 warm-up launches, operands rotated through a pool larger than
the 126 MB L2 so every timed launch reads cold data.  GEMM throughput is reported next to ``torch.matmul`` (cuBLAS)
on the same operands and as a fraction of the measured bf16 peak when ``MEASURED_PEAKS.json`` is present.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from lm_engine_b200.ops import _lib, gemm


def _peaks() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _time(fn, n_pool: int, iters: int = 10, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i % n_pool)
    torch.cuda.synchronize()
    start = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    end = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        start[i].record()
        fn(i % n_pool)
        end[i].record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in zip(start, end))
    return times[len(times) // 2] * 1e-3


def _sustained(fn, n_pool: int, seconds: float = 1.5) -> float:
    """Mean seconds per call over a back-to-back loop long enough for the power limit to settle the clocks."""
    fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn(0)
    e1.record()
    torch.cuda.synchronize()
    n = max(8, int(seconds / max(e0.elapsed_time(e1) * 1e-3, 1e-6)))
    half = n // 2
    e0.record()
    for i in range(half):
        fn(i % n_pool)
    e1.record()           # first half warms the clocks down to their sustained level
    e2 = torch.cuda.Event(enable_timing=True)
    for i in range(half):
        fn(i % n_pool)
    e2.record()
    torch.cuda.synchronize()
    return e1.elapsed_time(e2) * 1e-3 / half


def bench_gemm(M, N, K, a_mn=False, b_mn=False, sustained=False, probe=0, **kw):
    dev = "cuda"
    bytes_per = 2 * (M * K + N * K + M * N)
    n_pool = max(2, min(8, int(300e6 // bytes_per) + 1))
    As = [torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16) for _ in range(n_pool)]
    Bs = [torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16) for _ in range(n_pool)]
    out = torch.empty((M, N // 2 if kw.get("swiglu") else N), device=dev, dtype=torch.bfloat16)
    timer = _sustained if sustained else _time
    t_ours = timer(lambda i: gemm(As[i], Bs[i], a_mn=a_mn, b_mn=b_mn, out=out, probe=probe, **kw), n_pool)

    def ref(i):
        A = As[i].t() if a_mn else As[i]
        B = Bs[i] if b_mn else Bs[i].t()
        torch.matmul(A, B)

    t_ref = timer(ref, n_pool)
    fl = 2.0 * M * N * K
    return {"M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn, "epilogue": ",".join(sorted(kw)) or "none",
            "ms": t_ours * 1e3, "tflops": fl / t_ours / 1e12, "cublas_ms": t_ref * 1e3,
            "cublas_tflops": fl / t_ref / 1e12}


def bench_gemm_fp8(M, N, K, sustained=False):
    """8-bit GEMM (pre-quantised operands) and the quantiser feeding it, on one forward-shaped problem."""
    from lm_engine_b200.ops import fp8

    dev = "cuda"
    n_pool = max(2, min(8, int(300e6 // (M * K + N * K + 2 * M * N)) + 1))
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(n_pool)]
    ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) for _ in range(n_pool)]
    xq = [fp8.quantize(x, fp8.E4M3) for x in xs]
    wq = [fp8.quantize(w, fp8.E4M3) for w in ws]
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    timer = _sustained if sustained else _time
    t = timer(lambda i: fp8.gemm_fp8(xq[i].q, 0, xq[i].scale_inv, wq[i].q, 0, wq[i].scale_inv, out=out), n_pool)
    tq = _time(lambda i: fp8.quantize(xs[i], fp8.E4M3, transposed=True), n_pool)
    return {"M": M, "N": N, "K": K, "ms": t * 1e3, "tflops": 2.0 * M * N * K / t / 1e12, "quantize_ms": tq * 1e3,
            "quantize_gbs": M * K * 4 / tq / 1e9}


def bench_elementwise(peaks: dict, small: bool = False) -> list[dict]:
    """Bandwidth-bound kernels at the 8B model's shapes: algorithmic bytes / device time against the measured copy
    bandwidth.  Operand sets rotate through a pool larger than L2."""
    from lm_engine_b200.ops import adamw_step, cross_entropy_sum, qkv_split_rope, rmsnorm, swiglu_backward
    from lm_engine_b200.ops import fp8

    dev, T, H, I = "cuda", 8192, 4096, 14336
    bf = torch.bfloat16
    pool = 2 if small else 3   # small: under 2 GB on the device for profiler captures, operands still > L2
    rows = []

    def add(name, fn, nbytes):
        t = _time(fn, pool)
        rows.append({"name": name, "ms": t * 1e3, "gbs": nbytes / t / 1e9,
                     "frac_of_hbm": nbytes / t / 1e9 / peaks["hbm_gbs"]})
        print(f"{name:28s} {t * 1e3:8.3f} ms  {nbytes / t / 1e9:7.0f} GB/s  "
              f"({100 * rows[-1]['frac_of_hbm']:5.1f}% of {peaks['source']} copy bandwidth)", flush=True)

    xs = [torch.randn(T, H, device=dev, dtype=bf) for _ in range(pool)]
    rs = [torch.randn(T, H, device=dev, dtype=bf) for _ in range(pool)]
    w = torch.ones(H, device=dev, dtype=bf, requires_grad=True)
    add("rmsnorm fwd (+residual)", lambda i: rmsnorm(xs[i], w, 1e-5, rs[i]), T * H * 2 * 4)
    ys = []
    for i in range(pool):
        x = xs[i].clone().requires_grad_(True)
        y, _ = rmsnorm(x, w, 1e-5)
        ys.append((x, y))
    g = torch.randn(T, H, device=dev, dtype=bf)
    add("rmsnorm bwd", lambda i: torch.autograd.grad(ys[i][1], ys[i][0], g, retain_graph=True), T * H * 2 * 3)
    pre = [torch.randn(T, 2 * I, device=dev, dtype=bf) for _ in range(pool)]
    dy = torch.randn(T, I, device=dev, dtype=bf)
    add("swiglu bwd", lambda i: swiglu_backward(pre[i], dy), T * I * 2 * (2 + 1 + 2))
    Hkv, G, D = 8, 4, 128
    qkv = [torch.randn(T, Hkv * (G + 2) * D, device=dev, dtype=bf) for _ in range(pool)]
    inv = 1.0 / (500000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(4096, device=dev).float(), inv)
    cos, sin = torch.cat((fr, fr), -1).cos(), torch.cat((fr, fr), -1).sin()
    add("qkv split + rope", lambda i: qkv_split_rope(qkv[i].view(2, 4096, -1), Hkv, G, D, cos, sin, None, 4096),
        T * Hkv * (G + 2) * D * 2 * 2)
    n = 40_000_000 if small else 218_112_000 // 2
    ps = [(torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev),
           torch.randn(n, device=dev, dtype=bf), torch.empty(n, device=dev, dtype=bf)) for _ in range(2)]
    one = torch.ones(1, device=dev)
    add("adamw (fp32 state, bf16 grad+copy)",
        lambda i: adamw_step(ps[i % 2][0], ps[i % 2][1], ps[i % 2][2], ps[i % 2][3], ps[i % 2][4], lr=1e-4,
                             betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1, step=3, gscale=one), n * (12 + 12 + 2 + 2))
    V = 128256
    ce_rows = 1024 if small else 2048
    lg = [torch.randn(ce_rows, V, device=dev, dtype=bf) for _ in range(pool)]
    lb = torch.randint(0, V, (ce_rows,), device=dev)
    add("cross entropy fwd (logits)", lambda i: cross_entropy_sum(lg[i], lb), ce_rows * V * 2)
    add("fp8 quantize + transpose", lambda i: fp8.quantize(xs[i], fp8.E4M3, transposed=True), T * H * (2 + 2 + 1 + 1))
    return rows


def bench_recurrent(small: bool = False) -> list[dict]:
    """Scan kernels at training shapes: ms per call and ns per time step (the scans are latency chains, so time per
    step is the figure of merit), plus the PyTorch time loop on a 128-step prefix for scale."""
    from lm_engine_b200.ops import m2rnn as m2op
    from lm_engine_b200.ops import rnn as rnnop
    from lm_engine_b200.ops.recurrence import gru_scan, m2rnn_scan, rnn_scan

    dev, bf = "cuda", torch.bfloat16
    B, S = 2, (512 if small else 4096)
    rows = []

    def add(name, make, ref):
        args = make(S)
        for a in args:
            if isinstance(a, torch.Tensor):
                a.requires_grad_(True)
        fwd = _time(lambda i: make_call(name, args), 1, iters=5, warmup=2)

        def both(i):
            y, h = make_call(name, args)
            y.backward(torch.ones_like(y))

        tot = _time(both, 1, iters=5, warmup=2)
        short = tuple(a.to(bf) if isinstance(a, torch.Tensor) else a for a in make(128))
        loop = _time(lambda i: ref(*short), 1, iters=2, warmup=1)
        rows.append({"name": name, "S": S, "fwd_ms": fwd * 1e3, "fwd_bwd_ms": tot * 1e3,
                     "fwd_ns_per_step": fwd * 1e9 / S, "torch_loop_fwd_ms_at_128_steps": loop * 1e3})
        print(f"{name:34s} S={S}  fwd {fwd * 1e3:7.3f} ms ({fwd * 1e9 / S:6.0f} ns/step)  fwd+bwd {tot * 1e3:7.3f} ms"
              f"   PyTorch loop fwd, 128 steps: {loop * 1e3:7.2f} ms", flush=True)

    def make_call(name, args):
        if name.startswith("m2rnn"):
            return m2op.m2rnn_cuda(*args)
        if name.startswith("gru"):
            return rnnop.gru_cuda(*args)
        return rnnop.rnn_cuda(*args)

    def m2(N, K, V, shared):
        def make(s):
            nq = 1 if shared else N
            return (torch.randn(B, s, nq, K, device=dev).to(bf) * 0.5, torch.randn(B, s, nq, K, device=dev).to(bf) * 0.5,
                    torch.randn(B, s, N, V, device=dev).to(bf), torch.sigmoid(torch.randn(B, s, N, device=dev) + 2),
                    (torch.eye(V, device=dev) + 0.05 * torch.randn(N, V, V, device=dev)).to(bf), None, 1.0)
        return make

    def vec(N, H, gates):
        def make(s):
            xs = [torch.randn(B, s, N, H, device=dev).to(bf) for _ in range(gates)]
            ws = [(torch.randn(N, H, H, device=dev) / H ** 0.5).to(bf) for _ in range(gates)]
            return (*xs, *ws, None, 1.0)
        return make

    # the chunk-parallel forms at the published gated-delta-net layout (block operands by batched matmuls and a
    # triangular solve in PyTorch; the delta rule's chain over the blocks on its own kernels)
    from lm_engine_b200.ops.recurrence import gated_delta_rule, linear_attention

    def chunked(name, fn, make_args):
        args = make_args()
        for a in args:
            if isinstance(a, torch.Tensor) and a.is_floating_point():
                a.requires_grad_(True)
        fwd = _time(lambda i: fn(*args), 1, iters=5, warmup=2)

        def both(i):
            y, _ = fn(*args)
            y.backward(torch.ones_like(y))

        tot = _time(both, 1, iters=5, warmup=2)
        rows.append({"name": name, "S": S, "fwd_ms": fwd * 1e3, "fwd_bwd_ms": tot * 1e3})
        print(f"{name:34s} S={S}  fwd {fwd * 1e3:7.3f} ms  fwd+bwd {tot * 1e3:7.3f} ms   (chunk-parallel form)",
              flush=True)

    def gdn_args():
        N, K, V = 3, 256, 512
        return (torch.randn(B, S, N, K, device=dev).to(bf), torch.randn(B, S, N, K, device=dev).to(bf),
                torch.randn(B, S, N, V, device=dev).to(bf), -torch.rand(B, S, N, device=dev) * 0.1,
                torch.rand(B, S, N, device=dev))

    chunked("gated delta rule K=256 V=512 N=3", gated_delta_rule, gdn_args)
    chunked("linear attention K=64 V=64 N=32", linear_attention,
            lambda: tuple(torch.randn(B, S, 32, 64, device=dev).to(bf) * 0.3 for _ in range(3)))
    add("m2rnn K=64 V=16 N=132 (shared q,k)", m2(132, 64, 16, True), m2rnn_scan)
    add("m2rnn K=64 V=64 N=32", m2(32, 64, 64, False), m2rnn_scan)
    add("rnn H=16 N=128", vec(128, 16, 1), rnn_scan)
    add("gru H=16 N=128", vec(128, 16, 3), gru_scan)
    return rows


def bench_attention(peaks: dict, small: bool = False) -> list[dict]:
    """Own tcgen05 attention forward against the library (cuDNN through SDPA) forward at training shapes."""
    import torch.nn.functional as F

    from lm_engine_b200.ops.attention_cuda import flash_attention_forward

    rows = []
    for name, B, S, Hq, Hkv in ([("capture", 1, 8192, 8, 2)] if small else
                                [("8b-shape", 2, 4096, 32, 8), ("1b-shape", 2, 4096, 16, 8), ("long", 1, 16384, 32, 8)]):
        qkv = torch.randn(B, S, (Hq + 2 * Hkv) * 128, device="cuda").to(torch.bfloat16)
        q, k, v = (t.view(B, S, -1, 128) for t in qkv.split((Hq * 128, Hkv * 128, Hkv * 128), dim=-1))
        scale = 128 ** -0.5
        flops = 4 * B * Hq * S * S * 128 / 2
        ours = _time(lambda i: flash_attention_forward(q, k, v, causal=True, softmax_scale=scale), 1)
        qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
        lib = _time(lambda i: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale,
                                                             enable_gqa=True), 1)
        r = {"name": name, "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "ms": ours * 1e3, "tflops": flops / ours / 1e12,
             "library_ms": lib * 1e3, "library_tflops": flops / lib / 1e12,
             "frac_of_peak": flops / ours / 1e12 / peaks["bf16_tflops"]}
        print(f"attention fwd causal {name:9s} B={B} S={S} Hq={Hq} Hkv={Hkv}: ours {r['ms']:7.3f} ms {r['tflops']:6.1f} TF "
              f"({100 * r['frac_of_peak']:4.1f}% of {peaks['source']} GEMM peak)   library {r['library_ms']:7.3f} ms "
              f"{r['library_tflops']:6.1f} TF", flush=True)
        # backward alone (2.5x the forward FLOPs by the usual count: 5 products against 2)
        from .attention_cuda import flash_attention_backward

        out, lse = flash_attention_forward(q, k, v, causal=True, softmax_scale=scale, return_lse=True)
        dout = torch.randn_like(out)
        bwd = _time(lambda i: flash_attention_backward(dout, q, k, v, out, lse, causal=True, softmax_scale=scale), 1)
        ql, kl, vl = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        ol = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, scale=scale, enable_gqa=True)
        dl = dout.transpose(1, 2)
        lib_bwd = _time(lambda i: torch.autograd.grad(ol, (ql, kl, vl), dl, retain_graph=True), 1)
        r.update({"bwd_ms": bwd * 1e3, "bwd_tflops": 2.5 * flops / bwd / 1e12, "library_bwd_ms": lib_bwd * 1e3,
                  "library_bwd_tflops": 2.5 * flops / lib_bwd / 1e12})
        rows.append(r)
        print(f"attention bwd causal {name:9s}: ours {r['bwd_ms']:7.3f} ms {r['bwd_tflops']:6.1f} TF (incl. the delta "
              f"pass)   library {r['library_bwd_ms']:7.3f} ms {r['library_bwd_tflops']:6.1f} TF", flush=True)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--attention", action="store_true", help="time the attention forward kernel instead")
    ap.add_argument("--recurrent", action="store_true", help="time the RNN-family scan kernels instead")
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--sustained", action="store_true", help="time ~1.5 s back-to-back loops (power-limited clocks)")
    ap.add_argument("--fp8", action="store_true", help="also time the 8-bit GEMM and its quantiser")
    ap.add_argument("--elementwise", action="store_true", help="time the bandwidth-bound kernels instead")
    ap.add_argument("--small", action="store_true", help="smaller operand pools (profiler captures)")
    ap.add_argument("--only", default=None, help="run the one shape with this name (small profiler captures)")
    ap.add_argument("--probe", default=None, choices=["noload", "nomma"],
                    help="GEMM timing probe: skip the operand loads (tensor-pipe ceiling) or the MMAs (load ceiling)")
    args = ap.parse_args()
    peaks = _peaks()
    if args.attention:
        rows = bench_attention(peaks, small=args.small)
        st = _lib.read_status()
        print("device status:", st)
        if args.json:
            json.dump({"peaks": peaks, "attention": rows, "status": st}, open(args.json, "w"), indent=1)
        return
    if args.recurrent:
        rows = bench_recurrent(small=args.small)
        st = _lib.read_status()
        print("device status:", st)
        if args.json:
            json.dump({"recurrent": rows, "status": st}, open(args.json, "w"), indent=1)
        return
    if args.elementwise:
        rows = bench_elementwise(peaks, small=args.small)
        st = _lib.read_status()
        print("device status:", st)
        if args.json:
            json.dump({"peaks": peaks, "elementwise": rows, "status": st}, open(args.json, "w"), indent=1)
        return
    T = 8192
    shapes = [
        ("qkv fwd", T, 6144, 4096, False, False, {}),
        ("attn-out fwd", T, 4096, 4096, False, False, {}),
        ("fc1+swiglu fwd", T, 28672, 4096, False, False, {"swiglu": True}),
        ("fc2 fwd", T, 4096, 14336, False, False, {}),
        ("fc1 dgrad", T, 4096, 28672, False, True, {}),
        ("fc1 wgrad", 28672, 4096, T, True, True, {}),
        ("fc2 wgrad", 4096, 14336, T, True, True, {}),
        ("lm-head fwd", T, 128256, 4096, False, False, {}),
    ]
    if args.quick:
        shapes = shapes[:3]
    if args.only is not None:
        shapes = [s for s in shapes if s[0] == args.only]
        assert shapes, f"no shape named {args.only!r}"
    rows = []
    for name, M, N, K, a_mn, b_mn, kw in shapes:
        r = bench_gemm(M, N, K, a_mn, b_mn, sustained=args.sustained,
                       probe={"noload": 64, "nomma": 128, None: 0}[args.probe], **kw)
        r["name"] = name
        r["frac_of_peak"] = r["tflops"] / peaks["bf16_tflops_sustained" if args.sustained else "bf16_tflops"]
        rows.append(r)
        print(f"{name:16s} M={M:6d} N={N:6d} K={K:6d}  ours {r['ms']:8.3f} ms {r['tflops']:7.1f} TF "
              f"({100 * r['frac_of_peak']:5.1f}% of {peaks['source']} peak)   cuBLAS {r['cublas_ms']:8.3f} ms "
              f"{r['cublas_tflops']:7.1f} TF", flush=True)
    if args.fp8:
        for name, M, N, K, a_mn, b_mn, kw in shapes:
            if a_mn or b_mn or kw:
                continue
            r = bench_gemm_fp8(M, N, K, sustained=args.sustained)
            r["name"] = name + " fp8"
            rows.append(r)
            print(f"{name:16s} fp8 e4m3  M={M:6d} N={N:6d} K={K:6d}  {r['ms']:8.3f} ms {r['tflops']:7.1f} TF   "
                  f"quantize(+transpose) {r['quantize_ms']:7.3f} ms {r['quantize_gbs']:6.0f} GB/s", flush=True)
    st = _lib.read_status()
    print("device status:", st)
    if args.json:
        json.dump({"peaks": peaks, "gemm": rows, "status": st}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
