"""Out-of-bounds and determinism checks of the hand-written kernels without a sanitizer: outputs sit inside larger
allocations whose borders hold a canary pattern that must survive, and every kernel runs twice on the same inputs and
has to return the same bits (none of them uses atomics on its outputs)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

CANARY = 0x7A5C


def _guarded(shape, dtype, pad=4096):
    """A tensor of `shape` inside a flat buffer with `pad` canary elements on both sides."""
    n = 1
    for s in shape:
        n *= s
    flat = torch.empty(n + 2 * pad, dtype=dtype, device="cuda")
    raw = flat.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)
    raw.fill_(CANARY)
    return flat, flat[pad:pad + n].view(shape), pad


def _intact(flat, pad, dtype):
    raw = flat.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)
    return bool((raw[:pad] == CANARY).all()) and bool((raw[-pad:] == CANARY).all())


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(384, 520, 200, False, False), (200, 136, 328, False, True),
                                             (264, 392, 136, True, True), (128, 8, 64, False, False)])
def test_gemm_stays_inside_its_output_and_is_deterministic(M, N, K, a_mn, b_mn):
    from lm_engine_b200.ops import _lib, gemm

    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).to(torch.bfloat16)
    outs = []
    for _ in range(2):
        flat, out, pad = _guarded((M, N), torch.bfloat16)
        gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out)
        torch.cuda.synchronize()
        assert _intact(flat, pad, torch.bfloat16)
        outs.append(out.clone())
    assert torch.equal(outs[0], outs[1])
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    assert float((outs[0].float() - A @ B).norm() / (A @ B).norm()) < 1e-2
    assert _lib.read_status()[0] == 0


def test_bmm_stays_inside_its_output():
    from lm_engine_b200.ops.gemm import _bmm_kernel

    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(5, 200, 72, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(5, 40, 72, device="cuda", generator=g).to(torch.bfloat16)
    import lm_engine_b200.ops.gemm  # noqa: F401
    import sys

    mod = sys.modules["lm_engine_b200.ops.gemm"]
    flat, out, pad = _guarded((5, 200, 40), torch.float32)
    rc = mod._lib.cuda_lib().lme_gemm_bf16_batched(
        a.data_ptr(), 0, a.stride(1), a.stride(0), b.data_ptr(), 0, b.stride(1), b.stride(0), out.data_ptr(),
        out.stride(1), out.stride(0), 5, 200, 40, 72, mod._lib.GEMM_OUT_F32, 0, mod._lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert _intact(flat, pad, torch.float32)
    ref = torch.bmm(a.float(), b.float().transpose(1, 2))
    assert float((out - ref).norm() / ref.norm()) < 2e-3
    assert torch.equal(_bmm_kernel(a, b, False, False, torch.float32), out)


def test_rmsnorm_and_reduce_scatter_stay_inside_their_outputs():
    import ctypes

    from lm_engine_b200.ops import _lib, rmsnorm

    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(300, 1032, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(1032, device="cuda", generator=g).to(torch.bfloat16)
    a = rmsnorm(x, w, 1e-5)[0]
    b = rmsnorm(x, w, 1e-5)[0]
    assert torch.equal(a, b)
    # reduce-scatter kernel with four local "ranks" (every signal word already set)
    lib = _lib.cuda_lib()
    n, world, rank = 128 * 77, 4, 1
    bufs = [torch.randn(world * n, device="cuda", generator=g).to(torch.bfloat16) for _ in range(world)]
    srcs = (ctypes.c_void_p * 8)(*([t.data_ptr() + rank * n * 2 for t in bufs] + [None] * 4))
    pads = [torch.full((16,), 5, dtype=torch.int32, device="cuda") for _ in range(world)]
    pad_arr = (ctypes.c_void_p * 8)(*([p.data_ptr() for p in pads] + [None] * 4))
    flat, out, pad = _guarded((n,), torch.bfloat16)
    part_flat, part, ppad = _guarded((24,), torch.float32, pad=64)
    _lib.check(lib.lme_reduce_scatter_peers(srcs, pad_arr, None, rank, world, 5, out.data_ptr(), n, 1, 0.25, 0,
                                            part.data_ptr(), 24, _lib.stream_ptr()), "lme_reduce_scatter_peers")
    torch.cuda.synchronize()
    assert _intact(flat, pad, torch.bfloat16) and _intact(part_flat, ppad, torch.float32)
    assert _lib.read_status()[0] == 0
