"""The fused gradient reduce-scatter kernel on ONE GPU: the "ranks" are slices of local buffers and every signal word
is already set when the kernel starts, so nothing waits on another launch.  Checked against an fp32 PyTorch sum:
mean over ranks, overwrite and accumulate, bf16 and fp32 gradients, per-CTA partial sums of squares."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(world, rank, n, dtype, accumulate, ctas):
    from lm_engine_b200.ops import _lib

    lib = _lib.cuda_lib()
    torch.manual_seed(world * 100 + rank)
    bufs = [torch.randn(world * n, device="cuda").to(dtype) for _ in range(world)]      # every rank's full buffer
    esz = bufs[0].element_size()
    srcs = (ctypes.c_void_p * 8)(*([b.data_ptr() + rank * n * esz for b in bufs] + [None] * (8 - world)))
    seq = 3
    pads = [torch.full((16,), seq, dtype=torch.int32, device="cuda") for _ in range(world)]   # all announced
    pad_arr = (ctypes.c_void_p * 8)(*([p.data_ptr() for p in pads] + [None] * (8 - world)))
    out = torch.randn(n, device="cuda").to(dtype)
    old = out.clone()
    partials = torch.full((ctas,), -1.0, device="cuda")
    scale = 1.0 / world
    _lib.check(lib.lme_reduce_scatter_peers(srcs, pad_arr, None, rank, world, seq, out.data_ptr(), n,
                                            int(dtype == torch.bfloat16), scale, int(accumulate),
                                            partials.data_ptr(), ctas, _lib.stream_ptr()), "lme_reduce_scatter_peers")
    total = torch.zeros(1, device="cuda")
    _lib.check(lib.lme_sum_partials(partials.data_ptr(), ctas, total.data_ptr(), 0, _lib.stream_ptr()),
               "lme_sum_partials")
    torch.cuda.synchronize()
    ref = sum(b[rank * n:(rank + 1) * n].float() for b in bufs) * scale
    if accumulate:
        ref = ref + old.float()
    assert _lib.read_status()[0] == 0
    return out, ref, float(total)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("accumulate", [False, True])
def test_reduce_scatter_kernel_matches_fp32_sum(world, dtype, accumulate):
    n = 128 * 1031                      # not a multiple of the grid's stride: exercises the ragged last pass
    out, ref, total = _run(world, world - 1, n, dtype, accumulate, ctas=24)
    tol = 8e-3 if dtype == torch.bfloat16 else 1e-6
    assert torch.allclose(out.float(), ref, rtol=tol, atol=tol)
    want = float(out.float().pow(2).sum())           # the norm is taken of the stored (rounded) values
    assert abs(total - want) <= 1e-4 * want


def test_reduce_scatter_kernel_is_deterministic_and_covers_small_inputs():
    a = _run(8, 2, 128, torch.bfloat16, False, ctas=48)
    b = _run(8, 2, 128, torch.bfloat16, False, ctas=48)
    assert torch.equal(a[0], b[0]) and a[2] == b[2]
    assert torch.allclose(a[0].float(), a[1], rtol=8e-3, atol=8e-3)


def test_reduce_scatter_rejects_bad_arguments():
    from lm_engine_b200.ops import _lib

    lib = _lib.cuda_lib()
    x = torch.zeros(256, device="cuda", dtype=torch.bfloat16)
    srcs = (ctypes.c_void_p * 8)(x.data_ptr(), *([None] * 7))
    pads = (ctypes.c_void_p * 8)(*([None] * 8))
    assert lib.lme_reduce_scatter_peers(srcs, pads, None, 0, 9, 1, x.data_ptr(), 256, 1, 1.0, 0, None, 8, None) == -1
    assert lib.lme_reduce_scatter_peers(srcs, pads, None, 0, 1, 1, x.data_ptr(), 100, 1, 1.0, 0, None, 8, None) == -1
    assert lib.lme_reduce_scatter_peers(srcs, pads, None, 0, 1, 1, x.data_ptr() + 2, 256, 1, 1.0, 0, None, 8,
                                        None) == -2
