"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some hosts of this library are not allowed to allocate device memory at call time (their process reserved the whole
GPU up front, or an allocation's synchronisation is unacceptable where they call from).  For them
``lme_rmsnorm_bwd_static_scratch`` keeps its workspace in a fixed array inside the shared object.  The test drives it
with raw pointers exactly like a C caller would and checks it against the regular entry point, whose workspace the
caller passes in - twice in a row with different shapes, because the built-in workspace is shared by all calls and
still holds the previous call's contents.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_PARTIAL_ROWS = 444                      # LME_RMSNORM_BWD_MAX_PARTIAL_ROWS
STATIC_SCRATCH_FLOATS = MAX_PARTIAL_ROWS * 4096
ERR_TOO_LARGE = -6


def _symbols():
    from lm_engine_b200.ops import _lib

    lib = _lib.cuda_lib()
    P, I = ctypes.c_void_p, ctypes.c_int
    fn = lib.lme_rmsnorm_bwd_static_scratch
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    fn.restype = I
    return lib, fn


def _problem(T, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)  # noqa: E731
    dy, h, dres = mk(T, H), mk(T, H), mk(T, H)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5).contiguous()
    return dy, h, w, rstd, dres


def _run_pair(T, H, seed):
    lib, static_fn = _symbols()
    dy, h, w, rstd, dres = _problem(T, H, seed)
    stream = torch.cuda.current_stream().cuda_stream
    # regular entry point: the caller owns the scratch
    rows = lib.lme_rmsnorm_bwd_partial_rows(T)
    scratch = torch.empty(rows, H, device="cuda", dtype=torch.float32)
    dx_ref = torch.empty_like(h)
    dw_ref = torch.empty(H, device="cuda", dtype=torch.float32)
    rc = lib.lme_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                             dx_ref.data_ptr(), scratch.data_ptr(), dw_ref.data_ptr(), 0, T, H, stream)
    assert rc == 0
    # allocation-free entry point: no scratch argument
    dx = torch.empty_like(h)
    dw = torch.empty(H, device="cuda", dtype=torch.float32)
    rc = static_fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(),
                   dw.data_ptr(), 0, T, H, stream)
    assert rc == 0
    torch.cuda.synchronize()
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()  # noqa: E731
    assert rel(dx, dx_ref) < 1e-2
    assert rel(dw, dw_ref) < 1e-2
    # and both agree with a plain fp32 PyTorch statement of the op
    hf = h.float().requires_grad_()
    wf = w.float().requires_grad_()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    y.backward(dy.float())
    assert rel(dx, hf.grad + dres.float()) < 1e-2
    assert rel(dw, wf.grad) < 1e-2


def test_two_calls_in_a_row_match_the_regular_entry_point():
    _run_pair(T=1000, H=4096, seed=1)   # 444 partial rows x 4096: uses the built-in workspace to the last float
    _run_pair(T=37, H=1024, seed=2)     # smaller problem right after: stale workspace contents must not leak


def test_accepts_up_to_the_capacity_and_rejects_beyond_it():
    lib, static_fn = _symbols()
    assert lib.lme_rmsnorm_bwd_partial_rows(10**6) == MAX_PARTIAL_ROWS
    _run_pair(T=222, H=8192, seed=3)    # a wider row with fewer rows: 222 * 8192 == 444 * 4096, still accepted
    z = torch.zeros(8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for T, H in ((444, 4104), (4096, 8192), (223, 8192)):      # one vector, twice, one row beyond the capacity
        assert lib.lme_rmsnorm_bwd_partial_rows(T) * H > STATIC_SCRATCH_FLOATS
        rc = static_fn(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, z.data_ptr(), z.data_ptr(), 0,
                       T, H, stream)
        assert rc == ERR_TOO_LARGE      # refused before anything is launched
