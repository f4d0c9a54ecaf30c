"""ctypes binding of ``liblme_cuda.so`` / ``liblme_host.so``.

The CUDA library exposes a C ABI (raw device pointers + ``cudaStream_t``); there is no pybind / torch-extension layer,
which keeps the build to one nvcc invocation of a few seconds and lets non-Python callers link the same symbols.
On a machine with a GPU a missing library is an error (no silent fallback to eager PyTorch); on a CPU-only machine
the wrappers in :mod:`lm_engine_b200.ops` route to their PyTorch reference implementations instead.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C")
_cuda_lib: ctypes.CDLL | None = None
_host_lib: ctypes.CDLL | None = None

LME_OK = 0
_ERRORS = {
    -1: "unsupported shape",
    -2: "misaligned pointer",
    -3: "tensor map encode failed",
    -4: "kernel launch failed",
    -5: "driver entry point unavailable",
    -6: "size beyond the entry point's maximum",
}

GEMM_OUT_F32 = 1
GEMM_ACCUMULATE = 2
GEMM_SWIGLU = 4
SUMSQ_MAX_PARTIALS = 1184


class LMEKernelError(RuntimeError):
    pass


def _load(name: str, builder: str) -> ctypes.CDLL:
    path = os.path.join(_DIR, name)
    if not os.path.exists(path):
        from .. import build as _build

        getattr(_build, builder)()
    if not os.path.exists(path):
        raise LMEKernelError(f"{path} is missing and could not be built")
    return ctypes.CDLL(path)


def cuda_lib() -> ctypes.CDLL:
    global _cuda_lib
    if _cuda_lib is None:
        lib = _load("liblme_cuda.so", "build_cuda")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        sigs = {
            "lme_gemm_bf16": [P, I, L, P, I, L, P, L, I, I, I, I, P, P, L, P, L, I, P],
            "lme_gemm_fp8": [P, I, L, P, I, L, P, P, P, L, I, I, I, I, P, P, L, P, L, I, P],
            "lme_gemm_bf16_allgather_a": [P, L, P, I, L, P, L, I, I, I, I, P, P, L, P, L, P, P, P, P, P, L, I, I, I, I, I, I, P],
            "lme_gather_signal": [P, I, I, I, P],
            "lme_gather_wait_peer": [P, I, I, P],
            "lme_stream_write_words": [P, I, I, P],
            "lme_stream_wait_word": [P, I, P],
            "lme_gemm_bf16_reduce_scatter": [P, L, P, I, L, P, L, I, I, I, P, P, L, P, P, I, I, I, I, P],
            "lme_gemm_bf16_grouped": [P, L, P, I, L, P, L, I, I, I, I, I, P, L, P, I, P],
            "lme_gemm_bf16_grouped_wgrad": [P, L, P, L, P, L, I, I, I, I, P, P, I, I, P],
            "lme_moe_scatter_rows": [P, P, P, P, I, I, I, P],
            "lme_moe_gather_reduce": [P, P, P, P, I, I, I, P],
            "lme_moe_row_dots": [P, P, P, P, I, I, I, P],
            "lme_moe_topk_softmax_fwd": [P, I, I, I, I, P, P, P, P],
            "lme_moe_topk_softmax_bwd": [P, P, P, P, I, I, I, I, P, P],
            "lme_moe_route_chunks": [I],
            "lme_ep_flag_words": [],
            "lme_ep_publish_counts": [P, P, P, I, I, I, I, P],
            "lme_ep_bases": [P, P, I, I, I, I, I, P, P, P, P, P, P],
            "lme_ep_dest": [P, P, P, P, I, I, I, I, P, P],
            "lme_ep_offer_rows": [P, P, P, I, P, I, I, I, P],
            "lme_ep_land_rows": [P, P, P, P, I, I, I, I, I, P],
            "lme_ep_wait": [P, I, I, I, P],
            "lme_ep_signal_done": [P, I, I, I, P],
            "lme_ep_pull_rows": [P, P, P, I, I, I, I, I, P],
            "lme_moe_route_layout": [P, I, I, P, P, P, P, P, I, P, P],
            "lme_delta_chain_fwd": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P],
            "lme_delta_chain_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, P],
            "lme_causal_conv1d_fwd": [P, P, P, P, P, I, I, I, I, I, P],
            "lme_causal_conv1d_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
            "lme_reduce_slices": [P, I, P, L, I, F, I, P],
            "lme_reduce_scatter_peers": [P, P, P, I, I, I, P, L, I, F, I, P, I, P],
            "lme_sum_partials": [P, I, P, I, P],
            "lme_set_peer_wait_limit_ms": [L],
            "lme_ssd_decay_matrix": [P, P, P, L, I, I, I, P],
            "lme_ssd_dcb": [P, P, P, L, I, I, I, P],
            "lme_ssd_prep": [P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, P],
            "lme_ssd_combine": [P, P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, I, P],
            "lme_ssd_boundary_fwd": [P, P, P, P, P, P, I, I, I, I, P],
            "lme_ssd_boundary_bwd": [P, P, P, P, P, P, P, I, I, I, I, P],
            "lme_gemm_bf16_batched": [P, I, L, L, P, I, L, L, P, L, L, I, I, I, I, I, I, P],
            "lme_m2rnn": [P, I, P],
            "lme_rnn": [P, I, P],
            "lme_attention_fwd": [P, L, P, L, P, L, P, L, P, I, I, I, I, I, I, I, F, P, L, P, I, I, P],
            "lme_attention_bwd": [P, L, P, L, P, L, P, L, P, L, P, P, P, L, P, L, P, L, I, I, I, I, I, I, I, F, P, L, P],
            "lme_embedding_fwd": [P, P, P, L, I, L, L, P],
            "lme_embedding_bwd": [P, P, P, P, L, I, L, L, P],
            "lme_pack_rows": [P, P, P, I, I, L, L, P],
            "lme_unpack_rows": [P, P, P, I, I, L, P],
            "lme_fp8_amax": [P, L, P, P],
            "lme_fp8_quantize": [P, I, I, L, P, I, P, L, P, L, P, P],
            "lme_read_status": [P, I],
            "lme_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
            "lme_rmsnorm_bwd_partial_rows": [I],
            "lme_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
            "lme_swiglu_fwd": [P, P, L, L, P],
            "lme_swiglu_bwd": [P, P, P, L, L, P],
            "lme_swiglu_bwd_tiles": [P, P, P, L, L, P, P],
            "lme_qkv_rope": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
            "lme_ce_stats": [P, L, P, P, P, P, I, I, I, P],
            "lme_ce_grad": [P, L, P, P, I, I, I, F, P, L, P],
            "lme_adamw": [P, P, P, P, I, P, L, F, F, F, F, F, I, P, P],
            "lme_sumsq": [P, I, L, P, P, I, P],
            "lme_clip_coef": [P, F, P, P, P],
        }
        for fn, args in sigs.items():
            f = getattr(lib, fn)
            f.argtypes = args
            f.restype = c_int
        _cuda_lib = lib
    return _cuda_lib


def host_lib() -> ctypes.CDLL:
    global _host_lib
    if _host_lib is None:
        _host_lib = _load("liblme_host.so", "build_host")
    return _host_lib


def have_cuda_kernels() -> bool:
    """True when the hand-written kernels are the compute path (a CUDA device is present)."""
    return torch.cuda.is_available()


def check(rc: int, what: str) -> None:
    if rc != LME_OK:
        raise LMEKernelError(f"{what}: {_ERRORS.get(rc, rc)}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def raise_peer_wait_limit() -> None:
    """Cross-GPU waits inside kernels (flags that another rank writes) get ``LME_PEER_WAIT_MS`` (default 60 s)
    instead of the 2 s of waits that only this GPU's work feeds: ranks drift apart by seconds around first-step
    allocations, lazy communicator set-up, evaluation and checkpoints.  Called by everything that sets up such waits."""
    import os

    check(cuda_lib().lme_set_peer_wait_limit_ms(int(os.environ.get("LME_PEER_WAIT_MS", "60000"))),
          "lme_set_peer_wait_limit_ms")


def read_status(clear: bool = True) -> list[int]:
    """Synchronises and returns the 8-word device status block (word 0 != 0: a bounded wait expired)."""
    buf = (ctypes.c_uint * 8)()
    check(cuda_lib().lme_read_status(buf, int(clear)), "lme_read_status")
    return list(buf)


# number of kernels of this library launched since import (the bench reports it)
launch_count = 0


def count_launch(n: int = 1) -> None:
    global launch_count
    launch_count += n
