"""A device-side wait on a flag that nothing sets runs out after its wall-clock limit, records a status word that the
host reads, and leaves the context usable (one thread waits for about two seconds; nothing faults or traps)."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_times_out_and_reports_status():
    from lm_engine_b200.ops import _lib

    lib = _lib.cuda_lib()
    _lib.read_status(clear=True)
    pad = torch.zeros(16, dtype=torch.int32, device="cuda")       # signal pad: sig[1] stays 0 forever
    torch.cuda.synchronize()
    t0 = time.time()
    _lib.check(lib.lme_gather_wait_peer(pad.data_ptr(), 1, 5, _lib.stream_ptr()), "lme_gather_wait_peer")
    torch.cuda.synchronize()
    waited = time.time() - t0
    status = _lib.read_status(clear=True)
    assert 1.5 < waited < 10, waited
    assert status[0] == 2                                          # STATUS_FLAG_TIMEOUT
    assert status[1] == 861                                        # which wait: peer signal of source rank 1
    # the context is intact: a satisfied wait returns at once and normal work runs
    pad[1] = 7
    _lib.check(lib.lme_gather_wait_peer(pad.data_ptr(), 1, 5, _lib.stream_ptr()), "lme_gather_wait_peer")
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0
    assert _lib.read_status(clear=True)[0] == 0
