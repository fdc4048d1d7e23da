"""The error path of the kernels' bounded waits, end to end on the GPU without a fault or a hang: a wait that nothing satisfies gives
up at its limit, the kernel returns, the host reads the status, and the library keeps working."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(dev):
    from spinf_serve_b200 import _lib, ops
    from spinf_serve_b200._lib import SpinfError

    _lib.init(dev)
    assert _lib.last_status(False) == 0
    t0 = time.perf_counter()
    _lib.check(_lib.lib().spinf_selftest_bounded_wait(50_000_000, _lib.stream_ptr()), "spinf_selftest_bounded_wait")  # 50 ms
    with pytest.raises(SpinfError, match="device status 4"):
        _lib.last_status()  # synchronises: the kernel has returned by itself
    waited = time.perf_counter() - t0
    assert 0.04 < waited < 1.0, waited
    assert _lib.last_status(False) == 0  # read once, cleared
    # the context is intact: an ordinary operator runs and leaves a clean status
    x = torch.randn((64, 256), device=dev).to(torch.bfloat16)
    x8, xs = ops.fp8_rowwise_quant(x)
    assert torch.isfinite(xs).all() and _lib.last_status(False) == 0
    # argument errors are host-side
    assert _lib.lib().spinf_selftest_bounded_wait(0, _lib.stream_ptr()) == -1
    assert _lib.lib().spinf_selftest_bounded_wait(2_000_000_000, _lib.stream_ptr()) == -1
