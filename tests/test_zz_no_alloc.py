"""The allocation-free option log-prob entry point (spinf_option_logprobs_static) against the workspace-taking one, through the C
ABI. It exists for callers that cannot allocate device memory when they call: a server whose own allocator holds all of HBM, a
binding from a host language without a device allocator, or a latency path where cudaMalloc's device-wide synchronisation is
unwelcome. Its scratch is a fixed array inside the library that every call shares and that keeps the previous call's contents, so
the check runs two calls in a row with different shapes: stale partials from the first must not leak into the second.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(R, hidden, vocab, n_cols, seed, dev):
    g = torch.Generator().manual_seed(seed)
    h = (torch.randn((R, hidden), generator=g) * 1.5).to(torch.bfloat16).to(dev)
    W = (torch.randn((vocab, hidden), generator=g) * 0.05).to(torch.bfloat16).to(dev)
    cols = np.sort(np.random.default_rng(seed).choice(vocab, size=n_cols, replace=False)).astype(np.int32)
    return h, W, torch.from_numpy(cols).to(dev)


def _static(h, W, cols, softcap, status):
    from spinf_serve_b200 import _lib

    out = torch.empty((h.shape[0], cols.numel()), dtype=torch.float32, device=h.device)
    rc = _lib.lib().spinf_option_logprobs_static(
        _lib.ptr(h), _lib.ptr(W), h.shape[0], h.shape[1], W.shape[0], _lib.ptr(cols), cols.numel(), ctypes.c_float(softcap or 0.0),
        _lib.ptr(out), _lib.ptr(status), _lib.stream_ptr(),
    )
    return rc, out


def test_static_scratch_variant_matches_on_two_calls_in_a_row(dev):
    from spinf_serve_b200 import ops

    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # first call: many rows and a wide vocabulary fill a large part of the shared scratch
    h1, W1, c1 = _case(700, 512, 50000, 33, 31, dev)
    rc1, got1 = _static(h1, W1, c1, None, status)
    # second call, straight after on the same stream: fewer rows, smaller vocabulary, soft-capping on
    h2, W2, c2 = _case(130, 1024, 9000, 7, 32, dev)
    rc2, got2 = _static(h2, W2, c2, 30.0, status)
    assert rc1 == 0 and rc2 == 0
    want1 = ops.option_logprobs(h1, W1, c1, None)
    want2 = ops.option_logprobs(h2, W2, c2, 30.0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # same kernels in the same order: the results agree to well within the 2e-3 the other log-prob tests allow; in fact bit for bit
    assert float((got1 - want1).abs().max()) <= 2e-3 and float((got2 - want2).abs().max()) <= 2e-3
    assert torch.equal(got1, want1) and torch.equal(got2, want2)


def test_static_scratch_variant_rejects_oversize_calls(dev):
    """beyond the fixed array the call is refused on the host with SPINF_ERR_TOO_LARGE (-4) and launches nothing"""
    h, W, c = _case(8, 64, 512, 2, 33, dev)
    from spinf_serve_b200 import _lib

    out = torch.full((4096, 2), 7.0, dtype=torch.float32, device=dev)
    rc = _lib.lib().spinf_option_logprobs_static(
        _lib.ptr(h), _lib.ptr(W), 4096, 64, 262144, _lib.ptr(c), 2, ctypes.c_float(0.0), _lib.ptr(out), None, _lib.stream_ptr()
    )
    torch.cuda.synchronize()
    assert rc == -4 and bool((out == 7.0).all())


def test_static_scratch_variant_allocates_nothing_and_works_without_a_status_pointer(dev):
    """after a first call has resolved the array's address, a call moves neither the driver's free-memory figure nor torch's
    allocation count (the output is allocated before the window); with status NULL the status word sits in the array's first bytes
    and the result is the same"""
    from spinf_serve_b200 import _lib, ops

    h, W, c = _case(200, 512, 20000, 5, 34, dev)
    want = ops.option_logprobs(h, W, c, None)
    _static(h, W, c, None, None)  # first call on the device done
    out = torch.empty((h.shape[0], c.numel()), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info(dev)[0]
    allocs0 = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
    rc = _lib.lib().spinf_option_logprobs_static(
        _lib.ptr(h), _lib.ptr(W), h.shape[0], h.shape[1], W.shape[0], _lib.ptr(c), c.numel(), ctypes.c_float(0.0), _lib.ptr(out), None,
        _lib.stream_ptr(),
    )
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.cuda.mem_get_info(dev)[0] == free0 and torch.cuda.memory_stats(dev)["allocation.all.allocated"] == allocs0
    assert torch.equal(out, want)
