"""GPU parity of the fused option-log-prob read against the oracle of Scorer._logprobs + column gather
(spinf_serve/scorer.py:340-355, :254)."""

import numpy as np
import pytest
import torch

from oracle import head as OH

pytestmark = pytest.mark.gpu


def _case(R, hidden, vocab, n_cols, seed):
    g = torch.Generator().manual_seed(seed)
    h = (torch.randn((R, hidden), generator=g) * 1.5).to(torch.bfloat16)
    W = (torch.randn((vocab, hidden), generator=g) * 0.05).to(torch.bfloat16)
    cols = np.sort(np.random.default_rng(seed).choice(vocab, size=n_cols, replace=False)).astype(np.int32)
    return h, W, cols


@pytest.mark.parametrize("R,hidden,vocab,n_cols,softcap", [(16, 256, 1024, 4, None), (130, 3840, 8192, 37, None), (300, 1024, 20000, 5, 30.0), (1, 512, 4096, 1, None)])
def test_option_logprobs_vs_oracle(dev, R, hidden, vocab, n_cols, softcap):
    from spinf_serve_b200 import ops

    h, W, cols = _case(R, hidden, vocab, n_cols, 11)
    cols[0] = 0
    cols[-1] = max(cols[-1], vocab - 1) if n_cols > 1 else cols[-1]  # first and last vocabulary ids
    cols = np.unique(cols).astype(np.int32)
    out = ops.option_logprobs(h.to(dev), W.to(dev), torch.from_numpy(cols).to(dev), softcap).cpu()
    ref = OH.option_logprobs(h, W, cols, softcap)
    err = (out - ref).abs().max().item()
    print(f"option logprobs R={R} vocab={vocab}: max abs err {err:.3e}")
    assert err < 2e-3  # the tolerance the benchmark specification states for option log-probs


def test_option_logprobs_rows_do_not_depend_on_R(dev):
    from spinf_serve_b200 import ops

    h, W, cols = _case(400, 1024, 16384, 9, 12)
    h, W, c = h.to(dev), W.to(dev), torch.from_numpy(cols).to(dev)
    full = ops.option_logprobs(h, W, c)
    for R in (1, 127, 129):
        assert torch.equal(ops.option_logprobs(h[:R].contiguous(), W, c), full[:R])
