"""Size-independent properties at the BASELINE configurations' full layer shapes and stream sizes (depth reduced to keep the test
short): a content scores bit-identically alone and inside a 32 768-token bulk pass whose trunks run past the sliding window, on the
12B shapes (head_dim 256) and the 31B-class shapes (head_dim 128); every option log-prob is a log-probability."""

import numpy as np
import pytest
import torch

from oracle import head as OH

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,layers", [("gemma12b", 2), ("gemma31b", 1)])
def test_bulk_pass_at_full_width_is_batch_invariant(dev, name, layers):
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.gemma_stack import CONFIGS, GemmaConfig, GemmaStack, GemmaWeights
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    cfg = GemmaConfig(**{**CONFIGS[name], "layers": layers, "pattern": 2})  # one sliding and one full layer on the 12B shapes
    stack = GemmaStack(GemmaWeights.random(cfg, seed=1, device=dev))
    wl = workloads.config3(seed=0, n_contents=20)  # trunks 200-2000 tokens, 56 questions, 2-5 options: ~1.2 passes of 32 768
    sc = Scorer(stack, EngineConfig(token_budget=32768, max_tokens=65536), dev)
    bulk = sc.score_grouped(wl.items)
    assert sc.stats.forwards >= 2 and sc.stats.tokens == wl.n_tokens
    for key, _, tree in (wl.items[0], wl.items[7], wl.items[-1]):
        alone = sc.score_grouped([(key, 0, tree)])[key]
        assert len(alone) == 56
        for a, b in zip(alone, bulk[key]):
            assert np.array_equal(a, b)
    n_q = 0
    for key, _, tree in wl.items:
        for lp in bulk[key]:
            n_q += 1
            assert np.isfinite(lp).all() and (lp <= 0).all()
            p, residual = OH.read_probs(lp)
            assert abs(p.sum() - 1) < 1e-9 and 0.0 <= residual <= 1.0
    assert n_q == wl.n_questions
    del stack, sc
    torch.cuda.empty_cache()
