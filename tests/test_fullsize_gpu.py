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


def test_attention_at_full_stream_size_by_properties(dev):
    """the tree attention over a whole configuration-2 stream (27 648 tokens, 16 query / 8 KV heads of 256) through properties
    that need no oracle: with every value row of a KV head equal to one vector the output is that vector (the weights of a row sum
    to one, whatever the mask); the per-token output maxima match the stored output; and the first content's rows are bit-identical
    to the same content run alone"""
    from spinf_serve_b200 import attention as A
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.packer import Packer

    def batches(wl):
        pk = Packer(32768, 65536, True, 1024)
        return [b for key, first, t in wl.items for b in pk.push((key, first), t)] + list(pk.flush())

    (b,) = batches(workloads.config2(seed=0))
    (b1,) = batches(workloads.config2(seed=0, n_contents=1))
    n, H, Hkv, D = b.length, 16, 8, 256
    g = torch.Generator().manual_seed(0)
    q = torch.randn((n, H, D), generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    masks = A.stream_masks(b.art, b.end, b.pos, 1024, dev, always_window=True)
    for kind in ("full_attention", "sliding_attention"):
        const = torch.randn((1, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
        out = A.tree_attention(q, k, const.expand(n, Hkv, D).contiguous(), masks[kind], D**-0.5)
        want = const.repeat_interleave(H // Hkv, dim=1).expand(n, H, D)
        assert (out.float() - want.float()).abs().max() <= 2.0**-7 * want.float().abs().max()
        amax = torch.zeros(n, dtype=torch.float32, device=dev)
        full = A.tree_attention(q, k, v, masks[kind], D**-0.5, row_amax=amax)
        assert torch.equal(amax, full.float().abs().amax(dim=(1, 2)))
        m1 = A.stream_masks(b1.art, b1.end, b1.pos, 1024, dev, always_window=True)
        n1 = b1.length
        alone = A.tree_attention(q[:n1].contiguous(), k[:n1].contiguous(), v[:n1].contiguous(), m1[kind], D**-0.5)
        assert torch.equal(alone, full[:n1])
