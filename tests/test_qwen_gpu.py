"""GPU parity of the Qwen-style hybrid stack (Gated DeltaNet + gated attention layers, int4 weight-only linears) with the oracle
restated from the reference's model code (spinf_serve/models/qwen35/qwen.py:502-775), and batch invariance of its scores."""

import numpy as np
import pytest
import torch

from oracle import qwen as OQ
from spinf_serve_b200 import packer as P
from spinf_serve_b200.scorer import forward_one
from spinf_serve_b200.gdn_plan import tree_plan

pytestmark = pytest.mark.gpu

SMALL = dict(layers=4, hidden=256, ffn=512, vocab=2048, hk=2, hv=4, dk=128, dv=128, heads=4, kv_heads=2, head_dim=128, rotary=32,
             group=128, every=2)


def _content(rng, n_trunk, n_q, vocab=2048):
    trunk = rng.integers(5, vocab, n_trunk).tolist()
    prompts = [trunk + [10 + i] + rng.integers(5, vocab, int(rng.integers(3, 14))).tolist() for i in range(n_q)]
    return P.build_grouped_tree(prompts, [P.ReadPlan.build([[7], [8], [9, 11]]) for _ in prompts])


def _build(dev, layers=4):
    from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights

    ocfg = OQ.QwenConfig(**{**SMALL, "layers": layers})
    W = OQ.init_weights(ocfg, seed=3)
    stack = QwenStack(QwenWeights(QwenConfig(**{**SMALL, "layers": layers}), W, dev))
    return ocfg, W, stack


def test_hybrid_forward_vs_oracle(dev):
    ocfg, W, stack = _build(dev)
    rng = np.random.default_rng(2)
    pk = P.Packer(2048, 8192, align=True)
    for j in range(3):
        list(pk.push(j, _content(rng, int(rng.integers(30, 200)), 4)))
    (b,) = list(pk.flush())
    real = torch.from_numpy(b.art >= 0)
    taps_o, taps_g = {}, {}
    ref = OQ.forward(ocfg, W, b.ids, b.art, b.end, b.pos, tree_plan(b.prev, b.art >= 0, "cpu"), taps=taps_o)
    out = forward_one(stack, b, dev, taps=taps_g)[0].cpu()
    for i in range(ocfg.layers):
        o = taps_o[i][real].float()
        err = ((taps_g[i].cpu()[real].float() - o).pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()
        print(f"residual stream after layer {i} ({ocfg.layer_types[i]}): rms err / rms = {err:.3e}")
        assert err < 2e-2  # bf16 activations, no re-quantisation: differences stay at the bf16 rounding level
    o = ref[real].float()
    err = ((out[real].float() - o).pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()
    print(f"final hidden: rms err / rms = {err:.3e}")
    assert err < 2e-2


def test_hybrid_scores_bit_identical_alone_and_packed(dev):
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    _, _, stack = _build(dev)
    rng = np.random.default_rng(5)
    target = (("T",), 0, _content(rng, 211, 5))
    others = [((f"c{j}",), 0, _content(rng, int(rng.integers(30, 400)), int(rng.integers(1, 6)))) for j in range(8)]
    sc = Scorer(stack, EngineConfig(token_budget=8192, max_tokens=8192), dev)
    runs = [[target], [target] + others[:3], others[:3] + [target], others[:4] + [target] + others[4:]]
    res = [sc.score_grouped(r)[("T",)] for r in runs]
    for r in res[1:]:
        for a, b in zip(r, res[0]):
            assert np.array_equal(a, b)
    assert all(np.isfinite(a).all() and (a < 0).all() for a in res[0])


def test_compact_rows_equal_the_stream_layout(dev):
    """the model on compact rows (real tokens only, the stream layout rebuilt around the attention; Qwen35Stack.compact_rows,
    qwen.py:1039-1048) gives bit-identical hidden states at every real position, for the whole stream and for selected read rows"""
    from spinf_serve_b200.qwen_stack import QwenStack

    _, _, stack = _build(dev)
    plain = QwenStack(stack.w, compact=False)
    rng = np.random.default_rng(9)
    pk = P.Packer(4096, 8192, align=True)
    for j in range(4):
        list(pk.push(j, _content(rng, int(rng.integers(30, 300)), 3)))
    (b,) = list(pk.flush())
    real = torch.from_numpy(b.art >= 0).to(dev)
    assert stack.compact_rows(b) < b.length  # aligned jobs leave pads that the compact layout drops
    a = forward_one(stack, b, dev)[0]
    c = forward_one(plain, b, dev)[0]
    assert a.shape == c.shape and torch.equal(a[real], c[real])
    sel = torch.from_numpy(b.sel).to(dev)
    assert torch.equal(forward_one(stack, b, dev, rows=sel), c.index_select(0, sel))


def test_hybrid_scores_against_the_oracle(dev):
    """int4 weights with bf16 activations through the public scorer: no re-quantisation between the layers; the option log-probs
    of the 4-layer hybrid stack against the oracle, next to the oracle's own sensitivity to one legitimate rounding change"""
    from oracle import attention as OA
    from oracle import head as OH
    from spinf_serve_b200 import parity, reads
    from spinf_serve_b200.scorer import EngineConfig, Scorer, read_grouped

    ocfg, W, stack = _build(dev)
    rng = np.random.default_rng(12)
    items = [((f"c{j}",), 0, _content(rng, int(rng.integers(30, 300)), int(rng.integers(2, 6)))) for j in range(5)]
    sc = Scorer(stack, EngineConfig(token_budget=2048, max_tokens=8192), dev)
    got = sc.score_grouped(items)
    pk = P.Packer(2048, 8192, True, 1024)
    batches = [b for key, first, t in items for b in pk.push((key, first), t)] + list(pk.flush())

    def oracle_scores():
        want = {key: [None] * len(t.plans) for key, _, t in items}
        for b in batches:
            cols = Scorer._cols(b)
            hf = OQ.forward(ocfg, W, b.ids, b.art, b.end, b.pos, tree_plan(b.prev, b.art >= 0, "cpu"))
            lp = OH.option_logprobs(hf[torch.as_tensor(b.sel, dtype=torch.int64)], W["lm_head"], cols, None)
            read_grouped(lp.numpy(), cols, b, want)
        return want

    want = oracle_scores()
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        pert = oracle_scores()
    finally:
        OA.tree_attention = exact
    m, floor = parity.compare(want, got), parity.compare(want, pert)
    dp = np.concatenate([np.abs(reads.option_probs(g)[1] - reads.option_probs(w)[1]) for k in want for g, w in zip(got[k], want[k])])
    print(f"int4 hybrid, 4 layers, library vs oracle: {m}; p max abs {dp.max():.3e}, mean {dp.mean():.3e}")
    print(f"int4 hybrid, 4 layers, oracle vs itself with P rounded to bf16: {floor}")
    assert m["lp_mean_abs"] < 3 * floor["lp_mean_abs"] + 5e-3 and m["lp_max_abs"] < 3 * floor["lp_max_abs"] + 5e-2
    assert m["raw_sign_agree"] > 0.95 and m["raw_corr"] > 0.995
