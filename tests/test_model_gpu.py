"""GPU parity of the packed forward and the scorer against the model-level oracle (oracle.gemma, itself pinned to the
transformers layer code the reference runs), and batch invariance of the scores end to end."""

import numpy as np
import pytest
import torch

from oracle import attention as OA
from oracle import gemma as OG
from spinf_serve_b200 import packer as P
from spinf_serve_b200.scorer import forward_one

pytestmark = pytest.mark.gpu


def _cfg(D=128, layers=4):
    return dict(layers=layers, hidden=512, heads=4, kv_heads=2, head_dim=D, ffn=1024, vocab=4096, window=64, pattern=2)


def _content(rng, n_trunk, n_q, vocab=4096):
    trunk = rng.integers(5, vocab, n_trunk).tolist()
    prompts = [trunk + [10 + i] + rng.integers(5, vocab, int(rng.integers(3, 14))).tolist() for i in range(n_q)]
    plans = [P.ReadPlan.build([[7], [8], [9, 11]]) for _ in prompts]
    return P.build_grouped_tree(prompts, plans)


def _build(dev, D, layers):
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights

    ocfg = OG.GemmaConfig(**_cfg(D, layers))
    W = OG.init_weights(ocfg, seed=2)
    Q = OG.quantize(W)
    # the same quantized weights on both sides: CUDA's load-time quantiser differs from the CPU's in the last bit of the scale
    # (division by a scalar becomes a reciprocal multiply), which would move a few weights by one fp8 step
    stack = GemmaStack(GemmaWeights.from_quantized(GemmaConfig(**_cfg(D, layers)), W, Q, dev))
    return ocfg, W, Q, stack


@pytest.mark.parametrize("D", [128, 256])
def test_forward_vs_oracle_layer_by_layer(dev, D):
    ocfg, W, Q, stack = _build(dev, D, 3)
    rng = np.random.default_rng(1)
    pk = P.Packer(2048, 8192, align=True)
    for j in range(3):
        list(pk.push(j, _content(rng, int(rng.integers(40, 300)), 4)))
    (b,) = list(pk.flush())
    taps_o, taps_g = {}, {}
    ref = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_o)
    out = forward_one(stack, b, dev, taps=taps_g)[0].cpu()
    real = torch.from_numpy(b.art >= 0)
    # layer 0 inputs are identical, so q / k / v (projection, head norm, rotary) agree up to rare last-bit flips
    for key in ("q", "k", "v"):
        g, o = taps_g[0][key].cpu()[real].float(), taps_o[0][key][real].float()
        frac = (g != o).float().mean().item()
        print(f"D={D} layer0 {key}: differing elements {frac:.4%}, max abs {(g - o).abs().max():.3e}")
        assert frac < 0.01 and (g - o).abs().max() <= 2.0**-6 * o.abs().max()
    # Beyond the first quantiser the comparison is statistical: per-token fp8 re-quantisation turns one-ulp bf16 differences into
    # 6 % steps, so two correct implementations drift apart layer by layer. The yardstick is the oracle against itself with a
    # single legitimate rounding change (P rounded to bf16 before P V, as the kernels and the reference's attention do).
    taps_p = {}
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_p)
    finally:
        OA.tree_attention = exact
    for i in range(3):
        o = taps_o[i]["h"][real].float()
        rms = lambda x: (x.pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()  # noqa: E731
        mine, floor = rms(taps_g[i]["h"].cpu()[real].float() - o), rms(taps_p[i]["h"][real].float() - o)
        print(f"D={D} hidden after layer {i}: rms err / rms = {mine:.3e} (oracle's own rounding sensitivity {floor:.3e})")
        assert mine < 3 * floor + 1e-3
    o = ref[real].float()
    mine = ((out[real].float() - o).pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()
    print(f"D={D} final hidden: rms err / rms = {mine:.3e}")
    assert mine < 0.5


def _items(rng, n):
    return [((f"c{j}",), 0, _content(rng, int(rng.integers(30, 500)), int(rng.integers(1, 7)))) for j in range(n)]


@pytest.mark.parametrize("layers", [0, 1, 2, 4])
def test_scorer_logprobs_vs_oracle(dev, layers):
    """option log-probs through the public scorer against the oracle. With no decoder layer (embedding, final norm, lm-head read)
    the 2e-3 absolute tolerance the benchmark specification states holds; with fp8 layers in between the error is bounded by a multiple of the
    oracle's own sensitivity to one legitimate rounding change (see test_forward_vs_oracle_layer_by_layer)"""
    from spinf_serve_b200.scorer import EngineConfig, Scorer, read_grouped

    ocfg, W, Q, stack = _build(dev, 128, layers)
    items = _items(np.random.default_rng(8), 6)
    sc = Scorer(stack, EngineConfig(token_budget=2048, max_tokens=8192), dev)
    got = sc.score_grouped(items)
    pk = P.Packer(2048, 8192, True, 1024)
    batches = [b for key, first, t in items for b in pk.push((key, first), t)] + list(pk.flush())

    def oracle_scores():
        want = {key: [None] * len(t.plans) for key, _, t in items}
        for b in batches:
            cols = Scorer._cols(b)
            read_grouped(OG.score(ocfg, W, Q, b, cols).numpy(), cols, b, want)
        return want

    want = oracle_scores()
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        pert = oracle_scores()
    finally:
        OA.tree_attention = exact

    def dist(x, y):
        d = np.concatenate([np.abs(g - w) for key in y for g, w in zip(x[key], y[key])])
        return float(d.max()), float(d.mean())

    (worst, mean), (fworst, fmean) = dist(got, want), dist(pert, want)
    print(f"{layers} layers: option log-prob max abs err {worst:.3e}, mean {mean:.3e}; oracle's own sensitivity max {fworst:.3e}, mean {fmean:.3e}")
    if layers == 0:
        assert worst < 2e-3
    else:
        assert mean < 3 * fmean + 2e-3 and worst < 3 * fworst + 2e-2
    assert sc.stats.forwards == len(batches) and sc.stats.tokens == sum(b.n_tokens for b in batches)


def test_scores_bit_identical_alone_and_packed(dev):
    """a content's option log-probs are bit-identical scored alone, packed first, packed last and among many others"""
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    _, _, _, stack = _build(dev, 256, 4)
    rng = np.random.default_rng(21)
    target = (("T",), 0, _content(rng, 333, 6))
    others = _items(rng, 14)
    sc = Scorer(stack, EngineConfig(token_budget=8192, max_tokens=8192), dev)
    runs = [[target], [target] + others[:4], others[:4] + [target], others[:7] + [target] + others[7:]]
    res = [sc.score_grouped(r)[("T",)] for r in runs]
    for r in res[1:]:
        for a, b in zip(r, res[0]):
            assert np.array_equal(a, b)


def test_per_tensor_schemes_vs_oracle(dev):
    """the reference's other two fp8 schemes on the same stack: calibration (dynamic scheme + largest inputs -> power-of-two scales)
    agrees with the oracle's, the static forward tracks the oracle's static forward like the row-wise one does, the monitor
    reports no clipping on the calibration data, and only the static scheme's scores are independent of a content's neighbours"""
    from spinf_serve_b200 import gemma_stack as GS
    from spinf_serve_b200 import linears
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    layers = 3
    ocfg = OG.GemmaConfig(**_cfg(128, layers))
    cfg = GS.GemmaConfig(**_cfg(128, layers))
    W = OG.init_weights(ocfg, seed=3)
    rng = np.random.default_rng(5)
    pk = P.Packer(2048, 8192, align=True)
    for j in range(3):
        list(pk.push(j, _content(rng, int(rng.integers(40, 300)), 4)))
    (b,) = list(pk.flush())
    real = torch.from_numpy(b.art >= 0)

    tab_o = OG.calibrate(ocfg, W, [b], 2.0)
    tab_g = GS.calibrate(cfg, W, [b], dev, 2.0)
    assert tab_g["scheme"] == "fp8s" and len(tab_g["scales"]) == layers
    for k in ("q", "k", "v"):  # layer 0's first inputs are the same tensor on both sides
        assert tab_g["amax"][0][k] == tab_o["amax"][0][k]
    same = [tab_g["scales"][i][k] == tab_o["scales"][i][k] for i in range(layers) for k in OG.LINEARS]
    ratio = [tab_g["amax"][i][k] / tab_o["amax"][i][k] for i in range(layers) for k in OG.LINEARS]
    print(f"calibration: {sum(same)} of {len(same)} scales equal; amax ratio {min(ratio):.3f}..{max(ratio):.3f}")
    # maxima are extreme values of activations that already differ by fp8 rounding noise; one beside a power of two may fall either side
    assert sum(same) >= len(same) - 2 and 0.8 < min(ratio) and max(ratio) < 1.25

    for scheme in ("fp8", "fp8s"):
        Q = OG.quantize(W, scheme)
        stack = GS.GemmaStack(GS.GemmaWeights.from_quantized(cfg, W, Q, dev, scheme, tab_o["scales"]))
        taps_o, taps_g, peaks_o = {}, {}, {}
        OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_o, scheme=scheme, scales=tab_o["scales"], peaks=peaks_o)
        linears.MONITOR["on"] = scheme == "fp8s"
        try:
            forward_one(stack, b, dev, taps=taps_g)[0]
        finally:
            linears.MONITOR["on"] = False
        for key in ("q", "k", "v"):
            g, o = taps_g[0][key].cpu()[real].float(), taps_o[0][key][real].float()
            frac = (g != o).float().mean().item()
            print(f"{scheme} layer0 {key}: differing elements {frac:.4%}")
            assert frac < 0.01 and (g - o).abs().max() <= 2.0**-6 * o.abs().max()
        # later layers: statistical, against the oracle's own sensitivity to one legitimate rounding change (P rounded to bf16
        # before P V), as in test_forward_vs_oracle_layer_by_layer; one scale per tensor makes the fp8 steps coarser than row-wise
        taps_p = {}
        exact = OA.tree_attention
        try:
            OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
            OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_p, scheme=scheme, scales=tab_o["scales"])
        finally:
            OA.tree_attention = exact
        for i in range(layers):
            o = taps_o[i]["h"][real].float()
            rms = lambda x: (x.pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()  # noqa: E731
            err, floor = rms(taps_g[i]["h"].cpu()[real].float() - o), rms(taps_p[i]["h"][real].float() - o)
            print(f"{scheme} hidden after layer {i}: rms err / rms = {err:.3e} (oracle's own rounding sensitivity {floor:.3e})")
            assert err < 3 * floor + 1e-3
        if scheme == "fp8s":
            pk_g = stack.peaks()
            assert pk_g[(0, "q")] == peaks_o[(0, "q")]  # the same input, the same scale
            assert 0.0 < max(pk_g.values()) <= 0.55  # headroom 2 over this very batch: nothing clips
            assert all(abs(pk_g[k] - v) <= 0.1 * v for k, v in peaks_o.items())

    # neighbours: static scores are the same bits alone and packed; the dynamic scheme's move with the stream's maximum
    target = (("T",), 0, _content(rng, 200, 5))
    others = _items(rng, 6)
    res = {}
    for scheme in ("fp8", "fp8s"):
        stack = GS.GemmaStack(GS.GemmaWeights.from_bf16(cfg, W, dev, scheme, tab_o["scales"]))
        sc = Scorer(stack, EngineConfig(token_budget=4096, max_tokens=8192), dev)
        res[scheme] = [sc.score_grouped(r)[("T",)] for r in ([target], others[:3] + [target] + others[3:])]
    assert all(np.array_equal(a, c) for a, c in zip(*res["fp8s"]))
    assert not all(np.array_equal(a, c) for a, c in zip(*res["fp8"]))

    # the sampled monitor through the scorer: nothing seen without it, a clipped input shows as a peak above 1
    tight = [{k: v / 16 for k, v in d.items()} for d in tab_o["scales"]]  # a table whose calibration did not cover these inputs
    stack = GS.GemmaStack(GS.GemmaWeights.from_bf16(cfg, W, dev, "fp8s", tight))
    assert Scorer(stack, EngineConfig(token_budget=4096, max_tokens=8192), dev).fp8s_peak() is None
    sc = Scorer(stack, EngineConfig(token_budget=4096, max_tokens=8192, fp8s_monitor_every=1), dev)
    sc.score_grouped([target])
    worst, where = sc.fp8s_peak()
    assert worst > 1.0 and where[1] in OG.LINEARS
    assert linears.MONITOR["on"]
    linears.MONITOR["on"] = False


@pytest.mark.parametrize("scheme", ["w8a8", "w8a16", "bf16"])
def test_int8_and_bf16_schemes_vs_oracle(dev, scheme):
    """the reference's remaining quant options on the same stack: forward against the oracle's (statistical beyond the first layer,
    as above) and scores bit-identical alone and packed (every one of these schemes is row-independent)"""
    from spinf_serve_b200 import gemma_stack as GS
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    layers = 3
    ocfg, cfg = OG.GemmaConfig(**_cfg(128, layers)), GS.GemmaConfig(**_cfg(128, layers))
    W = OG.init_weights(ocfg, seed=4)
    Q = OG.quantize(W, scheme)
    rng = np.random.default_rng(6)
    pk = P.Packer(2048, 8192, align=True)
    for j in range(3):
        list(pk.push(j, _content(rng, int(rng.integers(40, 300)), 4)))
    (b,) = list(pk.flush())
    real = torch.from_numpy(b.art >= 0)
    stack = GS.GemmaStack(GS.GemmaWeights.from_quantized(cfg, W, Q, dev, scheme))
    taps_o, taps_g, taps_p = {}, {}, {}
    OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_o, scheme=scheme)
    forward_one(stack, b, dev, taps=taps_g)[0]
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps_p, scheme=scheme)
    finally:
        OA.tree_attention = exact
    for key in ("q", "k", "v"):
        g, o = taps_g[0][key].cpu()[real].float(), taps_o[0][key][real].float()
        frac = (g != o).float().mean().item()
        print(f"{scheme} layer0 {key}: differing elements {frac:.4%}")
        assert frac < 0.02 and (g - o).abs().max() <= 2.0**-6 * o.abs().max()
    for i in range(layers):
        o = taps_o[i]["h"][real].float()
        rms = lambda x: (x.pow(2).mean().sqrt() / o.pow(2).mean().sqrt()).item()  # noqa: E731
        err, floor = rms(taps_g[i]["h"].cpu()[real].float() - o), rms(taps_p[i]["h"][real].float() - o)
        print(f"{scheme} hidden after layer {i}: rms err / rms = {err:.3e} (oracle's own rounding sensitivity {floor:.3e})")
        assert err < 3 * floor + 2e-3
    target = (("T",), 0, _content(rng, 200, 5))
    others = _items(rng, 6)
    sc = Scorer(GS.GemmaStack(GS.GemmaWeights.from_bf16(cfg, W, dev, scheme)), EngineConfig(token_budget=4096, max_tokens=8192), dev)
    alone, packed = (sc.score_grouped(r)[("T",)] for r in ([target], others[:3] + [target] + others[3:]))
    assert all(np.array_equal(a, c) for a, c in zip(alone, packed))


def _scores_and_oracle(dev, stack, ocfg, W, Q, items, scheme):
    from oracle import head as OH
    from spinf_serve_b200.scorer import EngineConfig, Scorer, read_grouped

    sc = Scorer(stack, EngineConfig(token_budget=2048, max_tokens=8192), dev)
    got = sc.score_grouped(items)
    pk = P.Packer(2048, 8192, True, 1024)
    want = {key: [None] * len(t.plans) for key, _, t in items}
    for b in [b for key, first, t in items for b in pk.push((key, first), t)] + list(pk.flush()):
        cols = Scorer._cols(b)
        hf = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, scheme=scheme)
        lp = OH.option_logprobs(hf[torch.as_tensor(b.sel, dtype=torch.int64)], W["embed"], cols, ocfg.softcap)
        read_grouped(lp.numpy(), cols, b, want)
    return got, want


@pytest.mark.parametrize("layers", [2, 4])
def test_bf16_scheme_scores_against_the_oracle(dev, layers):
    """the unquantised scheme through the public scorer: no fp8 re-quantisation amplifies anything, what is left is bf16 rounding
    of the activations in two different orders of operations. Measured against the oracle's own sensitivity to one legitimate
    rounding change (P rounded to bf16 before P V): at this model's logit scale that noise alone is several 1e-3 of a log-prob, so
    the benchmark's 2e-3 figure is asserted on top of it, not instead of it; ranking metrics must be intact"""
    from spinf_serve_b200 import gemma_stack as GS
    from spinf_serve_b200 import parity, reads

    ocfg, cfg = OG.GemmaConfig(**_cfg(128, layers)), GS.GemmaConfig(**_cfg(128, layers))
    W = OG.init_weights(ocfg, seed=5)
    Q = OG.quantize(W, "bf16")
    stack = GS.GemmaStack(GS.GemmaWeights.from_quantized(cfg, W, Q, dev, "bf16"))
    items = _items(np.random.default_rng(8), 6)
    got, want = _scores_and_oracle(dev, stack, ocfg, W, Q, items, "bf16")
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        _, pert = _scores_and_oracle(dev, stack, ocfg, W, Q, items, "bf16")
    finally:
        OA.tree_attention = exact
    m, floor = parity.compare(want, got), parity.compare(want, pert)
    dp = np.concatenate([np.abs(reads.option_probs(g)[1] - reads.option_probs(w)[1]) for k in want for g, w in zip(got[k], want[k])])
    print(f"bf16 scheme, {layers} layers, library vs oracle: {m}; p max abs {dp.max():.3e}, mean {dp.mean():.3e}")
    print(f"bf16 scheme, {layers} layers, oracle vs itself with P rounded to bf16: {floor}")
    assert m["lp_mean_abs"] < 3 * floor["lp_mean_abs"] + 2e-3 and m["lp_max_abs"] < 3 * floor["lp_max_abs"] + 2e-2
    assert m["raw_mean_abs"] < 3 * floor["raw_mean_abs"] + 2e-3 and m["raw_sign_agree"] >= floor["raw_sign_agree"] - 0.1
    assert m["raw_corr"] > 0.99 and dp.mean() < 2e-2


def test_fp8_rowwise_parity_metrics_at_depth(dev):
    """the benchmark's scheme through 48 layers of a narrow model: the reference's own parity metrics (log-prob and raw-score
    differences, correlation, sign agreement) between this library and the oracle, next to the oracle's sensitivity to one
    legitimate rounding change. Through fp8 layers these are statistical: on a trained 12B model the reference reports 0.12 mean
    raw difference and 97 % sign agreement between two compile variants of its own kernels"""
    from spinf_serve_b200 import gemma_stack as GS
    from spinf_serve_b200 import parity

    layers = 48
    ocfg, W, Q, stack = _build(dev, 128, layers)
    items = _items(np.random.default_rng(9), 4)
    got, want = _scores_and_oracle(dev, stack, ocfg, W, Q, items, "fp8row")
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        _, pert = _scores_and_oracle(dev, stack, ocfg, W, Q, items, "fp8row")
    finally:
        OA.tree_attention = exact
    mine, floor = parity.compare(want, got), parity.compare(want, pert)
    print(f"fp8 row-wise, {layers} layers, library vs oracle: {mine}")
    print(f"fp8 row-wise, {layers} layers, oracle vs itself with P rounded to bf16: {floor}")
    # a narrow random-weight model 48 layers deep is chaotic under fp8 re-quantisation: one rounding change inside the oracle moves
    # its own scores as far as the library is from it. What is asserted is that the library is no further than that.
    assert mine["lp_mean_abs"] < 2 * floor["lp_mean_abs"] + 2e-3 and mine["raw_mean_abs"] < 2 * floor["raw_mean_abs"] + 2e-3
    assert mine["raw_sign_agree"] >= floor["raw_sign_agree"] - 0.15
