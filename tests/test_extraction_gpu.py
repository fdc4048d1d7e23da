"""Extraction on the scoring pass, on the GPU: one Scorer.score_grouped call over trees that carry both scored prompts and
extraction branches (the reference's score_grouped with xbranches, spinf_serve/scorer.py:383-420,474-481,768-818) returns the
same option log-probs as without extraction and the same answers as the pieces run by hand (capture, decode.Decoder,
decode.search_text); small budgets cut the decoding into several chunks; both model families."""

import copy
import types

import numpy as np
import pytest
import torch

from spinf_serve_b200 import decode as D
from spinf_serve_b200 import packer as P
from spinf_serve_b200.scorer import EngineConfig, Scorer, forward_one

pytestmark = pytest.mark.gpu

STOP, BANNED, BEAM = [1, 2, 3], [0], 3
MIN_P = 1e-9  # random weights spread the probability thin: keep beams the production floor (0.002) would drop


def _scorer(stack, dev, **cfg):
    sc = Scorer(stack, EngineConfig(token_budget=4096, min_stream=1024, **cfg), dev, stop_ids=STOP, banned_ids=BANNED, beam=BEAM)
    sc.extractor.min_p = MIN_P
    return sc


def _mixed_trees(seed, spec, vocab):
    """spec: per tree (prefix length, scored questions, template lengths): scored prompts with option plans, then template
    branches whose answers are generated"""
    rng = np.random.default_rng(seed)
    trees = []
    for gi, (n_prefix, n_q, Ts) in enumerate(spec):
        prefix = rng.integers(5, vocab, n_prefix).tolist()
        prompts = [prefix + [40 + q] + rng.integers(5, vocab, int(rng.integers(3, 9))).tolist() for q in range(n_q)]
        t = P.build_grouped_tree(prompts, [P.ReadPlan.build([[7], [8], [9, 11]]) for _ in prompts]) if n_q else P.GroupedTree(prefix, [], [], [])
        for j, T in enumerate(Ts):
            t.branches.append([20 + j] + rng.integers(5, vocab, T - 1).tolist())
            if t.parents:
                t.parents.append(-1)
            t.xbranches.append((len(t.branches) - 1, types.SimpleNamespace(key=(gi, j), max_tokens=4)))
        trees.append(t)
    return trees


def _by_hand(stack, trees, cfg, dev, hybrid):
    """the same trees packed the same way, captured and decoded step by step outside the scorer"""
    pk = P.Packer(cfg.token_budget, cfg.max_tokens, cfg.align_jobs, cfg.min_stream)
    batches = [b for j, t in enumerate(trees) for b in pk.push((j, 0), t, cfg.pack_window)] + list(pk.flush())
    (b,) = batches
    with stack.capture(None, b, b.owners) as cap:
        hidden = forward_one(stack, b, dev)[0]
    groups = []
    for o in b.owners:
        g = D.Group(dict(cap["kv"][("p", id(o))]), o.prefix_len)
        if hybrid:
            g.extra = {"state": dict(cap["extra"]["state"][("p", id(o))]), "tmpl": []}
        for bs, bl, pr in o.xbranches:
            key = ("t", pr.key)
            g.prompts.append((pr, dict(cap["kv"].get(key, {})), bl, hidden[bs + bl - 1]))
            if hybrid:
                g.extra["tmpl"].append({"tok": cap["extra"]["tok"][key], "pre": cap["extra"]["pre"][key]})
        groups.append(g)
    dec = (D.HybridDecoder if hybrid else D.Decoder)(stack, groups, dev, beam=BEAM)
    return D.search_text(dec, stack.w.lm_weight, STOP, BANNED, min_p=MIN_P)


def _check_family(stack, trees, dev, hybrid):
    cfg = EngineConfig(token_budget=4096, min_stream=1024)
    sc = _scorer(stack, dev)
    out = sc.score_grouped([(j, 0, t) for j, t in enumerate(trees)])
    found = dict(sc.x_found)
    keys = {pr.key for t in trees for _, pr in t.xbranches}
    assert set(found) == keys and all(found[k] for k in keys)
    assert sc.extractor.chunks_run == 1 and sc.extractor._held == []

    # the option log-probs do not notice the extraction: the same stream scored by a scorer that generates nothing
    plain = copy.deepcopy(trees)
    for t in plain:
        t.xbranches = []
    ref = Scorer(stack, cfg, dev).score_grouped([(j, 0, t) for j, t in enumerate(plain)])
    assert set(out) == set(ref)
    for j in out:
        assert len(out[j]) == len(ref[j]) and all(np.array_equal(a, r) for a, r in zip(out[j], ref[j], strict=True))

    # the answers are those of the pieces run by hand
    hand = _by_hand(stack, trees, cfg, dev, hybrid)
    assert set(hand) == keys
    for k in keys:
        assert [t for t, _ in found[k]] == [t for t, _ in hand[k]], k
        assert np.allclose([lp for _, lp in found[k]], [lp for _, lp in hand[k]], atol=1e-6)
    print(f"{len(keys)} extraction prompts next to {sum(len(t.plans) for t in trees)} scored ones: best answers "
          + ", ".join(f"{k}: {found[k][0][0]} ({found[k][0][1]:.3f})" for k in sorted(keys)))

    # a decoder budget that holds one prompt's run at a time: several chunks, every prompt still answered
    per_tok = stack.kv_bytes_per_token()
    small = _scorer(stack, dev, decoder_budget_gib=1e-9)
    small.score_grouped([(j, 0, t) for j, t in enumerate(trees)])
    assert small.extractor.chunks_run == len(keys) and set(small.x_found) == keys and per_tok
    for k in keys:  # a chunk's padding changes the split of the prefix keys, hence the last bits: the best answer's score stays close
        assert abs(small.x_found[k][0][1] - found[k][0][1]) < 0.1, k

    # a hold budget below one group: every forward's captures are decoded at once, same answers as above
    eager = _scorer(stack, dev, decode_budget_gib=1e-9)
    eager.score_grouped([(j, 0, t) for j, t in enumerate(trees)])
    assert eager.extractor.chunks_run == len(trees) and set(eager.x_found) == keys


def test_scoring_and_extraction_in_one_call(dev):
    from oracle import gemma as OG
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights
    from tests.test_decode_gpu import _cfg

    W = OG.init_weights(OG.GemmaConfig(**_cfg()), seed=4)
    stack = GemmaStack(GemmaWeights.from_quantized(GemmaConfig(**_cfg()), W, OG.quantize(W, "fp8row"), dev))
    _check_family(stack, _mixed_trees(8, ((70, 3, (5, 9)), (130, 2, (7,)), (40, 0, (4, 6))), 4096), dev, hybrid=False)


def test_scoring_and_extraction_in_one_call_hybrid(dev):
    from oracle import qwen as OQ
    from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights
    from tests.test_qwen_gpu import SMALL

    W = OQ.init_weights(OQ.QwenConfig(**SMALL), seed=3)
    stack = QwenStack(QwenWeights(QwenConfig(**SMALL), W, dev))
    _check_family(stack, _mixed_trees(9, ((70, 3, (5, 9)), (130, 2, (7,))), 2048), dev, hybrid=True)


@pytest.mark.parametrize("family", ["gemma", "hybrid"])
def test_extract_jobs_with_and_without_template_tokens(dev, family):
    """Scorer.extract: a prompt whose slot starts right after the prefix decodes like the same prompt with the prefix's last
    token moved into its template"""
    from spinf_serve_b200.extraction import ExtractJob, ExtractPrompt

    if family == "gemma":
        from oracle import gemma as OG
        from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights
        from tests.test_decode_gpu import _cfg

        W = OG.init_weights(OG.GemmaConfig(**_cfg()), seed=4)
        stack, vocab = GemmaStack(GemmaWeights.from_quantized(GemmaConfig(**_cfg()), W, OG.quantize(W, "bf16"), dev, "bf16")), 4096
    else:
        from oracle import qwen as OQ
        from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights
        from tests.test_qwen_gpu import SMALL

        stack, vocab = QwenStack(QwenWeights(QwenConfig(**SMALL), OQ.init_weights(OQ.QwenConfig(**SMALL), seed=3), dev)), 2048
    rng = np.random.default_rng(12)
    prefix = rng.integers(5, vocab, 90).tolist()
    tmpl = rng.integers(5, vocab, 6).tolist()
    sc = _scorer(stack, dev)
    a = sc.extract([ExtractJob(prefix, [ExtractPrompt("bare", [], 3), ExtractPrompt("tmpl", tmpl, 3)])])
    b = sc.extract([ExtractJob(prefix[:-1], [ExtractPrompt("moved", prefix[-1:], 3)])])
    assert set(a) == {"bare", "tmpl"} and a["bare"] and a["tmpl"] and sc.x_found == {}
    (t0, lp0), (t1, lp1) = a["bare"][0], b["moved"][0]
    print(f"{family}: bare slot {t0} ({lp0:.3f}); the same sequence with the last prefix token as its template {t1} ({lp1:.3f})")
    assert t0 == t1 and abs(lp0 - lp1) < 0.05


def test_extraction_branches_need_stop_ids(dev):
    from oracle import gemma as OG
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights
    from tests.test_decode_gpu import _cfg

    W = OG.init_weights(OG.GemmaConfig(**_cfg()), seed=4)
    stack = GemmaStack(GemmaWeights.from_quantized(GemmaConfig(**_cfg()), W, OG.quantize(W, "fp8row"), dev))
    trees = _mixed_trees(8, ((70, 1, (5,)),), 4096)
    sc = Scorer(stack, EngineConfig(token_budget=4096, min_stream=1024), dev)
    with pytest.raises(RuntimeError, match="stop_ids"):
        sc.score_grouped([(0, 0, trees[0])])
    out = sc.score_grouped([(0, 0, _mixed_trees(8, ((70, 1, ()),), 4096)[0])])  # the scorer is usable after the refusal
    assert len(out[0]) == 1 and torch.cuda.is_available()
