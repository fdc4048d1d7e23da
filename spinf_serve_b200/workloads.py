"""Seeded synthetic workloads with the shapes of the benchmark configurations (they stand in for the reference's Wikinews benchmark
of 24 articles x 56 two-option questions, benchmarks/README.md:31-37 in the spinf-serve tree: same token counts, uniform random
token ids, no text). A workload is a list of score_grouped items: ((content id,), 0, GroupedTree)."""

from dataclasses import dataclass

import numpy as np

from spinf_serve_b200 import packer as P


@dataclass
class Workload:
    name: str
    items: list
    n_questions: int
    n_tokens: int  # real tokens (trunks once + branches)
    token_budget: int


def _content(rng, vocab, trunk_len, branch_lens, option_counts):
    """one content: a trunk of uniform random ids, one branch per question whose first token is distinct (so the trie cannot
    merge siblings), each question ending in a choice among single-token options"""
    trunk = rng.integers(0, vocab, trunk_len).tolist()
    first = rng.choice(vocab, size=len(branch_lens), replace=False).tolist()
    prompts, plans = [], []
    for f, bl, no in zip(first, branch_lens, option_counts):
        prompts.append(trunk + [f] + rng.integers(0, vocab, bl - 1).tolist())
        plans.append(P.ReadPlan.build([[int(t)] for t in rng.choice(vocab, size=no, replace=False)]))
    return P.build_grouped_tree(prompts, plans)


def fixed(name, n_contents, trunk, n_questions, branch, n_options, vocab, token_budget, seed=0, first_id=0) -> Workload:
    rng = np.random.default_rng(seed)
    items = [((first_id + c,), 0, _content(rng, vocab, trunk, [branch] * n_questions, [n_options] * n_questions)) for c in range(n_contents)]
    return Workload(name, items, n_contents * n_questions, n_contents * (trunk + n_questions * branch), token_budget)


def config1(seed=0):
    """attention alone: 2 contents x (470-token trunk + 8 questions of 16 tokens) = 1196 tokens"""
    return fixed("cfg1-attention", 2, 470, 8, 16, 2, 262144, 16384, seed)


def config2(seed=0, n_contents=24, first_id=0):
    """12B fp8: 24 contents x (470-token trunk + 56 questions of 12 tokens, 2 single-token options) = 1344 questions, one forward"""
    # 24 aligned contents of 1152 tokens fill exactly one 27648-token stream: with this budget a bulk call of k x 24 contents packs
    # into k forwards of that shape (a larger budget would pack 28 per forward and change the shape)
    return fixed("cfg2-gemma12b-24x56", n_contents, 470, 56, 12, 2, 262144, 27648, seed, first_id)


def config3(seed=0, n_contents=8192):
    """bulk: trunks uniform in 200-2000, 56 questions with branches uniform in 8-24 and 2-5 options, 32768-token passes"""
    rng = np.random.default_rng(seed)
    items, nq, nt = [], 0, 0
    for c in range(n_contents):
        trunk = int(rng.integers(200, 2001))
        bl = rng.integers(8, 25, 56).tolist()
        no = rng.integers(2, 6, 56).tolist()
        items.append(((c,), 0, _content(rng, 262144, trunk, bl, no)))
        nq += 56
        nt += trunk + sum(bl)
    return Workload("cfg3-bulk", items, nq, nt, 32768)


def bulk_content(seed: int, cid: int):
    """content `cid` of the bulk configuration, drawn from its own generator (seed, cid): any replica can make any content
    without the others, and a content is the same whichever replica draws it -> (item, questions, real tokens)"""
    rng = np.random.default_rng([seed, cid])
    trunk = int(rng.integers(200, 2001))
    bl = rng.integers(8, 25, 56).tolist()
    no = rng.integers(2, 6, 56).tolist()
    return ((cid,), 0, _content(rng, 262144, trunk, bl, no)), 56, trunk + sum(bl)


def bulk_slice(seed: int, n_contents: int, first_id: int = 0) -> Workload:
    """contents first_id .. first_id + n_contents - 1 of the bulk configuration (the shapes of config3, per-content seeding)"""
    parts = [bulk_content(seed, first_id + c) for c in range(n_contents)]
    return Workload("cfg3-bulk-slice", [p[0] for p in parts], sum(p[1] for p in parts), sum(p[2] for p in parts), 32768)


def config4(seed=0, n_contents=2048):
    """31B-class: contents of a 1000-token trunk + 32 questions of 16 tokens, 5 options"""
    return fixed("cfg4-gemma31b", n_contents, 1000, 32, 16, 5, 262144, 32768, seed)


def attended_pairs(b, window: int | None = None) -> int:
    """(query, key) pairs of a packed batch that attend: the mask rule counted job by job (a token never attends outside its job;
    a pad attends to itself). This is the count the attention's algorithmic FLOPs are quoted on: 4 x head_dim x heads per pair."""
    art, end, pos = np.asarray(b.art), np.asarray(b.end), np.asarray(b.pos)
    total = int((art < 0).sum())
    real = np.flatnonzero(art >= 0)
    cuts = np.flatnonzero(np.diff(art[real])) + 1
    for idx in np.split(real, cuts):
        q = idx[:, None]
        k = idx[None, :]
        vis = (k <= q) & (q < end[idx][None, :])
        if window:
            vis &= (pos[idx][:, None] - pos[idx][None, :]) < window
        vis |= q == k
        total += int(vis.sum())
    return total


def gemm_flops(cfg, n_tokens: int) -> float:
    """algorithmic FLOPs of the quantized linears over n_tokens real tokens"""
    return 2.0 * cfg.linear_params * cfg.layers * n_tokens


def head_flops(cfg, n_rows: int) -> float:
    return 2.0 * n_rows * cfg.hidden * cfg.vocab
