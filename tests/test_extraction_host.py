"""Host logic of extraction on the scoring pass (extraction.Extractor; the reference's Scorer._x_collect / _x_chunks / _x_split /
_x_tree_bytes, spinf_serve/scorer.py:768-895), on CPU with captures that are plain CPU tensors and a decoder that is never built:
what a forward will capture for a tree, when held captures are decoded, and how groups are cut into chunks under a budget."""

import types

import torch

from spinf_serve_b200 import decode as D
from spinf_serve_b200 import packer as P
from spinf_serve_b200.extraction import Extractor

PER_TOK = {0: 64, 1: 64, 2: 32}  # bytes of K and V per stored token, by layer


def _stack():
    return types.SimpleNamespace(hybrid=False, kv_bytes_per_token=lambda: dict(PER_TOK), cfg=types.SimpleNamespace(), n_layers=3)


def _group(gi, n_prefix, Ts, max_tokens=4):
    kv = lambda n: {li: (torch.zeros(n, 1, 1), torch.zeros(n, 1, 1)) for li in PER_TOK}  # noqa: E731
    g = D.Group(kv(n_prefix), n_prefix)
    for j, T in enumerate(Ts):
        g.prompts.append((types.SimpleNamespace(key=(gi, j), max_tokens=max_tokens), kv(T), T, torch.zeros(8)))
    return g


def _extractor(**kw):
    return Extractor(_stack(), "cpu", (1,), beam=2, **kw)


def test_tree_bytes_counts_prefix_and_templates():
    x = _extractor()
    t = P.GroupedTree(list(range(100)), [[1, 2, 3], [4, 5], [6]], [], [])
    assert x.tree_bytes(t) == 0
    pr = types.SimpleNamespace(key=0, max_tokens=4)
    t.xbranches = [(0, pr), (2, pr), (-1, pr)]  # two templates and a slot that starts right after the prefix
    assert x.tree_bytes(t) == (100 + 3 + 1) * sum(PER_TOK.values())


def test_chunks_stay_under_the_budget_and_keep_every_prompt_in_order():
    groups = [_group(0, 300, (5, 9, 7, 4, 6)), _group(1, 50, (3,)), _group(2, 120, (8, 8)), _group(3, 40, (2, 2, 2))]
    keys = [p[0].key for g in groups for p in g.prompts]
    big = _extractor(chunk_budget=1e12)
    (one,) = list(big._chunks(list(groups)))
    assert [p[0].key for g in one for p in g.prompts] == keys

    whole = big._chunk_bytes([groups[0]])
    one_prompt = big._chunk_bytes([big._run(groups[0], 0, 1)])
    budget = (whole + one_prompt) // 2  # group 0 does not fit alone, a run of it does
    x = _extractor(chunk_budget=budget)
    prefix0 = groups[0].prefix_kv[0][0]
    chunks = list(x._chunks(groups))
    assert groups == []  # consumed: the caller's references are gone
    assert len(chunks) > 2
    assert [p[0].key for c in chunks for g in c for p in g.prompts] == keys
    for c in chunks:
        assert x._chunk_bytes(c) <= budget or (len(c) == 1 and len(c[0].prompts) == 1)
    runs0 = [g for c in chunks for g in c if g.prompts[0][0].key[0] == 0]
    assert len(runs0) > 1 and all(g.prefix_kv[0][0] is prefix0 and g.P == 300 for g in runs0)  # the runs share the prefix captures
    # each run is the longest that fits: adding the next prompt of the group would pass the budget
    flat = [p for g in runs0 for p in g.prompts]
    at = 0
    for g in runs0[:-1]:
        at += len(g.prompts)
        longer = D.Group(dict(g.prefix_kv), g.P, list(g.prompts) + [flat[at]])
        assert x._chunk_bytes([longer]) > budget


def test_held_captures_are_decoded_when_they_pass_the_budget():
    flushed = []

    class Recording(Extractor):
        def flush(self):
            flushed.append([p[0].key for g in self._held for p in g.prompts])
            self._held, self._held_bytes = [], 0

    probe = _extractor()
    need = [D.group_bytes(_group(i, 200, (5, 5)), PER_TOK, 5, 2) for i in range(3)]
    x = Recording(_stack(), "cpu", (1,), beam=2, hold_budget=need[0] + need[1] + 1)

    def owner(gi, n_prefix, Ts):
        prs = [types.SimpleNamespace(key=(gi, j), max_tokens=4) for j in range(len(Ts))]
        o = types.SimpleNamespace(prefix_len=n_prefix, xbranches=[(1000 + 10 * j, T, pr) for j, (T, pr) in enumerate(zip(Ts, prs, strict=True))])
        kv = lambda n: {li: (torch.zeros(n, 1, 1), torch.zeros(n, 1, 1)) for li in PER_TOK}  # noqa: E731
        cap = {("p", id(o)): kv(n_prefix)}
        cap.update({("t", pr.key): kv(T) for T, pr in zip(Ts, prs, strict=True)})
        return o, cap

    assert Extractor.ends([owner(0, 10, (5, 7))[0]]) == [1004, 1016]
    for gi in range(3):
        o, kv = owner(gi, 200, (5, 5))
        x.collect([o], {"kv": kv, "extra": None}, torch.zeros(2, 8))
        assert not kv  # the captures moved into the group
    assert flushed == [[(0, 0), (0, 1), (1, 0), (1, 1)]]  # the third group did not fit beside the first two
    assert [p[0].key for g in x._held for p in g.prompts] == [(2, 0), (2, 1)]
    x.drop()
    assert x._held == [] and x._held_bytes == 0
    # a group over the budget on its own is decoded at once
    flushed.clear()
    y = Recording(_stack(), "cpu", (1,), beam=2, hold_budget=10)
    o, kv = owner(5, 200, (5,))
    y.collect([o], {"kv": kv, "extra": None}, torch.zeros(1, 8))
    assert flushed == [[(5, 0)]] and probe.found == {}
