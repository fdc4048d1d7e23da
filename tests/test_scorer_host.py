"""Host logic of the scorer's two-thread flow, without a GPU: the real Scorer._execute / _prepare / _harvest run here over
stand-ins for the CUDA pieces (staging blocks that copy nothing, a launch that computes its result on the host, events that are
always complete). Failures are made on the host: an exception in the packing thread, an out-of-memory error raised by the launch."""

import threading
from collections import deque

import numpy as np
import pytest
import torch

from spinf_serve_b200 import packer as P
from spinf_serve_b200 import scorer as S


def fake_lp(prev, target):
    return -((prev * 31 + target * 7) % 97) / 10.0


class Done:
    def query(self):
        return True

    def synchronize(self):
        pass


class Block:
    copied = None

    def __init__(self):
        self.packs = 0

    def pack(self, arrays):
        self.packs += 1
        self.arrays = arrays


class FakeStack:
    window = None

    def __init__(self):
        self.planned = 0

    def plan(self, sc, b):
        self.planned += 1


def make_scorer(n_blocks=2, fail_at=None, error=None):
    sc = object.__new__(S.Scorer)
    sc.cfg = S.EngineConfig(token_budget=512, max_tokens=4096, prefetch=n_blocks - 1)
    sc.device, sc.torch, sc.stack = "cpu", torch, FakeStack()
    sc.budget, sc.max_tokens, sc.min_stream = 512, 4096, sc.cfg.min_stream
    sc.stats = S.Stats()
    sc._blocks = [Block() for _ in range(n_blocks)]
    sc._results, sc._workspace = [], None
    sc.launched = []

    def launch(t, flow):
        if fail_at is not None and len(sc.launched) == fail_at:
            raise error
        sc.launched.append(t.batch)
        flow.give_block(t.block)
        b, cols = t.batch, t.cols
        lp = np.array([[fake_lp(int(b.ids[q]), c) for c in cols] for q in b.sel], np.float32).reshape(len(b.sel), len(cols))
        return S._Flight(b, cols, torch.from_numpy(lp), Done(), torch.zeros(1))

    sc._launch = launch
    sc._settle = lambda check: None
    return sc


def jobs(n, seed=4):
    rng = np.random.default_rng(seed)
    items, truth = [], {}
    for j in range(n):
        trunk = rng.integers(1, 300, int(rng.integers(1, 120))).tolist()
        prompts = [trunk + rng.integers(1, 300, int(rng.integers(1, 7))).tolist() for _ in range(int(rng.integers(1, 6)))]
        options = [[rng.integers(1, 40, int(rng.integers(1, 4))).tolist() for _ in range(int(rng.integers(2, 5)))] for _ in prompts]
        items.append((("job", j), 0, P.build_grouped_tree(prompts, [P.ReadPlan.build(o) for o in options])))
        truth[("job", j)] = [
            [sum(fake_lp((pr + opt)[len(pr) - 1 + i], opt[i]) for i in range(len(opt))) for opt in opts] for pr, opts in zip(prompts, options)
        ]
    return items, truth


def check(out, truth):
    assert out.keys() == truth.keys()
    for key, want in truth.items():
        for got, w in zip(out[key], want):
            assert np.allclose(got, w, atol=1e-4)


def test_a_call_scores_every_job_and_recycles_its_staging_blocks():
    items, truth = jobs(40)
    sc = make_scorer(n_blocks=2)
    check(sc.score_grouped(iter(items)), truth)  # a one-shot iterator: the items are consumed lazily, once
    assert sc.stats.forwards == len(sc.launched) > 2 and sc.stack.planned == sc.stats.forwards
    assert sum(b.packs for b in sc._blocks) == sc.stats.forwards  # more forwards than blocks: the free list went round
    assert sc.stats.tokens == sum(t.n_tokens for _, _, t in items)


def test_v0_jobs():
    prompts = [[1, 2, 3, 4], [1, 2, 3, 9, 8]]
    options = [[[20], [21, 22], [21, 23]], [[30, 31, 32], [33]]]
    res = make_scorer().score_trees([("a", prompts, options)])
    for pr, opts, got in zip(prompts, options, res["a"].logprobs):
        for opt, g in zip(opts, got):
            assert abs(g - sum(fake_lp((pr + opt)[len(pr) - 1 + i], opt[i]) for i in range(len(opt)))) < 1e-4
    assert res["a"].trees == 1 and res["a"].packed_tokens > 0
    with pytest.raises(ValueError, match="unique"):
        make_scorer().score_trees([("a", prompts, options), ("a", prompts, options)])


def test_an_exception_in_the_packing_thread_reaches_the_caller_and_the_scorer_stays_usable():
    items, truth = jobs(30)

    def broken():
        for i, it in enumerate(items):
            if i == 17:
                raise KeyError("tokenizer gave up")
            yield it

    sc = make_scorer(n_blocks=2)
    before = threading.active_count()
    with pytest.raises(KeyError, match="tokenizer gave up"):
        sc.score_grouped(broken())
    assert threading.active_count() == before  # the packing thread has ended
    check(sc.score_grouped(items), truth)


def test_an_oversize_job_is_refused_like_the_reference_refuses_it():
    tree = P.build_grouped_tree([list(range(1, 5000))], [P.ReadPlan.build([[7], [8]])])
    with pytest.raises(ValueError, match="exceed"):
        make_scorer().score_grouped([(("big",), 0, tree)])


@pytest.mark.parametrize("error", [torch.OutOfMemoryError("CUDA out of memory (made up on the host)"), RuntimeError("launch failed")])
def test_a_failure_in_the_gpu_loop_cancels_the_packing_thread(error):
    """the third forward fails while the packing thread is ahead and waiting for a block: the call raises that error, the thread
    wakes and ends, and the next call on the same scorer works"""
    items, truth = jobs(60)
    sc = make_scorer(n_blocks=2, fail_at=2, error=error)
    before = threading.active_count()
    with pytest.raises(type(error)):
        sc.score_grouped(items)
    assert threading.active_count() == before
    assert len(sc.launched) == 2
    good = make_scorer(n_blocks=2)
    good._blocks = sc._blocks  # the failed call's staging blocks serve the next call
    check(good.score_grouped(items), truth)


def test_a_failed_call_keeps_none_of_its_extraction_captures():
    """a forward fails after earlier forwards of the call left captures with the extractor: the error reaches the caller, the held
    captures are dropped and the stack is told to close its capture; a call that succeeds decodes what it held at its end"""
    calls = []

    class FakeExtractor:
        found = {}

        def __init__(self):
            self.held = ["captures of the first forward"]

        def flush(self):
            calls.append(("flush", list(self.held)))
            self.held = []

        def drop(self):
            calls.append(("drop", list(self.held)))
            self.held = []

        tree_bytes = staticmethod(lambda tree: 0)

    items, truth = jobs(60)
    sc = make_scorer(n_blocks=2, fail_at=2, error=RuntimeError("launch failed"))
    sc.extractor = FakeExtractor()
    sc.stack.abandon = lambda s: calls.append(("abandon", s is sc))
    with pytest.raises(RuntimeError, match="launch failed"):
        sc.score_grouped(items)
    assert calls == [("drop", ["captures of the first forward"]), ("abandon", True)] and sc.extractor.held == []
    calls.clear()
    good = make_scorer(n_blocks=2)
    good.extractor = FakeExtractor()
    check(good.score_grouped(items), truth)
    assert calls == [("flush", ["captures of the first forward"])] and good.x_found == {}


def test_results_are_handed_over_in_launch_order_and_at_most_lag_stay_back():
    class Later(Done):
        def __init__(self):
            self.ready = False

        def query(self):
            return self.ready

        def synchronize(self):
            self.ready = True

    sc = make_scorer()
    seen = []
    flights = deque()
    b = type("B", (), {"sel": np.zeros(1), "n_tokens": 1})()
    for i in range(4):
        flights.append(S._Flight(b, [i], torch.zeros((1, 1)), Later(), torch.zeros(1)))
        sc._harvest(flights, lambda lp, cols, bb: seen.append(cols[0]), keep=1)
    assert seen == [0, 1, 2] and len(flights) == 1  # nothing was complete early: only the lag bound forced hand-overs
    flights[0].done.ready = True
    sc._harvest(flights, lambda lp, cols, bb: seen.append(cols[0]), keep=1)
    assert seen == [0, 1, 2, 3]  # a finished forward is handed over without waiting for the next launch


def test_packer_forward_count_of_the_bulk_benchmark_call():
    """k x 24 configuration-2 contents at the 27648-token budget are k forwards of 27648 tokens (the benchmark's end-to-end leg)"""
    from spinf_serve_b200 import workloads

    wl = workloads.config2(seed=0)
    assert wl.token_budget == 27648
    for steps in (1, 5, 20):
        pk = P.Packer(wl.token_budget, 65536, True, 1024)
        bulk = [((s,) + tuple(k), f, t) for s in range(steps) for k, f, t in wl.items]
        bs = [b for key, first, t in bulk for b in pk.push((key, first), t)] + list(pk.flush())
        assert [b.length for b in bs] == [27648] * steps
