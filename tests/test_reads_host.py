"""p / residual / floor reads (the product side of compiler._read and the floor job, spinf_serve/compiler.py:649-656, 428-452)
against the oracle's restatement and the reference's own known answers (tests/test_protocol_compiler.py:237-264 geometry)."""

import math

import numpy as np
import pytest

from oracle import head as OH
from spinf_serve_b200 import packer as P
from spinf_serve_b200 import reads


def test_option_probs_equals_the_oracle_and_the_definition():
    rng = np.random.default_rng(0)
    for n in (2, 3, 5):
        lp = np.log(rng.dirichlet(np.ones(n + 3))[:n])  # options take part of the mass
        got_lp, p, res = reads.option_probs(lp)
        want_p, want_res = OH.read_probs(lp)
        assert np.array_equal(got_lp, lp) and np.allclose(p, want_p, rtol=0, atol=1e-15) and abs(res - want_res) < 1e-15
        assert abs(p.sum() - 1) < 1e-12 and abs(res - (1 - np.exp(lp).sum())) < 1e-12


def test_case_variants_are_merged_before_normalising():
    v = np.log(np.array([0.10, 0.05, 0.20, 0.01, 0.02, 0.02]))
    lp, p, res = reads.option_probs(v, starts=[0, 2, 3])
    assert np.allclose(np.exp(lp), [0.15, 0.20, 0.05])
    assert np.allclose(p, np.array([0.15, 0.20, 0.05]) / 0.40) and abs(res - 0.60) < 1e-12


def test_residual_is_clamped_and_large_negative_logprobs_do_not_underflow_p():
    _, p, res = reads.option_probs(np.array([-1e-9, -30.0]))
    assert res == 0.0 or res < 1e-8
    _, p, res = reads.option_probs(np.array([-800.0, -801.0]))
    assert np.allclose(p, [1 / (1 + math.exp(-1)), math.exp(-1) / (1 + math.exp(-1))]) and res == 1.0
    with pytest.raises(ValueError):
        reads.option_probs([])


def test_floor_job_is_one_grouped_job_over_the_start_token():
    plans = [P.ReadPlan.build([[7], [8]]), P.ReadPlan.build([[7], [8], [9]])]
    items = reads.floor_items([2], [[11, 12, 13], [11, 12, 14, 15]], plans, budget=4096)
    assert [(k, f) for k, f, _ in items] == [(reads.FLOOR_KEY, 0)]
    tree = items[0][2]
    assert tree.prefix == [2, 11, 12] and len(tree.plans) == 2  # the start token and the templates' common start are the trunk
    with pytest.raises(ValueError, match="nothing"):
        reads.floor_items([], [[]], plans[:1], 4096)
    split = reads.floor_items([2], [list(range(100, 160)), list(range(200, 260))], plans, budget=70)
    assert [f for _, f, _ in split] == [0, 1]  # over the budget: contiguous runs, each re-sending the start token


def test_read_with_floor():
    scores = {("in", 0): [np.log([0.6, 0.2])], reads.FLOOR_KEY: [np.log([0.3, 0.3])]}
    r = reads.read_with_floor(scores, ("in", 0), 0, floor_index=0)
    assert np.allclose(r.p, [0.75, 0.25]) and abs(r.residual - 0.2) < 1e-12
    assert np.allclose(r.floor_p, [0.5, 0.5]) and abs(r.floor_residual - 0.4) < 1e-12
    assert reads.read_with_floor(scores, ("in", 0), 0).floor_p is None
    with pytest.raises(KeyError):
        reads.read_with_floor(scores, ("in", 0), 0, floor_index=3)
