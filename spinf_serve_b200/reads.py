"""From option log-probs to what a caller reads: per-option probability, residual mass and the empty-content floor.

The reference computes these in its protocol compiler, right after the scorer returns (spinf_serve/compiler.py:649-656 `_read`,
:428-452 the floor job, :593-629 `assemble`); the compiler itself (request schema, tokenisation, templates) is outside this
path, but its three numbers are outputs of the scoring path, so they live here:

    lp[j]       log P(option j | prompt); an option written in several case variants is the log-sum of its variants
    p[j]        lp normalised over the question's options (a softmax over the options)
    residual    the next-token mass the options leave over: max(0, 1 - sum_j exp(lp[j]))
    floor_p     p of the same question read with no content in front of it: the options' prior under the template alone.
                All floor prompts of a call form ONE extra job keyed ("floor",): the model's start token as the shared
                trunk, each distinct (filled template, options) once as a branch.

Everything is float64 on the host; the inputs are the float64 sums score_grouped returns."""

from dataclasses import dataclass

import numpy as np

from spinf_serve_b200.packer import split_grouped_trees

FLOOR_KEY = ("floor",)


@dataclass
class OptionRead:
    logprob: np.ndarray          # [options] float64
    p: np.ndarray                # [options], sums to 1
    residual: float
    floor_p: np.ndarray | None = None
    floor_residual: float | None = None


def option_probs(variant_lp, starts=None):
    """variant_lp: the log-probs score_grouped returned for one prompt (one entry per option variant); starts: index of every
    option's first variant (None: one variant per option) -> (lp per option, p, residual)"""
    v = np.asarray(variant_lp, np.float64)
    if v.ndim != 1 or not len(v):
        raise ValueError("option_probs: expected a non-empty vector of log-probs")
    lp = v if starts is None else np.logaddexp.reduceat(v, np.asarray(starts, np.int64))
    peak = float(lp.max())
    rel = np.exp(lp - peak)          # the largest term is exactly 1: no overflow, no 0 / 0
    total = float(rel.sum())
    return lp, rel / total, max(0.0, 1.0 - np.exp(peak) * total)


def floor_items(start_ids, suffixes, plans, budget: int) -> list:
    """the content-less job: start_ids = what precedes a template when there is no content (the model's start token; may be empty
    when every suffix is non-empty), suffixes[k] = the token ids of floor prompt k (a filled template), plans[k] its ReadPlan ->
    score_grouped items keyed FLOOR_KEY, split over the budget like any other job (compiler.py:451-452)"""
    start = list(start_ids)
    for k, s in enumerate(suffixes):
        if not start and not len(s):
            raise ValueError(f"floor prompt {k} is empty and there is no start token: an option cannot be read after nothing")
    prompts = [start + list(s) for s in suffixes]
    return [(FLOOR_KEY, first, tree) for first, tree in split_grouped_trees(prompts, list(plans), budget)]


def read_with_floor(scores: dict, key, prompt: int, starts=None, floor_index: int | None = None) -> OptionRead:
    """scores: what score_grouped returned for a call that included floor_items; (key, prompt) the question's place in it;
    floor_index: its prompt in the floor job, None = the question asked for no floor (assemble, compiler.py:593-629)"""
    lp, p, res = option_probs(scores[key][prompt], starts)
    out = OptionRead(lp, p, res)
    if floor_index is not None:
        floor = scores.get(FLOOR_KEY)
        if floor is None or floor_index >= len(floor) or floor[floor_index] is None:
            raise KeyError(f"floor prompt {floor_index} was not scored in this call")
        _, out.floor_p, out.floor_residual = option_probs(floor[floor_index], starts)
    return out
