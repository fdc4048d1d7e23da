"""Parity metrics between two sets of scores, in the form the reference's parity runs report them (spinf_serve/parity.py:40-56):
absolute differences of the option log-probs, and of the "raw" score of a two-option question (log P(first) - log P(second)),
with their correlation and sign agreement. Inputs are the dicts Scorer.score_grouped returns ({key: [per prompt, float64 log-probs
per option]}) or the v0 form ({job id: [[lp_pos, lp_neg], ...]})."""

import numpy as np


def compare(ref: dict, got: dict) -> dict:
    """metrics over every prompt of `ref` (the same keys and shapes must be in `got`). Raw-score metrics use the first two options
    of every prompt; prompts with fewer than two options only enter the log-prob metrics."""
    r = [np.asarray(x, np.float64) for k in ref for x in ref[k]]
    g = [np.asarray(x, np.float64) for k in ref for x in got[k]]
    if not r:
        raise ValueError("compare: nothing to compare")
    d = np.abs(np.concatenate(g) - np.concatenate(r))
    pairs = [(a, b) for a, b in zip(r, g) if len(a) >= 2]
    rr = np.array([a[0] - a[1] for a, _ in pairs])
    gr = np.array([b[0] - b[1] for _, b in pairs])
    dr = np.abs(gr - rr)
    out = {
        "n": len(r),
        "lp_max_abs": float(d.max()),
        "lp_mean_abs": float(d.mean()),
        "lp_exact_share": float((d == 0).mean()),
    }
    if len(pairs):
        out.update(
            raw_max_abs=float(dr.max()), raw_mean_abs=float(dr.mean()),
            raw_corr=float(np.corrcoef(rr, gr)[0, 1]) if len(pairs) > 1 and rr.std() > 0 and gr.std() > 0 else 1.0,
            raw_sign_agree=float((np.sign(rr) == np.sign(gr)).mean()),
        )
    return out
