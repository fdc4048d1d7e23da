"""Oracle of the lm-head read (CPU torch; test infrastructure only). Follows Scorer._logprobs in its `fp32` branch
(spinf_serve/scorer.py:346-355), which the reference states gives the same logits as the `f32out` GEMM, then the column gather of
Scorer._forward (scorer.py:254); read_options follows read_grouped (scorer.py:57-71) and compiler._read (compiler.py:649-656)."""

import numpy as np
import torch


def logprobs(h, W, softcap=None):
    """h [S, hidden] bf16, W [vocab, hidden] bf16 -> log-probs [S, vocab] fp32 (scorer.py:340-355)"""
    logits = h.float() @ W.float().t()
    if softcap:
        logits = torch.tanh(logits / softcap) * softcap
    return torch.log_softmax(logits.float(), dim=-1)


def option_logprobs(h, W, cols, softcap=None, chunk=256):
    """the [:, cols] columns of logprobs(h, W), computed in row chunks so [S, vocab] stays small (scorer.py:254)"""
    ci = torch.as_tensor(np.asarray(cols), dtype=torch.int64)
    out = [logprobs(h[s : s + chunk], W, softcap)[:, ci] for s in range(0, h.shape[0], chunk)]
    return torch.cat(out) if out else torch.zeros((0, len(ci)))


def read_probs(lp_variants):
    """per-option log-probs (one question, case variants already merged) -> (p, residual): compiler.py:649-656
    p = softmax over the options; residual = max(0, 1 - sum(exp(lp)))"""
    lp = np.asarray(lp_variants, np.float64)
    m = lp.max()
    e = np.exp(lp - m)
    return e / e.sum(), max(0.0, 1.0 - float(np.exp(lp).sum()))
