"""Oracle of the tree-mask attention (numpy / CPU torch; test infrastructure only, never imported by the product).

The visibility rule is the reference's mask_mod (spinf_serve/scorer.py:173-177; the same rule is the ground truth of the
reference's own packer tests, tests/test_packer.py:74-79):
    visible(q, k) = (k <= q and art[q] >= 0 and art[k] == art[q] and q < end[k]) or q == k
and on sliding layers additionally pos[q] - pos[k] < window (on positions, which restart on every branch). The operator is the
reference's FlexAttention call (spinf_serve/models/gemma4.py:110-119): bf16 inputs, fp32 scores and softmax, GQA by head
grouping, output [n, H, D]. On CPU the reference's eager flex_attention with its BlockMask equals this dense-mask form exactly."""

import numpy as np
import torch


def dense_mask(art, end, pos=None, window=None):
    """bool [n, n] (query row, key column)"""
    art = np.asarray(art)
    end = np.asarray(end)
    n = len(art)
    q = np.arange(n)[:, None]
    k = np.arange(n)[None, :]
    m = (k <= q) & (art[q] >= 0) & (art[k] == art[q]) & (q < end[k])
    if window:
        p = np.asarray(pos).astype(np.int64)
        m &= (p[q] - p[k]) < window
    return m | (q == k)


def tree_attention(q, k, v, art, end, pos, scale, window=None, round_p=False):
    """q [n, H, D], k / v [n, Hkv, D] (bf16 or float) -> [n, H, D] fp32: softmax(scale * q k^T over visible keys) v in fp32.
    round_p=True rounds the normalised probabilities' numerators to bf16 before the value product, as the kernels do."""
    n, H, D = q.shape
    Hkv = k.shape[1]
    mask = torch.from_numpy(dense_mask(art, end, pos, window))
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(H // Hkv, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(H // Hkv, dim=0)
    s = (qf @ kf.transpose(1, 2)) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    if round_p:
        m = s.amax(-1, keepdim=True)
        p = torch.exp(s - m)
        o = (p.to(torch.bfloat16).float() @ vf) / p.sum(-1, keepdim=True)
    else:
        o = torch.softmax(s, dim=-1) @ vf
    return o.permute(1, 0, 2).contiguous()


def unmasked_pairs(art, end, pos=None, window=None):
    """number of visible (q, k) pairs with a real query row (pads' self-pairs left out): the unit of attention FLOPs"""
    m = dense_mask(art, end, pos, window)
    return int(m[np.asarray(art) >= 0].sum())
