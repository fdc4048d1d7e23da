"""Oracle of the tree-mask attention (numpy / CPU torch; test infrastructure only, never imported by the product).

The visibility rule is the reference's mask_mod (spinf_serve/scorer.py:173-177; the same rule is the ground truth of the
reference's own packer tests, tests/test_packer.py:74-79):
    visible(q, k) = (k <= q and art[q] >= 0 and art[k] == art[q] and q < end[k]) or q == k
and on sliding layers additionally pos[q] - pos[k] < window (on positions, which restart on every branch). The operator is the
reference's FlexAttention call (spinf_serve/models/gemma4.py:110-119): bf16 inputs, fp32 scores and softmax, GQA by head
grouping, output [n, H, D]. On CPU the reference's eager flex_attention with its BlockMask equals this dense-mask form exactly.
Streams with images (spinf_serve/scorer.py:178-198): grp[t] = the image a placeholder token belongs to (-1 elsewhere); the
full_img / sliding_img rules add  grp[q] == grp[k] and grp[q] >= 0  (an image's placeholders see each other both ways), on models
whose global layers stay causal only on the sliding layers and only when pos[q] - pos[k] < window (grp_in_window)."""

import numpy as np
import torch


def dense_mask(art, end, pos=None, window=None, grp=None, grp_in_window=False):
    """bool [n, n] (query row, key column)"""
    art = np.asarray(art)
    end = np.asarray(end)
    n = len(art)
    q = np.arange(n)[:, None]
    k = np.arange(n)[None, :]
    m = (k <= q) & (art[q] >= 0) & (art[k] == art[q]) & (q < end[k])
    p = None if pos is None else np.asarray(pos).astype(np.int64)
    if window:
        m &= (p[q] - p[k]) < window
    m |= q == k
    if grp is not None:
        g = np.asarray(grp)
        img = (g[q] == g[k]) & (g[q] >= 0)
        if grp_in_window and window:
            img &= (p[q] - p[k]) < window
        m |= img
    return m


def tree_attention(q, k, v, art, end, pos, scale, window=None, round_p=False, grp=None, grp_in_window=False):
    """q [n, H, D], k / v [n, Hkv, D] (bf16 or float) -> [n, H, D] fp32: softmax(scale * q k^T over visible keys) v in fp32.
    round_p=True rounds the normalised probabilities' numerators to bf16 before the value product, as the kernels do."""
    n, H, D = q.shape
    Hkv = k.shape[1]
    mask = torch.from_numpy(dense_mask(art, end, pos, window, grp, grp_in_window))
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
