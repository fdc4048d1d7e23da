"""GPU parity of the tree-mask attention kernel (through the C ABI) with the oracle of the reference's FlexAttention call
(mask rule spinf_serve/scorer.py:173-177, operator spinf_serve/models/gemma4.py:110-119), and batch invariance."""

import numpy as np
import pytest
import torch

from oracle import attention as OA
from spinf_serve_b200 import packer as P

pytestmark = pytest.mark.gpu


def _cfg1_batch():
    rng = np.random.default_rng(0)
    pk = P.Packer(16384, 65536, align=True, min_stream=1024)
    for j in range(2):
        trunk = rng.integers(5, 262144, 470).tolist()
        prompts = [trunk + [1000 + 20 * j + q] + rng.integers(5, 262144, 15).tolist() for q in range(8)]
        list(pk.push(j, P.build_grouped_tree(prompts, [P.ReadPlan.build([[11], [12]]) for _ in prompts])))
    (b,) = list(pk.flush())
    return b


def _qkv(n, H, Hkv, D, seed, pre_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((n, H, D), generator=g) * pre_scale).to(torch.bfloat16)
    k = (torch.randn((n, Hkv, D), generator=g) * pre_scale).to(torch.bfloat16)
    v = (torch.randn((n, Hkv, D), generator=g) * pre_scale).to(torch.bfloat16)
    return q, k, v


def _run(dev, b, q, k, v, scale, window, layer):
    from spinf_serve_b200 import attention as A

    masks = A.stream_masks(b.art, b.end, b.pos, window, dev, always_window=True)
    return A.tree_attention(q.to(dev), k.to(dev), v.to(dev), masks[layer], scale).cpu()


def _check(out, ref, real, what):
    err = (out.float() - ref)[real].abs()
    tol = 2.0**-7 * ref[real].abs() + 2e-3 * ref[real].abs().max()  # bf16 output rounding + bf16 P rounding
    print(f"{what}: max abs err {err.max():.3e} (|ref| max {ref[real].abs().max():.3f})")
    assert bool((err <= tol).all()), f"{what}: max err {err.max():.3e}"


@pytest.mark.parametrize("reading", ["scale_arg", "pre_scaled"])
@pytest.mark.parametrize("layer", ["full_attention", "sliding_attention"])
def test_config1_attention(dev, reading, layer):
    """benchmark config 1: 2 contents x (470 + 8 x 16), 16 query / 8 KV heads, head_dim 256, seed 0. Two readings of "scaled by
    1/sqrt(256)": N(0,1) inputs with scale = 1/16 passed to the operator (primary), or inputs pre-multiplied with scale = 1"""
    b = _cfg1_batch()
    pre, scale = (1.0, 1.0 / 16) if reading == "scale_arg" else (1.0 / 16, 1.0)
    q, k, v = _qkv(b.length, 16, 8, 256, 0, pre)
    window = 1024 if layer == "sliding_attention" else None
    out = _run(dev, b, q, k, v, scale, 1024, layer)
    ref = OA.tree_attention(q, k, v, b.art, b.end, b.pos, scale, window)
    _check(out, ref, b.art >= 0, f"cfg1 {reading} {layer}")
    # pad rows attend to themselves only: their output is their own value row
    pads = np.flatnonzero(b.art < 0)
    assert torch.equal(out[pads], v[pads].repeat_interleave(2, dim=1))


@pytest.mark.parametrize("H,Hkv,D,window", [(4, 2, 128, 48), (6, 1, 256, 100), (2, 2, 128, None), (8, 4, 256, None)])
def test_random_tries_and_windows(dev, H, Hkv, D, window):
    """nested tries (multi-token lead-ins), ragged jobs, dense and aligned packing, a window that binds inside branches"""
    rng = np.random.default_rng(5)
    for align in (False, True):
        pk = P.Packer(2048, 65536, align=align)
        for j in range(5):
            trunk = rng.integers(1, 50, int(rng.integers(1, 400))).tolist()
            prompts = [trunk + rng.integers(50, 99, int(rng.integers(1, 30))).tolist() for _ in range(int(rng.integers(1, 7)))]
            list(pk.push(j, P.build_grouped_tree(prompts, [P.ReadPlan.build([[5], [6, 7], [6, 8, 9]]) for _ in prompts])))
        for b in pk.flush():
            q, k, v = _qkv(b.length, H, Hkv, D, 7)
            out = _run(dev, b, q, k, v, D**-0.5, window, "sliding_attention" if window else "full_attention")
            ref = OA.tree_attention(q, k, v, b.art, b.end, b.pos, D**-0.5, window)
            _check(out, ref, b.art >= 0, f"tries H{H}/{Hkv} D{D} w{window} align{align}")


def test_content_scores_bit_identical_alone_and_packed(dev):
    """batch invariance: a content's attention output is bit-identical alone, packed first, packed last and among many others,
    for both layer types (alignment makes its tile lists job-relative; the kernel's per-row order is ascending key sub-tiles)"""
    rng = np.random.default_rng(11)
    H, Hkv, D = 4, 2, 256

    def content(n_trunk, n_q):
        trunk = rng.integers(1, 1000, n_trunk).tolist()
        prompts = [trunk + [2000 + i] + rng.integers(1, 1000, int(rng.integers(3, 20))).tolist() for i in range(n_q)]
        return P.build_grouped_tree(prompts, [P.ReadPlan.build([[5], [6]]) for _ in prompts])

    target = content(700, 9)
    others = [content(int(rng.integers(20, 900)), int(rng.integers(1, 12))) for _ in range(12)]
    g = torch.Generator().manual_seed(3)
    n_t = -(-target.n_tokens // 128) * 128
    qt = torch.randn((n_t, H, D), generator=g).to(torch.bfloat16)
    kt = torch.randn((n_t, Hkv, D), generator=g).to(torch.bfloat16)
    vt = torch.randn((n_t, Hkv, D), generator=g).to(torch.bfloat16)
    results = []
    for order in ([target], [target] + others[:3], others[:3] + [target], others[:6] + [target] + others[6:]):
        pk = P.Packer(16384, 65536, align=True)
        for i, t in enumerate(order):
            list(pk.push("T" if t is target else i, t))
        (b,) = list(pk.flush())
        (o,) = [o for o in b.owners if o.job_id == "T"]
        gq = torch.Generator().manual_seed(99)
        q = torch.randn((b.length, H, D), generator=gq).to(torch.bfloat16)
        k = torch.randn((b.length, Hkv, D), generator=gq).to(torch.bfloat16)
        v = torch.randn((b.length, Hkv, D), generator=gq).to(torch.bfloat16)
        q[o.start : o.start + n_t], k[o.start : o.start + n_t], v[o.start : o.start + n_t] = qt, kt, vt
        per_layer = []
        for layer, w in (("full_attention", None), ("sliding_attention", 256)):
            out = _run(dev, b, q, k, v, 1.0 / 16, 256, layer)
            per_layer.append(out[o.start : o.start + o.n_tokens].clone())
        results.append(per_layer)
    for r in results[1:]:
        assert torch.equal(r[0], results[0][0]) and torch.equal(r[1], results[0][1])


def test_tree_flex_interface_shapes(dev):
    """the attention-interface callable takes [1, H, N, D] / [1, Hkv, N, D] views and returns ([1, N, H, D], None)"""
    from spinf_serve_b200 import attention as A

    b = _cfg1_batch()
    q, k, v = _qkv(b.length, 16, 8, 256, 1)
    masks = A.stream_masks(b.art, b.end, b.pos, 1024, dev)
    qd, kd, vd = (t.to(dev)[None].transpose(1, 2) for t in (q, k, v))
    out, none = A.tree_flex_forward(None, qd, kd, vd, masks["full_attention"], scaling=1.0 / 16)
    assert none is None and out.shape == (1, b.length, 16, 256) and out.is_contiguous()
    assert torch.equal(out[0], A.tree_attention(q.to(dev), k.to(dev), v.to(dev), masks["full_attention"], 1.0 / 16))


def test_row_maxima_of_the_output_come_with_it(dev):
    """the optional per-token max |out| (what the row-wise quantiser of the output projection's input needs) equals the maximum of
    the stored bf16 output, for both item layouts (one head per item; two heads sharing a key/value head)"""
    from spinf_serve_b200 import attention as A

    b = _cfg1_batch()
    for H, Hkv, D in ((16, 8, 256), (3, 3, 128)):
        q, k, v = _qkv(b.length, H, Hkv, D, 3)
        masks = A.stream_masks(b.art, b.end, b.pos, 1024, dev, always_window=True)
        amax = torch.zeros(b.length, dtype=torch.float32, device=dev)
        out = A.tree_attention(q.to(dev), k.to(dev), v.to(dev), masks["full_attention"], D**-0.5, row_amax=amax)
        assert torch.equal(amax, out.float().abs().amax(dim=(1, 2)))


@pytest.mark.parametrize("H,Hkv", [(2, 2), (2, 1)])
def test_very_long_stream_takes_the_unsorted_walk_with_the_same_bits(dev, H, Hkv):
    """beyond 2048 query blocks the kernel walks the stream in natural order instead of ranking blocks by cost: the order only moves
    whole items between CTAs, so a job's rows are the same bits inside a 2100-block stream as alone (one CTA each, and CTA pairs)"""
    from spinf_serve_b200 import attention as A

    nb, D = 2100, 128
    lens = np.where(np.arange(nb) % 3 == 0, 256, 128)  # jobs of one or two blocks, causal inside a job
    lens = lens[np.cumsum(lens) <= nb * 128]
    n = int(lens.sum())
    assert n // 128 > 2048
    start = np.concatenate(([0], np.cumsum(lens)[:-1]))
    art = np.repeat(np.arange(len(lens)), lens).astype(np.int32)
    end = np.repeat(start + lens, lens).astype(np.int32)
    pos = (np.arange(n) - np.repeat(start, lens)).astype(np.int32)
    g = torch.Generator().manual_seed(3)
    q = torch.randn((n, H, D), generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    full = A.tree_attention(q, k, v, A.stream_masks(art, end, pos, None, dev)["full_attention"], D**-0.5)
    for j in (0, 1, 700, len(lens) - 1):
        a, e = int(start[j]), int(start[j] + lens[j])
        m = A.stream_masks(np.zeros(e - a, np.int32), np.full(e - a, e - a, np.int32), pos[a:e], None, dev)["full_attention"]
        alone = A.tree_attention(q[a:e].contiguous(), k[a:e].contiguous(), v[a:e].contiguous(), m, D**-0.5)
        assert torch.equal(alone, full[a:e])
