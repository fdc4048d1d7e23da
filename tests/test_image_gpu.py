"""Streams with images on the GPU (through the C ABI): the visibility words of spinf_tile_mask_bits_img against the dense image
mask rules (spinf_serve/scorer.py:178-198), the tree attention over them against the oracle, a Gemma-style stack whose shared
prefix carries an image (two-way blocks, the image's rows laid over the placeholders' embeddings, gemma4.py:410-413) against the
oracle's forward, and that a job with an image scores bit-identically alone and packed."""

import json
import os

import numpy as np
import pytest
import torch

from oracle import attention as OA
from spinf_serve_b200 import packer as P

pytestmark = pytest.mark.gpu

NPZ = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "image_golden.npz"))
META = json.loads(bytes(NPZ["meta"]).decode())
CASES = [(name, bi) for name in sorted(META) for bi in range(META[name]["n_batches"])]


def _arrays(name, bi):
    key = f"{name}/b{bi}/"
    return {k: NPZ[key + k] for k in ("art", "end", "pos", "grp")}, META[name]["window"]


@pytest.mark.parametrize("name,bi", CASES)
@pytest.mark.parametrize("bidir_all", [True, False])
def test_mask_words_equal_the_dense_image_rules(dev, name, bi, bidir_all):
    from spinf_serve_b200 import attention as A

    a, window = _arrays(name, bi)
    n = len(a["art"])
    masks = A.stream_masks(a["art"], a["end"], a["pos"], window, dev, always_window=True, grp=a["grp"], bidir_all=bidir_all)
    for kind, w in (("full_attention", None), ("sliding_attention", window)):
        if kind == "sliding_attention" and not window:
            continue
        m = masks[kind]
        g = a["grp"] if (bidir_all or w) else None
        dense = OA.dense_mask(a["art"], a["end"], a["pos"], w, g, grp_in_window=not bidir_all)
        off, blocks = m.offsets.cpu().numpy(), m.blocks.cpu().numpy()
        bits = m.bits.cpu().numpy().view(np.uint64)  # [visited, 2, 128]
        seen = np.zeros((n, n), bool)
        for i in range(n // P.BLOCK):
            for e in range(off[i], off[i + 1]):
                j = int(blocks[e])
                words = bits[e]  # [2, 128]
                tile = ((words[:, :, None] >> np.arange(64, dtype=np.uint64)[None, None, :]) & np.uint64(1)).astype(bool)  # [half, row, col]
                seen[i * P.BLOCK : (i + 1) * P.BLOCK, j * P.BLOCK : (j + 1) * P.BLOCK] = np.concatenate([tile[0], tile[1]], axis=1)
        assert np.array_equal(seen, dense), (name, bi, kind, bidir_all)


def _qkv(n, H, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn((n, h, D), generator=g).to(torch.bfloat16) for h in (H, Hkv, Hkv))


@pytest.mark.parametrize("name,bi", [("img0", 0), ("img1", 0), ("img4", 0)])
@pytest.mark.parametrize("H,Hkv,D", [(4, 2, 256), (2, 2, 128)])
@pytest.mark.parametrize("bidir_all", [True, False])
def test_attention_with_image_blocks(dev, name, bi, H, Hkv, D, bidir_all):
    from spinf_serve_b200 import attention as A

    a, window = _arrays(name, bi)
    n = len(a["art"])
    q, k, v = _qkv(n, H, Hkv, D, 11)
    masks = A.stream_masks(a["art"], a["end"], a["pos"], window, dev, always_window=True, grp=a["grp"], bidir_all=bidir_all)
    real = a["art"] >= 0
    for kind, w in (("full_attention", None), ("sliding_attention", window)):
        out = A.tree_attention(q.to(dev), k.to(dev), v.to(dev), masks[kind], D**-0.5).cpu()
        g = a["grp"] if (bidir_all or w) else None
        ref = OA.tree_attention(q, k, v, a["art"], a["end"], a["pos"], D**-0.5, w, grp=g, grp_in_window=not bidir_all)
        err = (out.float() - ref)[real].abs()
        tol = 2.0**-7 * ref[real].abs() + 2e-3 * ref[real].abs().max()
        print(f"{name} {kind} H{H}/{Hkv} D{D} bidir_all={bidir_all}: max abs err {err.max():.3e}")
        assert bool((err <= tol).all())
        if g is not None:  # the image blocks matter: the causal rule alone gives another answer on the placeholders' rows
            causal = OA.tree_attention(q, k, v, a["art"], a["end"], a["pos"], D**-0.5, w)
            rows = a["grp"] >= 0
            assert float((causal - ref)[rows].abs().max()) > 10 * float(err.max())


# two layers, one sliding and one full, with a window that binds inside the prefixes
TINY = dict(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=512, window=64, layer_types=["sliding_attention", "full_attention"])


def _image_job(rng, cfg, n_prefix, span, n_prompts):
    prefix = rng.integers(5, cfg.vocab, n_prefix).tolist()
    prompts = [prefix + rng.integers(5, cfg.vocab, int(rng.integers(4, 12))).tolist() for _ in range(n_prompts)]
    tree = P.build_grouped_tree(prompts, [P.ReadPlan.build([[11], [12]]) for _ in prompts])
    g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    img = P.Image(span[1], (torch.randn((span[1], cfg.hidden), generator=g) * 0.5).to(torch.bfloat16))
    tree.media.append((span[0], img))
    return tree


@pytest.mark.parametrize("bidir_all", [True, False])
def test_stack_forward_with_an_image_in_the_prefix(dev, bidir_all):
    """two layers (one sliding, one full) of the bf16 scheme, so that the comparison with the oracle is not blurred by fp8 steps"""
    from oracle import gemma as OG
    from spinf_serve_b200 import scorer as S
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights

    ocfg, cfg = OG.GemmaConfig(**TINY), GemmaConfig(**TINY)
    rng = np.random.default_rng(21)
    W = OG.init_weights(ocfg, seed=4)
    Q = OG.quantize(W, "bf16")
    stack = GemmaStack(GemmaWeights.from_quantized(cfg, W, Q, dev, "bf16"), vision_bidir_all=bidir_all)
    pk = P.Packer(2048, 65536, align=True, min_stream=1024)
    list(pk.push(0, _image_job(rng, cfg, 300, (20, 200), 4)))
    list(pk.push(1, _image_job(rng, cfg, 150, (100, 40), 3)))
    (b,) = list(pk.flush())
    assert b.grp is not None and len(b.media) == 2
    h = S.forward_one(stack, b, dev)[0].float().cpu()
    media = [(s, o.embeds) for s, o in b.media]
    ref = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, scheme="bf16", grp=b.grp, bidir_all=bidir_all, media=media).float()
    real = b.art >= 0
    rel = float((h - ref)[real].pow(2).mean().sqrt() / ref[real].pow(2).mean().sqrt())
    plain = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, scheme="bf16", media=media).float()
    gap = float((plain - ref)[real].pow(2).mean().sqrt() / ref[real].pow(2).mean().sqrt())
    # the yardstick: the oracle against itself with one legitimate rounding change (P rounded to bf16 before P V, as the kernels do)
    exact = OA.tree_attention
    try:
        OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        alt = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, scheme="bf16", grp=b.grp, bidir_all=bidir_all, media=media).float()
    finally:
        OA.tree_attention = exact
    sens = float((alt - ref)[real].pow(2).mean().sqrt() / ref[real].pow(2).mean().sqrt())
    print(f"bidir_all={bidir_all}: hidden rms err / rms = {rel:.3e} (oracle's own rounding sensitivity {sens:.3e}); the causal mask alone differs by {gap:.3e}")
    assert rel < max(3 * sens, 1e-2) and gap > 10 * rel


def test_a_job_with_an_image_scores_the_same_alone_and_packed(dev):
    from spinf_serve_b200 import scorer as S
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights

    cfg = GemmaConfig(**TINY)
    stack = GemmaStack(GemmaWeights.random(cfg, seed=5, device=dev))
    trees = [_image_job(np.random.default_rng(30 + j), cfg, 260 + 90 * j, (10 + 50 * j, 150), 3) for j in range(3)]

    def hidden(items):
        pk = P.Packer(4096, 65536, align=True, min_stream=1024)
        for j, t in items:
            list(pk.push(j, t))
        (b,) = list(pk.flush())
        h = S.forward_one(stack, b, dev)[0]
        return {o.job_id: h[o.start : o.start + o.n_tokens].clone() for o in b.owners}

    packed = hidden(list(enumerate(trees)))
    for j, t in enumerate(trees):
        alone = hidden([(j, t)])
        assert torch.equal(alone[j], packed[j]), f"job {j}"
