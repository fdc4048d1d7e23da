"""Generates tests/golden/image_golden.npz by running the REFERENCE's own packer (spinf_serve.packer, imported from a read-only
checkout) on seeded jobs whose shared prefixes carry images and audio: the packed arrays with Batch.grp, and block_tables with the
grp argument (later key blocks of an image, blocks kept past the window). The fixture pins this repository's packer and tile
descriptor for streams with images to the reference bit for bit. Re-run only when a case is added:

    python tests/golden/make_image_golden.py /path/to/spinf-serve-checkout
"""

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# (align, window, always_window, budget, seed)
CASES = [(True, 64, True, 4096, 0), (False, 256, False, 2048, 1), (True, 1024, True, 8192, 2), (True, None, False, 4096, 3), (False, 96, False, 4096, 4)]


def random_job(rng, vocab=500):
    """-> (prompt ids, option ids, media spans [(offset, kind, n)]) with the spans inside the shared prefix, not overlapping"""
    n_prefix = int(rng.integers(150, 900))
    prefix = rng.integers(5, vocab, n_prefix).tolist()
    spans, at = [], int(rng.integers(0, 40))
    for _ in range(int(rng.integers(1, 4))):
        n = int(rng.integers(8, 300))
        if at + n > n_prefix:
            break
        spans.append((at, "image" if rng.random() < 0.75 else "audio", n))
        at += n + int(rng.integers(0, 120))
    prompts, options = [], []
    for _ in range(int(rng.integers(1, 9))):
        prompts.append(prefix + rng.integers(5, vocab, int(rng.integers(1, 20))).tolist())
        options.append([rng.integers(5, 60, int(rng.integers(1, 3))).tolist() for _ in range(int(rng.integers(2, 5)))])
    return prompts, options, spans


def main(ref_root):
    sys.path.insert(0, ref_root)
    from spinf_serve import media as M
    from spinf_serve import packer as R

    out, meta = {}, {}
    for align, window, always, budget, seed in CASES:
        rng = np.random.default_rng(500 + seed)
        pk = R.Packer(budget, 65536, align=align, min_stream=1024 if align else 0)
        jobs, batches = [], []
        for j in range(int(rng.integers(2, 6))):
            pr, op, spans = random_job(rng)
            jobs.append({"prompts": pr, "options": op, "spans": spans})
            plans = [R.ReadPlan.build(o) for o in op]
            tree = R.build_grouped_tree(pr, plans)
            for off, kind, n in spans:
                if off + n <= len(tree.prefix):
                    obj = M.Image(np.zeros((n, 1), np.float32), np.zeros((n, 2), np.int64)) if kind == "image" else M.Audio(np.zeros((n, 1), np.float32))
                    tree.media.append((off, obj))
            batches += list(pk.push(j, tree, window=4))
        batches += list(pk.flush())
        name = f"img{seed}"
        meta[name] = {"align": align, "window": window, "always_window": always, "budget": budget, "jobs": jobs, "n_batches": len(batches)}
        for bi, b in enumerate(batches):
            rec = {k: getattr(b, k) for k in ("ids", "pos", "seg", "art", "sel", "end", "prev")}
            rec["has_grp"] = np.bool_(b.grp is not None)
            if b.grp is not None:
                rec["grp"] = b.grp
            rec["media_start"] = np.array([s for s, _ in b.media], np.int64)
            rec["media_n"] = np.array([o.n_tokens for _, o in b.media], np.int64)
            rec["media_image"] = np.array([isinstance(o, M.Image) for _, o in b.media], np.bool_)
            full, sliding = R.block_tables(b.art, b.end, b.pos, window, b.grp, always)
            for tag, tab in (("full", full), ("sliding", sliding)):
                if tab is not None:
                    for nm, arr in zip(("pn", "pi", "fn", "fi"), tab):
                        rec[f"{tag}_{nm}"] = arr
            rec["has_sliding"] = np.bool_(sliding is not None)
            for k, v in rec.items():
                out[f"{name}/b{bi}/{k}"] = v
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "image_golden.npz"), **out)
    print(f"wrote image_golden.npz: {len(out)} arrays, {sum(m['n_batches'] for m in meta.values())} batches")


if __name__ == "__main__":
    main(sys.argv[1])
