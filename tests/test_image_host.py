"""Streams whose shared prefixes carry images and audio, on CPU: the packer's Batch.grp / Batch.media and the tile lists with
image groups against golden fixtures made by the reference's own packer (tests/golden/make_image_golden.py, packer.py:367-374,
455-467,479,485), and the tile lists against a dense evaluation of the image mask rules (spinf_serve/scorer.py:178-198)."""

import json
import os

import numpy as np
import pytest

from oracle import attention as OA
from spinf_serve_b200 import packer as P

NPZ = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "image_golden.npz"))
META = json.loads(bytes(NPZ["meta"]).decode())


def _batches(name):
    m = META[name]
    pk = P.Packer(m["budget"], 65536, align=m["align"], min_stream=1024 if m["align"] else 0)
    out = []
    for j, job in enumerate(m["jobs"]):
        plans = [P.ReadPlan.build(o) for o in job["options"]]
        tree = P.build_grouped_tree(job["prompts"], plans)
        for off, kind, n in job["spans"]:
            if off + n <= len(tree.prefix):
                tree.media.append((off, P.Image(n) if kind == "image" else P.Audio(n)))
        out += list(pk.push(j, tree, window=4))
    out += list(pk.flush())
    return m, out


@pytest.mark.parametrize("name", sorted(META))
def test_batches_and_tables_with_images_equal_the_reference(name):
    m, batches = _batches(name)
    assert len(batches) == m["n_batches"]
    for bi, b in enumerate(batches):
        key = f"{name}/b{bi}/"
        for k in ("ids", "pos", "seg", "art", "sel", "end", "prev"):
            got, want = getattr(b, k), NPZ[key + k]
            assert got.dtype == want.dtype and np.array_equal(got, want), (name, bi, k)
        assert (b.grp is not None) == bool(NPZ[key + "has_grp"])
        if b.grp is not None:
            assert b.grp.dtype == np.int32 and np.array_equal(b.grp, NPZ[key + "grp"])
        assert [s for s, _ in b.media] == NPZ[key + "media_start"].tolist()
        assert [o.n_tokens for _, o in b.media] == NPZ[key + "media_n"].tolist()
        assert [isinstance(o, P.Image) for _, o in b.media] == NPZ[key + "media_image"].tolist()
        full, sliding = P.block_tables(b.art, b.end, b.pos, m["window"], b.grp, m["always_window"])
        assert (sliding is not None) == bool(NPZ[key + "has_sliding"])
        for tag, tab in (("full", full), ("sliding", sliding)):
            if tab is not None:
                for nm, arr in zip(("pn", "pi", "fn", "fi"), tab):
                    assert np.array_equal(arr, NPZ[f"{key}{tag}_{nm}"]), (name, bi, tag, nm)


@pytest.mark.parametrize("name", sorted(META))
def test_tile_lists_cover_the_image_masks(name):
    """every visible pair of the dense rule lies in a visited tile, a tile flagged full / no-mask has every pair visible, and a
    query block's list is ascending, for both ways a model places the images' two-way blocks"""
    m, batches = _batches(name)
    later = 0
    for b in batches:
        n, nb = b.length, b.length // P.BLOCK
        for window in (None, m["window"]) if m["window"] else (None,):
            td = P.tile_desc(b.art, b.end, b.pos, window, b.grp)
            for bidir_all in (True, False):
                g = b.grp if (bidir_all or window) else None
                dense = OA.dense_mask(b.art, b.end, b.pos, window, g, grp_in_window=not bidir_all)
                tiles = dense.reshape(nb, P.BLOCK, nb, P.BLOCK).any(axis=(1, 3))
                for i in range(nb):
                    sl = slice(td.offsets[i], td.offsets[i + 1])
                    js, fl = td.blocks[sl], td.flags[sl]
                    assert np.all(np.diff(js) > 0)
                    assert set(np.nonzero(tiles[i])[0].tolist()) <= set(js.tolist()), (name, window, bidir_all, i)
                    for j, f in zip(js.tolist(), fl.tolist()):
                        if f & 3:
                            assert dense[i * P.BLOCK : (i + 1) * P.BLOCK, j * P.BLOCK : (j + 1) * P.BLOCK].all()
                    later += int((js > i).sum())
    print(f"{name}: {later} visited tiles lie after the diagonal")


def test_text_only_streams_are_unchanged_by_the_image_entry_points():
    """grp = None and a grp of all -1 give the tile lists of the text-only builder"""
    rng = np.random.default_rng(3)
    pk = P.Packer(4096, 65536, align=True, min_stream=1024)
    for j in range(3):
        prefix = rng.integers(5, 500, int(rng.integers(100, 700))).tolist()
        prompts = [prefix + rng.integers(5, 500, 9).tolist() for _ in range(5)]
        list(pk.push(j, P.build_grouped_tree(prompts, [P.ReadPlan.build([[7], [8]]) for _ in prompts])))
    (b,) = list(pk.flush())
    assert b.grp is None and b.media == []
    for window in (None, 64):
        a = P.tile_desc(b.art, b.end, b.pos, window)
        c = P.tile_desc(b.art, b.end, b.pos, window, np.full(b.length, -1, np.int32))
        assert np.array_equal(a.offsets, c.offsets) and np.array_equal(a.blocks, c.blocks) and np.array_equal(a.flags, c.flags)


def test_media_outside_the_prefix_is_refused():
    t = P.build_grouped_tree([[1, 2, 3, 4, 5], [1, 2, 3, 9, 9]], [P.ReadPlan.build([[7], [8]])] * 2)
    t.media.append((1, P.Image(5)))
    pk = P.Packer(1024, 65536, align=True, min_stream=0)
    with pytest.raises(ValueError, match="shared prefix"):
        list(pk.push(0, t)) + list(pk.flush())
