"""Generates tests/golden/*.npz by running the REFERENCE's own host code (spinf_serve.packer, imported from a read-only checkout)
on seeded random inputs. The fixtures pin this repository's packer / tile descriptor / read geometry to the reference bit for bit;
they travel with the repository, the reference checkout does not. Re-run only when a new case is added:

    python tests/golden/make_golden.py /path/to/spinf-serve-checkout
"""

import gzip
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def random_job(rng, n_prefix, n_prompts, max_branch, vocab, multi_token, shared_stems):
    """prompts = shared prefix + (optional shared stem) + own tail; options: 2-5 per prompt, some with several tokens"""
    prefix = rng.integers(5, vocab, n_prefix).tolist()
    stems = [rng.integers(5, vocab, rng.integers(1, 6)).tolist() for _ in range(max(1, n_prompts // 3))]
    prompts, options = [], []
    for c in range(n_prompts):
        tail = rng.integers(5, vocab, rng.integers(1, max_branch + 1)).tolist()
        stem = stems[rng.integers(0, len(stems))] if shared_stems else []
        prompts.append(prefix + stem + tail)
        opts = []
        for _ in range(int(rng.integers(2, 6))):
            n = int(rng.integers(1, 4)) if multi_token else 1
            opts.append(rng.integers(5, 60, n).tolist())  # small range: lead-ins collide on purpose
        options.append(opts)
    return prompts, options


def batch_record(b):
    rec = {k: getattr(b, k) for k in ("ids", "pos", "seg", "art", "sel", "end", "prev")}
    rec["n_tokens"] = np.int64(b.n_tokens)
    rec["owner_start"] = np.array([o.start for o in b.owners], np.int64)
    rec["owner_rows"] = np.array([o.n_rows for o in b.owners], np.int64)
    rec["owner_tokens"] = np.array([o.n_tokens for o in b.owners], np.int64)
    rec["owner_prefix"] = np.array([o.prefix_len for o in b.owners], np.int64)
    rec["owner_job"] = np.array([o.job_id for o in b.owners], np.int64)
    return rec


def main(ref_root):
    sys.path.insert(0, ref_root)
    from spinf_serve import packer as R

    cases = {}
    meta = {}
    for seed, (grouped, align, window, multi, stems, budget) in enumerate(
        [
            (True, True, 64, True, True, 4096),
            (True, False, 64, True, True, 2048),
            (False, True, 256, True, False, 4096),
            (False, False, None, False, False, 1024),
            (True, True, 1024, False, False, 8192),
            (True, True, 32, True, True, 1024),
        ]
    ):
        rng = np.random.default_rng(100 + seed)
        jobs = []
        for j in range(int(rng.integers(3, 9))):
            pr, op = random_job(rng, int(rng.integers(1, 700)), int(rng.integers(1, 12)), 24, 500, multi, stems)
            jobs.append((pr, op))
        pk = R.Packer(budget, 65536, align=align, min_stream=1024 if align else 0)
        batches = []
        for j, (pr, op) in enumerate(jobs):
            if grouped:
                plans = [R.ReadPlan.build(o) for o in op]
                runs = R.split_grouped_trees(pr, plans, pk.budget)
            else:
                runs = R.split_trees(pr, op, pk.budget)
            for first, t in runs:
                batches += list(pk.push(j, t, window=4))  # job ids are ints here so they fit an array
        batches += list(pk.flush())
        name = f"pack{seed}"
        meta[name] = {"grouped": grouped, "align": align, "window": window, "budget": budget, "jobs": jobs, "n_batches": len(batches)}
        for bi, b in enumerate(batches):
            rec = batch_record(b)
            full, sliding = R.block_tables(b.art, b.end, b.pos, window, None, align)
            for tag, tab in (("full", full), ("sliding", sliding)):
                if tab is not None:
                    for nm, arr in zip(("pn", "pi", "fn", "fi"), tab):
                        rec[f"{tag}_{nm}"] = arr
            rec["has_sliding"] = np.bool_(sliding is not None)
            for k, v in rec.items():
                cases[f"{name}/b{bi}/{k}"] = v
    # trees / plans / tries as JSON (literal structures)
    rng = np.random.default_rng(7)
    structs = []
    for _ in range(12):
        pr, op = random_job(rng, int(rng.integers(0, 9)), int(rng.integers(1, 7)), 5, 30, True, True)
        t = R.build_tree(pr, op)
        plans = [R.ReadPlan.build(o) for o in op]
        g = R.build_grouped_tree(pr, plans)
        structs.append(
            {
                "prompts": pr,
                "options": op,
                "tree": {"prefix": t.prefix, "branches": t.branches, "reads": [list(r) for r in t.reads], "n_options": t.n_options},
                "plans": [
                    {"leadins": [list(x) for x in p.leadins], "row": p.entry_row.tolist(), "tok": p.entry_tok.tolist(), "opt": p.entry_opt.tolist(), "n_opts": p.n_opts, "n_rows": p.n_rows}
                    for p in plans
                ],
                "grouped": {"prefix": g.prefix, "branches": g.branches, "parents": g.parents, "prompt_rows": [[list(x) for x in r] for r in g.prompt_rows], "n_tokens": g.n_tokens},
            }
        )
    # the config-1 attention layout: 2 contents x (470-token trunk + 8 questions of 16 tokens), aligned
    rng = np.random.default_rng(0)
    pk = R.Packer(16384, 65536, align=True, min_stream=1024)
    for j in range(2):
        trunk = rng.integers(5, 262144, 470).tolist()
        prompts = [trunk + [1000 + 20 * j + q] + rng.integers(5, 262144, 15).tolist() for q in range(8)]
        plans = [R.ReadPlan.build([[11], [12]]) for _ in prompts]
        list(pk.push(j, R.build_grouped_tree(prompts, plans)))
    (b,) = list(pk.flush())
    rec = batch_record(b)
    full, sliding = R.block_tables(b.art, b.end, b.pos, 1024, None, True)
    for tag, tab in (("full", full), ("sliding", sliding)):
        for nm, arr in zip(("pn", "pi", "fn", "fi"), tab):
            rec[f"{tag}_{nm}"] = arr
    for k, v in rec.items():
        cases[f"cfg1/{k}"] = v
    # recurrent-layer plans (qwen.tree_plan, indexed path) of some of the batches above, with several option sets
    from spinf_serve.models.qwen35.qwen import tree_plan

    plans = {}
    plan_meta = []
    for name in ("pack0", "pack1", "pack4", "pack5", "cfg1"):
        keys = sorted({k.split("/")[1] for k in cases if k.startswith(name + "/b")}) if name != "cfg1" else [None]
        for bk in keys[:2]:
            base = f"{name}/{bk}/" if bk else f"{name}/"
            prev, art = cases[base + "prev"], cases[base + "art"]
            real = art >= 0
            n_real = int(real.sum())
            for vi, kw in enumerate(
                [
                    dict(),
                    dict(short=8, call_tokens=96),
                    dict(rows=(n_real + 127) // 128 * 128, short=16),
                    dict(keep=[int(x) for x in np.flatnonzero(real)[:: max(1, n_real // 5)]], short=4, call_tokens=40),
                ]
            ):
                pl = tree_plan(prev, real, "cpu", **kw)
                tag = f"{base}v{vi}/"
                plan_meta.append({"batch": base, "tag": tag, "kw": kw, "n_levels": len(pl.levels), "n_calls": [len(c) for c in pl.levels],
                                  "kinds": [[c.kind for c in calls] for calls in pl.levels], "n_keep": pl.n_keep, "n_segments": pl.n_segments})
                plans[tag + "conv"] = pl.conv.numpy()
                plans[tag + "seg_of_row"] = np.asarray(pl.seg_of_row)
                plans[tag + "seg_level"] = np.asarray(pl.seg_level)
                plans[tag + "seg_slot"] = np.asarray(pl.seg_slot)
                if pl.sidx is not None:
                    plans[tag + "sidx"] = pl.sidx.numpy()
                for li, calls in enumerate(pl.levels):
                    for ci, c in enumerate(calls):
                        plans[f"{tag}L{li}/C{ci}/idx"] = c.idx.numpy()
                        plans[f"{tag}L{li}/C{ci}/cu"] = c.cu_cpu.numpy()
                        if c.h0_idx is not None:
                            plans[f"{tag}L{li}/C{ci}/h0"] = c.h0_idx.numpy()
                        if c.ht_idx is not None:
                            plans[f"{tag}L{li}/C{ci}/ht"] = c.ht_idx.numpy()
    np.savez_compressed(os.path.join(HERE, "plan_golden.npz"), **plans)
    with gzip.open(os.path.join(HERE, "plan_golden.json.gz"), "wt") as f:
        json.dump(plan_meta, f)
    print(f"{len(plans)} plan arrays, {len(plan_meta)} plans")
    np.savez_compressed(os.path.join(HERE, "packer_golden.npz"), **cases)
    with gzip.open(os.path.join(HERE, "packer_golden.json.gz"), "wt") as f:
        json.dump({"meta": meta, "structs": structs}, f)
    print(f"{len(cases)} arrays, {len(structs)} structures")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the spinf-serve tree>")
    main(sys.argv[1])
