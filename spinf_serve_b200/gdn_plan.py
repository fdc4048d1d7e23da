"""Host-side plan of the recurrent (Gated DeltaNet) layers over a packed stream of tries, interface-compatible with the reference's
tree_plan (spinf_serve/models/qwen35/qwen.py:125-276, the "indexed" path): the stream's path structure (Batch.prev) is cut into
segments, segments are grouped by depth into levels, and every level is a few kernel calls whose segments start from the state
their parent segment left behind (h0_idx) and leave their own final state where a child will need it (ht_idx).

A segment starts at a real token whose path predecessor is not the token just before it in the stream, or is a fork (a token with
several children); it runs to the next start or pad. conv[t] = the token's path predecessors 3, 2, 1 back and itself (index T, or
`rows` for compact rows = "none": a zero row), the taps of the layer's 4-wide path convolution."""

from dataclasses import dataclass

import numpy as np


@dataclass
class Call:
    idx: object      # [n] int64 rows of the call's tokens, segments back to back (device)
    cu: object       # [segs + 1] int64 cumulative lengths (device)
    cu_cpu: object   # the same on the host
    parent: object | None
    keep: bool
    kind: str = "chunked"            # chunked (longer than `short`) | recurrent
    h0_idx: object | None = None     # [segs] row of the previous level's states (-1 = zero state), None at level 0
    ht_idx: object | None = None     # [segs] row of this level's states to write (-1 = none), None when no segment keeps one
    table: object | None = None      # the call's 64-token chunk table (chunked calls), built on first use


@dataclass
class TreePlan:
    conv: object
    levels: list
    n_segments: int
    path: str = "indexed"
    n_keep: list | None = None
    rows: int | None = None
    sidx: object | None = None
    seg_of_row: object | None = None
    seg_level: object | None = None
    seg_slot: object | None = None
    cap: dict | None = None


def tree_plan(prev, real, device, max_init: int = 96, path: str = "indexed", short: int = 64, rows: int | None = None, keep=None,
              call_tokens: int = 8192) -> TreePlan:
    import torch

    if path != "indexed":
        raise ValueError("only the indexed recurrent path is built (the levels path runs a third-party chunk kernel per call)")
    prev = np.asarray(prev, np.int64)
    real = np.asarray(real, bool)
    T = len(prev)
    pos = np.arange(T)
    real_idx = np.flatnonzero(real)
    to_row = None  # stream position -> compact row; T (no tap) -> rows
    if rows is not None:
        if len(real_idx) > rows:
            raise ValueError(f"tree_plan: {len(real_idx)} real tokens do not fit {rows} compact rows")
        to_row = np.full(T + 1, rows, np.int64)
        to_row[real_idx] = np.arange(len(real_idx))

    has_prev = prev >= 0
    safe_prev = np.where(has_prev, prev, 0)
    children = np.bincount(prev[has_prev], minlength=T)
    fork_parent = has_prev & (children[safe_prev] > 1)
    is_start = real & (~has_prev | (prev != pos - 1) | fork_parent)
    starts = np.flatnonzero(is_start)
    n_seg = len(starts)
    seg = np.full(T, -1, np.int64)
    seg[real] = (np.cumsum(is_start) - 1)[real]
    lens = np.bincount(seg[real], minlength=n_seg)
    parent_seg = np.where(prev[starts] >= 0, seg[np.maximum(prev[starts], 0)], -1)
    depth = np.zeros(n_seg, np.int64)
    for s in range(n_seg):  # a parent precedes its children in the stream (pre-order)
        if parent_seg[s] >= 0:
            depth[s] = depth[parent_seg[s]] + 1
    keeps = np.zeros(n_seg, bool)
    keeps[parent_seg[parent_seg >= 0]] = True
    if keep is not None:
        for s in keep:
            if real[s]:
                keeps[seg[s]] = True

    def dev(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(device, non_blocking=True)

    def token_rows(part):
        offs = np.repeat(starts[part] - np.concatenate(([0], np.cumsum(lens[part])[:-1])), lens[part])
        t = np.arange(int(lens[part].sum())) + offs
        return t if to_row is None else to_row[t]

    levels, n_keep = [], []
    slot = np.full(n_seg, -1, np.int64)
    for d in range(int(depth.max()) + 1 if n_seg else 0):
        level = np.flatnonzero(depth == d)
        kept = level[keeps[level]]
        slot[kept] = np.arange(len(kept))
        n_keep.append(len(kept))
        calls = []
        for kind, group in (("chunked", level[lens[level] > short]), ("recurrent", level[lens[level] <= short])):
            if not len(group):
                continue
            parts = [group]
            if kind == "chunked" and lens[group].sum() > call_tokens:  # bound the tokens of one call
                parts, run, acc = [], [], 0
                for s in group:
                    if run and acc + lens[s] > call_tokens:
                        parts.append(np.array(run))
                        run, acc = [], 0
                    run.append(s)
                    acc += lens[s]
                parts.append(np.array(run))
            for part in parts:
                cu = torch.from_numpy(np.concatenate(([0], np.cumsum(lens[part]))))
                h0 = None if d == 0 else dev(np.where(parent_seg[part] >= 0, slot[np.maximum(parent_seg[part], 0)], -1))
                ht = dev(np.where(keeps[part], slot[part], -1)) if keeps[part].any() else None
                calls.append(Call(dev(token_rows(part)), cu.to(device, non_blocking=True), cu, None, False, kind, h0, ht))
        levels.append(calls)

    conv = np.empty((T, 4), np.int64)
    conv[:, 3] = pos
    p = np.where(real, prev, -1)
    for j in (2, 1, 0):
        conv[:, j] = np.where(p >= 0, p, T)
        p = np.where(p >= 0, prev[np.maximum(p, 0)], -1)
    sidx, seg_rows = None, seg
    if to_row is not None:
        compact = np.full((rows, 4), rows, np.int64)
        compact[: len(real_idx)] = to_row[conv[real_idx]]
        conv = compact
        sidx = dev(real_idx)
        seg_rows = np.full(rows, -1, np.int64)
        seg_rows[: len(real_idx)] = seg[real_idx]
    return TreePlan(dev(conv), levels, n_seg, path, n_keep, rows, sidx, seg_rows, depth, slot)
