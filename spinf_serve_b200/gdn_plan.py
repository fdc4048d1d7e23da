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
    fused: object | None = None   # FusedSchedule: the same plan laid out for the one-launch-per-level kernels (this build's)


UNIT_WORDS = 12
UF_UPDATE, UF_PARENT = 1, 2
LIGHT_UNITS = 16  # units per CTA in a group of read-only children


@dataclass
class FusedSchedule:
    """The plan as the fused kernels read it (spinf_gdn_tree_prep / spinf_gdn_tree_scan). Plan order = the segments one after the
    other in stream order; every segment is cut into chunks of at most 64 tokens. Per level the segments are grouped by parent: a
    group's CTA holds the parent's state while it walks the group's units. A child that only reads that state (one chunk, no state
    to keep) is "light": up to four light siblings share a 64-row unit at 16-row-aligned offsets. Any other child is "heavy": one
    unit per chunk, each updating the state, the last one storing it where the child's own children will read it."""

    plan_tokens: int
    row_of: object      # int64 [plan_tokens]
    chunk_p0: object    # int32 [n_chunks]
    chunk_len: object   # int32 [n_chunks]
    levels: list        # per level: (grp_parent int32 [G], grp_ubeg int32 [G + 1], units int32 [U, 12], unit_rows int32 [U, 4, 64])
    n_keep: list        # state slots per level
    workspace: object = None


def fused_schedule(starts, lens, parent_seg, depth, keeps, slot, row_of):
    """host arrays of the fused kernels from the segment structure tree_plan derives (all numpy)"""
    n_seg = len(starts)
    row_of = np.asarray(row_of, np.int64)
    if len(row_of) and int(row_of.max()) >= 2**31:
        raise ValueError("fused_schedule: stream rows must fit 31 bits")
    pt0 = np.concatenate(([0], np.cumsum(lens)))[:-1] if n_seg else np.zeros(0, np.int64)
    n_chunks_seg = (lens + 63) // 64
    seg_of_chunk = np.repeat(np.arange(n_seg), n_chunks_seg)
    first_chunk = np.concatenate(([0], np.cumsum(n_chunks_seg)))[:-1] if n_seg else np.zeros(0, np.int64)
    t0 = (np.arange(len(seg_of_chunk)) - first_chunk[seg_of_chunk]) * 64
    chunk_p0 = (pt0[seg_of_chunk] + t0).astype(np.int32)
    chunk_len = np.minimum(64, lens[seg_of_chunk] - t0).astype(np.int32)
    levels = []
    for d in range(int(depth.max()) + 1 if n_seg else 0):
        level = np.flatnonzero(depth == d)
        # groups: siblings share a parent; roots are groups of their own (stream order is kept inside a group)
        key = np.where(parent_seg[level] >= 0, parent_seg[level], -1 - level)
        order = np.argsort(key, kind="stable")
        level, key = level[order], key[order]
        bounds = np.concatenate(([0], np.flatnonzero(np.diff(key)) + 1, [len(level)]))
        grp_parent, grp_ubeg, units = [], [0], []
        for a, b in zip(bounds[:-1], bounds[1:]):
            ps = parent_seg[level[a]]
            pslot = int(slot[ps]) if ps >= 0 else -1
            first_unit = len(units)
            open_unit = None  # the light unit being filled: [pieces, rows used]
            for sgm in level[a:b]:
                L, p0 = int(lens[sgm]), int(pt0[sgm])
                if L <= 64 and not keeps[sgm]:
                    need = (L + 15) // 16 * 16
                    if open_unit is None or len(open_unit[0]) == 4 or open_unit[1] + need > 64:
                        open_unit = [[], 0]
                        units.append(open_unit)
                    open_unit[0].append((p0, L))
                    open_unit[1] += need
                else:
                    open_unit = None
                    n = (L + 63) // 64
                    for c in range(n):
                        flags = UF_UPDATE | (UF_PARENT if c == 0 else 0)
                        store = int(slot[sgm]) if (c == n - 1 and keeps[sgm]) else -1
                        units.append((flags, store, (p0 + 64 * c, min(64, L - 64 * c))))
            # a group whose children all only read the parent's state has no order to keep: it is cut into CTAs of at most
            # LIGHT_UNITS units (each reads the parent's state once more, from L2), so that many leaves do not queue behind one CTA
            n_units = len(units) - first_unit
            if n_units > LIGHT_UNITS and all(isinstance(u, list) for u in units[first_unit:]):
                for cut in range(first_unit + LIGHT_UNITS, len(units), LIGHT_UNITS):
                    grp_parent.append(pslot)
                    grp_ubeg.append(cut)
            grp_parent.append(pslot)
            grp_ubeg.append(len(units))
        words = np.zeros((len(units), UNIT_WORDS), np.int32)
        rows = np.zeros((len(units), 4, 64), np.int32)  # per unit row: plan token (-1: none), stream row, the piece's last token, its first row
        rows[:, 0] = -1
        for i, u in enumerate(units):
            if isinstance(u, list):
                words[i, 0], words[i, 1], words[i, 2] = len(u[0]), UF_PARENT, -1
                pieces = u[0]
            else:
                words[i, 0], words[i, 1], words[i, 2] = 1, u[0], u[1]
                pieces = [u[2]]
            off = 0
            for j, (p0, L) in enumerate(pieces):
                words[i, 4 + 2 * j], words[i, 5 + 2 * j] = p0, L
                rows[i, 0, off : off + L] = np.arange(p0, p0 + L)
                rows[i, 1, off : off + L] = row_of[p0 : p0 + L]
                rows[i, 2, off : off + L] = p0 + L - 1
                rows[i, 3, off : off + L] = off
                off += (L + 15) // 16 * 16
        levels.append((np.asarray(grp_parent, np.int32), np.asarray(grp_ubeg, np.int32), words, rows))
    return FusedSchedule(int(lens.sum()) if n_seg else 0, row_of, chunk_p0, chunk_len, levels, [])


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

    all_rows = token_rows(np.arange(n_seg)) if n_seg else np.zeros(0, np.int64)
    fused = fused_schedule(starts, lens, parent_seg, depth, keeps, slot, all_rows)
    fused.n_keep = list(n_keep)
    fused.row_of = dev(fused.row_of)
    fused.chunk_p0, fused.chunk_len = dev(fused.chunk_p0), dev(fused.chunk_len)
    fused.levels = [tuple(dev(x) for x in lv) for lv in fused.levels]

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
    return TreePlan(dev(conv), levels, n_seg, path, n_keep, rows, sidx, seg_rows, depth, slot, None, fused)
