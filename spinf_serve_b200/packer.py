"""Packed-stream layout of the scoring path, interface-compatible with spinf_serve/packer.py (same class names, fields, argument
meaning and errors), written for the B200 pipeline: the per-job arrays are produced with vectorised numpy instead of per-branch
loops, and the attention's tile descriptor comes from the C-ABI host function instead of an O(nb^2) interpreted loop.

A job is one content with several prompts; the prompts' longest common token prefix (the trunk) is laid out once, each prompt
continues as a branch that sees the trunk, its ancestors and itself (reference: packer.py:1-14). Grouped jobs lay a token trie
out in pre-order, so a token's descendants are the contiguous run that ends at Batch.end[token] (packer.py:141-185, 252-272).

Reference behaviour mirrored here, by symbol:
    build_tree            packer.py:38-64        ReadPlan.build        packer.py:81-104
    trie_branches         packer.py:141-185      build_grouped_tree    packer.py:188-198
    split_grouped_trees   packer.py:201-215      split_trees           packer.py:218-233
    Packer                packer.py:275-423      block_tables          packer.py:426-491
Media in the shared prefix (GroupedTree.media, packer.py:114-117,367-374): the packer records where each item's placeholders lie
(Batch.media) and which image every placeholder belongs to (Batch.grp: an image's placeholders attend to each other both ways).
Decoding images / audio and the towers that embed them are outside this path: Image / Audio below carry the placeholder count and,
for the stacks, the rows of input embeddings the caller computed.
"""

import ctypes
from dataclasses import dataclass, field

import numpy as np

BLOCK = 128  # stream block size: streams are multiples of it, aligned jobs start on it


def _round_up(n: int) -> int:
    return -(-n // BLOCK) * BLOCK


def _common_prefix(seqs) -> int:
    """length of the longest common prefix, leaving every sequence at least one token of its own"""
    if not seqs:
        raise ValueError("a job needs at least one prompt")
    limit = min(len(s) for s in seqs) - 1
    first = seqs[0]
    p = 0
    while p < limit:
        t = first[p]
        if any(s[p] != t for s in seqs):
            break
        p += 1
    return p


# ------------------------------------------------------------------------------------------------ trees (v0 format)
@dataclass
class Tree:
    prefix: list
    branches: list
    reads: list  # (branch index, offset in the branch, target token id, prompt index, option index)
    n_options: list

    @property
    def n_tokens(self) -> int:
        return len(self.prefix) + sum(len(b) for b in self.branches)


def build_tree(prompt_ids, option_ids) -> Tree:
    """one branch per prompt plus one per distinct multi-token lead-in; token j of an option is read at the position of token
    j-1, on the branch extended by the option's leading tokens"""
    p = _common_prefix(prompt_ids)
    if len(prompt_ids) != len(option_ids):
        raise ValueError("zip() argument 2 is shorter than argument 1" if len(option_ids) < len(prompt_ids) else "zip() argument 2 is longer than argument 1")
    branches, reads = [], []
    for c, (ids, options) in enumerate(zip(prompt_ids, option_ids)):
        own = list(ids[p:])
        branch_of = {(): len(branches)}
        branches.append(own)
        last = len(own) - 1
        for side, toks in enumerate(options):
            if not toks:
                raise ValueError(f"prompt {c}: option {side} is empty")
            lead = tuple(toks[:-1])
            reads.append((branch_of[()], last, toks[0], c, side))
            if lead:
                b = branch_of.get(lead)
                if b is None:
                    b = branch_of[lead] = len(branches)
                    branches.append(own + list(lead))
                reads.extend((b, last + j, toks[j], c, side) for j in range(1, len(toks)))
    return Tree(list(prompt_ids[0][:p]), branches, reads, [len(o) for o in option_ids])


# ------------------------------------------------------------------------------------------------ read plans / grouped trees
@dataclass(eq=False)
class ReadPlan:
    """vectorised read of a prompt's options: row 0 is the prompt's last token; each distinct lead-in (option[:-1]) adds one row
    per lead-in token; entry e adds log P(entry_tok[e]) at row entry_row[e] to option entry_opt[e]"""

    leadins: list
    entry_row: np.ndarray
    entry_tok: np.ndarray
    entry_opt: np.ndarray
    n_opts: int
    n_rows: int

    @classmethod
    def build(cls, option_ids) -> "ReadPlan":
        first_row = {}
        rows, toks, opts = [], [], []
        n_rows = 1
        for o, t in enumerate(option_ids):
            if not t:
                raise ValueError(f"option {o} is empty")
            rows.append(0)
            toks.append(t[0])
            opts.append(o)
            if len(t) == 1:
                continue
            lead = tuple(t[:-1])
            r0 = first_row.get(lead)
            if r0 is None:
                r0 = first_row[lead] = n_rows
                n_rows += len(lead)
            rows.extend(range(r0, r0 + len(t) - 1))
            toks.extend(t[1:])
            opts.extend([o] * (len(t) - 1))
        return cls(list(first_row), np.array(rows, np.int64), np.array(toks, np.int64), np.array(opts, np.int64), len(option_ids), n_rows)


@dataclass(eq=False)
class Image:
    """what the packed stream needs of an image in the shared prefix (the counterpart of media.Image, spinf_serve/media.py:41-50):
    the number of placeholder tokens and their input embeddings [n_tokens, hidden] bf16 (None: the ids' own embeddings stay)"""

    n_tokens: int
    embeds: object = None


@dataclass(eq=False)
class Audio:
    """the counterpart of media.Audio (spinf_serve/media.py:52-59): placeholders that attend causally, as text"""

    n_tokens: int
    embeds: object = None


def _is_image(obj) -> bool:
    return isinstance(obj, Image) or type(obj).__name__ == "Image"


@dataclass
class GroupedTree:
    prefix: list
    branches: list
    prompt_rows: list  # per prompt: (branch, offset) of each read row, in its plan's row order
    plans: list
    media: list = field(default_factory=list)
    xbranches: list = field(default_factory=list)
    parents: list = field(default_factory=list)  # branch a branch continues (-1: the prefix); empty = all continue the prefix
    aligned: list = field(default_factory=list)  # branches that start a query group on a BLOCK boundary (job-relative)

    @property
    def n_tokens(self) -> int:
        n = len(self.prefix)
        starts_group = set(self.aligned)
        for b, br in enumerate(self.branches):
            if b in starts_group:
                n = _round_up(n)
            n += len(br)
        return n


def trie_branches(suffixes, plans):
    """suffixes (each non-empty) and, under each suffix, its plan's lead-ins, merged into one token trie; -> (branches in
    pre-order, parents, prompt_rows). A branch is a maximal chain of trie nodes with a single child each."""
    if len(suffixes) != len(plans):
        raise ValueError("zip() argument 2 is shorter than argument 1" if len(plans) < len(suffixes) else "zip() argument 2 is longer than argument 1")
    child_of = {}        # (node, token) -> node
    kids = [[]]          # children of each node in insertion order; node 0 = end of the shared prefix
    token = [-1]

    def descend(node, seq, out):
        for t in seq:
            nxt = child_of.get((node, t))
            if nxt is None:
                nxt = child_of[(node, t)] = len(kids)
                kids[node].append(nxt)
                kids.append([])
                token.append(t)
            node = nxt
            out.append(node)
        return node

    read_nodes = []
    for suf, plan in zip(suffixes, plans):
        path = []
        tip = descend(0, suf, path)  # IndexError-free: an empty suffix leaves tip = 0, refused below
        if not path:
            raise IndexError("list index out of range")
        nodes = [tip]
        for lead in plan.leadins:
            descend(tip, lead, nodes)
        read_nodes.append(nodes)

    where = [(-1, -1)] * len(kids)
    branches, parents = [], []
    todo = [(n, -1) for n in reversed(kids[0])]
    while todo:
        node, parent = todo.pop()
        b = len(branches)
        chain = []
        while True:
            where[node] = (b, len(chain))
            chain.append(token[node])
            if len(kids[node]) != 1:
                break
            node = kids[node][0]
        branches.append(chain)
        parents.append(parent)
        todo.extend((n, b) for n in reversed(kids[node]))
    return branches, parents, [[where[n] for n in nodes] for nodes in read_nodes]


def build_grouped_tree(prompt_ids, plans) -> GroupedTree:
    p = _common_prefix(prompt_ids)
    branches, parents, prompt_rows = trie_branches([list(x[p:]) for x in prompt_ids], plans)
    return GroupedTree(list(prompt_ids[0][:p]), branches, prompt_rows, list(plans), parents=parents)


def _split(n_prompts, make, budget):
    """contiguous runs of prompts whose tree fits the budget, found by halving (each run re-sends the prefix)"""
    done = []
    todo = [(0, n_prompts)]
    while todo:
        a, b = todo.pop()
        t = make(a, b)
        if t.n_tokens <= budget:
            done.append((a, t))
        elif b - a == 1:
            raise ValueError(f"prompt {a} alone is {t.n_tokens} tokens, over the budget {budget}")
        else:
            mid = (a + b) // 2
            todo.append((mid, b))
            todo.append((a, mid))
    done.sort(key=lambda it: it[0])
    return done


def split_grouped_trees(prompt_ids, plans, budget):
    return _split(len(prompt_ids), lambda a, b: build_grouped_tree(prompt_ids[a:b], plans[a:b]), budget)


def split_trees(prompt_ids, option_ids, budget):
    return _split(len(prompt_ids), lambda a, b: build_tree(prompt_ids[a:b], option_ids[a:b]), budget)


# ------------------------------------------------------------------------------------------------ batches
@dataclass
class Owner:
    job_id: object
    n_rows: int
    n_tokens: int
    plan: list  # (row, target id, prompt index, option index); empty for a grouped job
    n_options: list
    row_start: np.ndarray | None = None
    plans: list | None = None
    start: int = 0
    prefix_len: int = 0
    xbranches: list = field(default_factory=list)


@dataclass
class Batch:
    ids: np.ndarray   # [N] int64
    pos: np.ndarray   # [N] int32, restarts at the prefix length (+ ancestors) for every branch
    seg: np.ndarray   # [N] int32: 0 prefix, k branch k, -1 pad
    art: np.ndarray   # [N] int32: job slot in the stream, -1 pad
    sel: np.ndarray   # read positions, int64
    owners: list
    n_tokens: int
    media: list = field(default_factory=list)
    grp: np.ndarray | None = None
    end: np.ndarray | None = None   # [N] int32: exclusive end of the token's subtree, -1 pad
    prev: np.ndarray | None = None  # [N] int64: previous token on the token's path, -1 for a job's first token and pads

    @property
    def length(self) -> int:
        return len(self.ids)


class Packer:
    """first-fit-decreasing packing of jobs into streams of at most `budget` tokens; align = every job starts on a BLOCK boundary
    (so a job's attention tiles do not depend on its neighbours), padded to at least min_stream tokens"""

    def __init__(self, budget: int, max_tokens: int | None = None, align: bool = False, min_stream: int = 0, cost=None, cost_budget: int = 0):
        self.budget = _round_up(budget)
        self.max_tokens = max(self.budget, (max_tokens or 0) + BLOCK - 1) // BLOCK * BLOCK
        self.align = align
        self.min_stream = min(self.budget, _round_up(min_stream)) if align else 0
        self.cost, self.cost_budget = cost, cost_budget
        self.buf = []

    def push(self, job_id, tree, window: int = 96):
        n = tree.n_tokens
        if n > self.max_tokens:
            raise ValueError(f"job {job_id}: {n} tokens exceed the maximum {self.max_tokens}")
        if n > self.budget:  # a long document runs alone, at once
            yield self._pack([(job_id, tree)], self._length(n))
            return
        self.buf.append((job_id, tree))
        if len(self.buf) >= window:
            yield from self._flush(final=False)

    def flush(self):
        yield from self._flush(final=True)

    def _length(self, n: int) -> int:
        return max(_round_up(n), self.min_stream)

    def _size(self, tree) -> int:
        return _round_up(tree.n_tokens) if self.align else tree.n_tokens

    def _flush(self, final: bool):
        order = sorted(range(len(self.buf)), key=lambda i: -self.buf[i][1].n_tokens)  # stable, as sorted() on the items is
        fill, cost, members = [], [], []
        for i in order:
            item = self.buf[i]
            n = self._size(item[1])
            c = self.cost(item[1]) if self.cost is not None else 0
            for b in range(len(fill)):
                if fill[b] + n <= self.budget and (c == 0 or cost[b] + c <= self.cost_budget):
                    fill[b] += n
                    cost[b] += c
                    members[b].append(item)
                    break
            else:
                fill.append(n)
                cost.append(c)
                members.append([item])
        bins = list(range(len(fill)))
        self.buf = []
        if not final and len(bins) > 1:
            bins.sort(key=lambda b: -fill[b])  # the least full stream waits for the next window
            self.buf = members[bins.pop()]
        for b in bins:
            yield self._pack(members[b], self._length(fill[b]))

    def _pack(self, items, n: int) -> Batch:
        ids = np.zeros(n, np.int64)
        pos = np.zeros(n, np.int32)
        seg = np.full(n, -1, np.int32)
        art = np.full(n, -1, np.int32)
        end = np.full(n, -1, np.int32)
        prev = np.full(n, -1, np.int64)
        sel_parts, owners = [], []
        media, grp = [], None
        n_sel = real = 0
        cursor = 0
        for slot, (jid, t) in enumerate(items):
            grouped = isinstance(t, GroupedTree)
            s0 = cursor
            P = len(t.prefix)
            for off, obj in getattr(t, "media", None) or ():
                if off + obj.n_tokens > P:
                    raise ValueError("media must lie in the shared prefix")
                media.append((s0 + off, obj))
                if _is_image(obj):
                    if grp is None:
                        grp = np.full(n, -1, np.int32)
                    grp[s0 + off : s0 + off + obj.n_tokens] = len(media)
            nb = len(t.branches)
            lens = np.fromiter((len(b) for b in t.branches), np.int64, nb)
            parents = np.asarray(getattr(t, "parents", None) or [-1] * nb, np.int64)
            group_heads = set(getattr(t, "aligned", ()))
            # depth below the prefix and subtree sizes: parents precede children (pre-order)
            depth = np.zeros(nb, np.int64)
            for b in range(nb):
                if parents[b] >= 0:
                    depth[b] = depth[parents[b]] + lens[parents[b]]
            size = lens.copy()
            for b in range(nb - 1, -1, -1):
                if parents[b] >= 0:
                    size[parents[b]] += size[b]
            # start of each branch in the stream (query groups start on a block of the job)
            start = np.empty(nb, np.int64)
            k = s0 + P
            if group_heads:
                for b in range(nb):
                    if b in group_heads:
                        k = s0 + _round_up(k - s0)
                    start[b] = k
                    k += lens[b]
            elif nb:
                start[:] = k + np.concatenate(([0], np.cumsum(lens[:-1])))
                k += int(lens.sum())
            job_end = k
            # trunk
            ids[s0 : s0 + P] = t.prefix
            pos[s0 : s0 + P] = np.arange(P, dtype=np.int32)
            seg[s0 : s0 + P] = 0
            art[s0 : s0 + P] = slot
            end[s0 : s0 + P] = job_end
            prev[s0 + 1 : s0 + P] = np.arange(s0, s0 + P - 1)
            # branches, all at once: token i of branch b sits at start[b] + i
            total = int(lens.sum())
            if total:
                owner_b = np.repeat(np.arange(nb), lens)
                within = np.arange(total) - np.repeat(np.cumsum(lens) - lens, lens)
                where = start[owner_b] + within
                ids[where] = np.fromiter((tok for br in t.branches for tok in br), np.int64, total)
                pos[where] = (P + depth[owner_b] + within).astype(np.int32)
                seg[where] = (owner_b + 1).astype(np.int32)
                art[where] = slot
                end[where] = (start[owner_b] + size[owner_b]).astype(np.int32)
                prev[where] = where - 1
                heads = lens > 0
                tail_of_parent = np.where(parents >= 0, start[np.maximum(parents, 0)] + lens[np.maximum(parents, 0)] - 1, s0 + P - 1 if P else -1)
                prev[start[heads]] = tail_of_parent[heads]
            real += P + total
            if grouped:
                row_start = np.empty(len(t.prompt_rows), np.int64)
                rows = []
                for c, pr in enumerate(t.prompt_rows):
                    row_start[c] = len(rows)
                    rows.extend(int(start[bi]) + off for bi, off in pr)
                xb = [(int(start[bi]), int(lens[bi]), p) if bi >= 0 else (s0 + P, 0, p) for bi, p in t.xbranches]
                owners.append(Owner(jid, len(rows), job_end - s0, [], [pl.n_opts for pl in t.plans], row_start, t.plans, s0, P, xb))
            else:
                # one read row per distinct stream position, shared by the options of one lead-in
                row_of, rows, plan = {}, [], []
                for bi, off, target, c, side in t.reads:
                    q = int(start[bi]) + off
                    r = row_of.get(q)
                    if r is None:
                        r = row_of[q] = len(rows)
                        rows.append(q)
                    plan.append((r, target, c, side))
                owners.append(Owner(jid, len(rows), job_end - s0, plan, t.n_options, start=s0))
            sel_parts.append(np.asarray(rows, np.int64))
            n_sel += len(rows)
            cursor = _round_up(job_end) if self.align else job_end
        sel = np.concatenate(sel_parts) if sel_parts else np.zeros(0, np.int64)
        return Batch(ids, pos, seg, art, sel.astype(np.int64), owners, real, media, grp, end, prev)


# ------------------------------------------------------------------------------------------------ tile descriptors
@dataclass
class TileDesc:
    """tiles the attention kernel visits: for query block i, key blocks blocks[offsets[i]:offsets[i+1]] in ascending order;
    flags bit 0 = "full" as the reference classifies tiles, bit 1 = the kernel may skip the mask evaluation. n_causal = nb (nb + 1) / 2, for the skipped fraction."""

    offsets: np.ndarray  # int32 [nb + 1]
    blocks: np.ndarray   # int32 [visited]
    flags: np.ndarray    # uint8 [visited]
    nb: int

    @property
    def visited(self) -> int:
        return int(self.offsets[-1])

    @property
    def skipped_fraction(self) -> float:
        causal = self.nb * (self.nb + 1) // 2
        return 1.0 - self.visited / causal if causal else 0.0


def _pad_to_block(art, end, pos, grp=None):
    n = len(art)
    m = _round_up(n)
    if m == n:
        return art, end, pos, grp
    fill = np.full(m - n, -1, np.int32)
    return (np.concatenate([art, fill]), np.concatenate([end, fill]), np.concatenate([pos, np.zeros(m - n, pos.dtype)]),
            None if grp is None else np.concatenate([grp, fill]))


def tile_desc(art, end, pos, window: int | None = None, grp=None) -> TileDesc:
    """the tile descriptor of one layer type: window None / <= 0 = full attention, else the sliding variant (no "full" tiles, key
    blocks wholly outside the window skipped). grp: the image of every placeholder token (Batch.grp) or None: blocks that share an
    image are kept past the window, and a query block also visits the later key blocks of its images. Built by the library's host
    function (spinf_tile_desc_build_host_img)."""
    from spinf_serve_b200 import _lib

    art, end, pos, grp = _pad_to_block(np.asarray(art), np.asarray(end), np.asarray(pos), None if grp is None else np.asarray(grp))
    art = np.ascontiguousarray(art, np.int32)
    end = np.ascontiguousarray(end, np.int32)
    pos = np.ascontiguousarray(pos, np.int32)
    grp = None if grp is None else np.ascontiguousarray(grp, np.int32)
    nb = len(art) // BLOCK
    counts = np.zeros(nb, np.int32)
    blocks = np.zeros(max(nb * nb, 1), np.int32)
    flags = np.zeros(max(nb * nb, 1), np.uint8)
    total = _lib.lib().spinf_tile_desc_build_host_img(
        _lib.ptr(art), _lib.ptr(end), _lib.ptr(pos), None if grp is None else _lib.ptr(grp), len(art),
        ctypes.c_int32(window if window else 0), _lib.ptr(counts), _lib.ptr(blocks), _lib.ptr(flags),
    )
    if total < 0:
        _lib.check(int(total), "spinf_tile_desc_build_host_img")
    offsets = np.zeros(nb + 1, np.int32)
    np.cumsum(counts, out=offsets[1:])
    if nb:
        keep = np.arange(nb)[None, :] < counts[:, None]
        b2 = blocks[: nb * nb].reshape(nb, nb)[keep]
        f2 = flags[: nb * nb].reshape(nb, nb)[keep]
    else:
        b2, f2 = blocks[:0], flags[:0]
    return TileDesc(offsets, np.ascontiguousarray(b2), np.ascontiguousarray(f2), nb)


def _tables(td: TileDesc):
    """TileDesc -> the reference's (partial_num, partial_idx, full_num, full_idx) arrays"""
    nb = td.nb
    pn = np.zeros(nb, np.int32)
    pi = np.zeros((nb, nb), np.int32)
    fn = np.zeros(nb, np.int32)
    fi = np.zeros((nb, nb), np.int32)
    for i in range(nb):
        sl = slice(td.offsets[i], td.offsets[i + 1])
        b, f = td.blocks[sl], td.flags[sl]
        p, q = b[(f & 1) == 0], b[(f & 1) != 0]
        pn[i], fn[i] = len(p), len(q)
        pi[i, : len(p)] = p
        fi[i, : len(q)] = q
    return pn, pi, fn, fi


def block_tables(art, end, pos, window: int | None, grp=None, always_window: bool = False):
    """the reference's block-table interface (packer.py:426-491): -> (tables of the full-attention layers, tables of the sliding
    layers or None when no position reaches the window and always_window is off). grp: Batch.grp of a stream with images."""
    pos = np.asarray(pos)
    binding = window is not None and (always_window or (len(pos) > 0 and int(pos.max()) >= window))
    full = _tables(tile_desc(art, end, pos, None, grp))
    return full, (_tables(tile_desc(art, end, pos, window, grp)) if binding else None)
