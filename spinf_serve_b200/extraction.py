"""Extraction on the scoring pass: the trees of a scoring call may carry extraction branches (GroupedTree.xbranches: a template
text after the shared prefix whose answer is generated, not scored). The forward that reads such a tree also captures what
decoding needs (Stack.capture), the decoding itself runs between forwards in chunks that fit a memory budget, and the answers
land in Extractor.found. The counterpart of the reference's Scorer._x_collect / _x_flush / _x_chunks / _x_split / _x_sub and
_x_tree_bytes (spinf_serve/scorer.py:768-895, budgets spinf_serve/config.py:35-43), arranged here as one object the scorer owns:

    collect(owners, cap, h_ends)   one forward's captures -> decode.Group per tree, held until the held bytes pass hold_budget
    flush()                        held groups -> chunks under chunk_budget (decode.chunk_bytes counts the padded chunk; a group
                                   that does not fit alone is cut into runs of its prompts, which share the prefix captures) ->
                                   decode.Decoder / HybridDecoder + decode.search_text -> found[prompt key] = [(tokens, log-prob)]
    tree_bytes(tree)               what a forward will capture for a tree: the packer's cost function, so that one stream's
                                   captures stay under capture_budget next to the forward's own peak

The search is the text kind (decode.search_text); which token ids end an answer and which may never appear is the caller's
knowledge of its tokenizer (stop_ids, banned_ids)."""

from dataclasses import dataclass, field

from spinf_serve_b200 import decode

GIB = float(2**30)


@dataclass
class ExtractPrompt:
    """one extraction read (extract.ExtractPrompt, spinf_serve/extract.py:58-69): the tokens after the job's prefix up to the slot
    (may be empty: the slot starts right after the prefix) and how many tokens an answer may have; `kind` is "text" here"""

    key: object
    ids: list
    max_tokens: int
    kind: str = "text"


@dataclass
class ExtractJob:
    """one content's extraction reads (extract.ExtractJob, :71-78): the prefix, read once, and the prompts that decode from it"""

    prefix: list
    prompts: list
    media: list = field(default_factory=list)


@dataclass
class Extractor:
    stack: object
    device: object
    stop_ids: tuple
    banned_ids: tuple = ()
    beam: int = decode.BEAM
    graphs: bool = False
    min_p: float = 0.002
    softcap: float | None = None
    hold_budget: float = 4.0 * GIB    # EngineConfig.decode_budget_gib: captures held between forwards
    chunk_budget: float = 4.0 * GIB   # EngineConfig.decoder_budget_gib: one decoder's working set
    found: dict = field(default_factory=dict)
    chunks_run: int = 0
    generated: int = 0
    _held: list = field(default_factory=list)
    _held_bytes: int = 0

    def __post_init__(self):
        self.hybrid = bool(getattr(self.stack, "hybrid", False))
        self.per_tok = self.stack.kv_bytes_per_token()  # {layer with K/V: bytes per stored token}
        cfg = self.stack.cfg
        if self.hybrid:
            rec = [i for i in range(self.stack.n_layers) if self.stack.w.layers[i]["kind"] == "linear_attention"]
            cd = 2 * cfg.hk * cfg.dk + cfg.hv * cfg.dv
            # per recurrent layer: a cached row (q, k, v bf16, g fp32, beta bf16), a prefix state, a template's three ring rows
            self.row_bytes = len(rec) * (2 * cd + 6 * cfg.hv)
            self.state_bytes = len(rec) * cfg.hv * cfg.dk * cfg.dv * 4
            self.ring_bytes = len(rec) * 3 * cd * 2
        else:
            self.row_bytes = self.state_bytes = self.ring_bytes = 0

    # ---- what a forward needs to know about a batch
    @staticmethod
    def owners(b) -> list:
        return [o for o in b.owners if o.xbranches]

    @staticmethod
    def ends(owners) -> list:
        """stream position of each template's last token (a branch of length 0: the prefix's last token), in collect's order"""
        return [bs + bl - 1 for o in owners for bs, bl, _ in o.xbranches]

    def tree_bytes(self, tree) -> int:
        """bytes the forward captures for a tree (0 without extraction branches): the prefix's and the templates' K/V, on the
        hybrid family also the templates' recurrent rows and rings and the prefix state"""
        xb = getattr(tree, "xbranches", None)
        if not xb:
            return 0
        tok = sum(self.per_tok.values())
        rows = sum(len(tree.branches[b]) for b, _ in xb if b >= 0)
        return len(tree.prefix) * tok + rows * (tok + self.row_bytes) + len(xb) * self.ring_bytes + self.state_bytes

    # ---- between forwards
    def collect(self, owners, cap: dict, h_ends) -> None:
        """owners: Extractor.owners(batch); cap: what Stack.capture yielded around the batch's forward; h_ends [len(ends), hidden]:
        the final hidden states at Extractor.ends(owners), from which a prompt's first generated token is read"""
        kv, extra = cap["kv"], cap.get("extra")
        k = 0
        for o in owners:
            g = decode.Group(kv.pop(("p", id(o))), o.prefix_len)
            if extra is not None:
                g.extra = {"state": extra["state"].pop(("p", id(o))), "tmpl": []}
            for _, bl, pr in o.xbranches:
                key = ("t", pr.key)
                g.prompts.append((pr, kv.pop(key, {}), bl, h_ends[k]))
                if extra is not None:
                    g.extra["tmpl"].append({"tok": extra["tok"].pop(key, {}), "pre": extra["pre"].pop(key, {})})
                k += 1
            if extra is not None:
                g.extra_bytes = self._extra_bytes(g)
            need = decode.group_bytes(g, self.per_tok, self._steps([g]), self.beam)
            if self._held and self._held_bytes + need > self.hold_budget:
                self.flush()
            self._held.append(g)
            self._held_bytes += need
        if self._held_bytes > self.hold_budget:  # one long prefix over the budget on its own: decode now
            self.flush()

    def flush(self) -> None:
        groups, self._held, self._held_bytes = self._held, [], 0
        for chunk in self._chunks(groups):
            cls = decode.HybridDecoder if self.hybrid else decode.Decoder
            dec = cls(self.stack, chunk, self.device, beam=self.beam, graphs=self.graphs)
            answers = decode.search_text(dec, self.stack.w.lm_weight, list(self.stop_ids), list(self.banned_ids), min_p=self.min_p,
                                         softcap=self.softcap)
            for key, a in answers.items():
                self.found[key] = a
                self.generated += sum(len(t) for t, _ in a[:1])
            del dec, chunk
            self.chunks_run += 1

    def drop(self) -> None:
        """a failed call keeps none of its captures"""
        self._held, self._held_bytes = [], 0

    # ---- chunking
    @staticmethod
    def _steps(groups) -> int:
        return 1 + max(p[0].max_tokens for g in groups for p in g.prompts)

    def _extra_bytes(self, g) -> int:
        rows = sum(p[2] for p in g.prompts) + len(g.prompts) * self.beam * self._steps([g])
        return self.state_bytes + rows * self.row_bytes + len(g.prompts) * self.beam * self.ring_bytes

    def _chunk_bytes(self, groups) -> int:
        return decode.chunk_bytes(groups, self.per_tok, sum(g.extra_bytes for g in groups), self.beam)

    def _chunks(self, groups: list):
        """greedy: parts in arrival order, a chunk closed when the next part would take the padded chunk over the budget. The
        caller's list is emptied as it goes, so a prefix's captures are freed once the last run that reads them has been decoded"""
        chunk = []
        while groups:
            for part in self._runs(groups.pop(0)):
                if chunk and self._chunk_bytes([*chunk, part]) > self.chunk_budget:
                    yield chunk
                    chunk = []
                chunk.append(part)
        if chunk:
            yield chunk

    def _runs(self, g) -> list:
        """a group that fits the chunk budget alone, or else consecutive runs of its prompts that do (each the longest that fits,
        found by bisection: a run's bytes grow with its length; one prompt at least); the runs share the prefix captures"""
        n = len(g.prompts)
        if n == 1 or self._chunk_bytes([g]) <= self.chunk_budget:
            return [g]
        runs, a = [], 0
        while a < n:
            lo, hi = a + 1, n  # the longest run [a, b) that fits has lo <= b <= hi
            while lo < hi:
                mid = (lo + hi + 1) // 2
                if self._chunk_bytes([self._run(g, a, mid)]) <= self.chunk_budget:
                    lo = mid
                else:
                    hi = mid - 1
            runs.append(self._run(g, a, lo))
            a = lo
        g.prefix_kv, g.extra, g.prompts = {}, None, []  # the runs hold the captures now
        return runs

    def _run(self, g, a: int, b: int):
        """prompts [a, b) of a group as a group of its own: the prefix captures by reference, the per-prompt captures sliced"""
        extra = None if g.extra is None else {"state": dict(g.extra["state"]), "tmpl": g.extra["tmpl"][a:b]}
        run = decode.Group(dict(g.prefix_kv), g.P, list(g.prompts[a:b]), extra)
        if extra is not None:
            run.extra_bytes = self._extra_bytes(run)
        return run
