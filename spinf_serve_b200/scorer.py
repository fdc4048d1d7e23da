"""One GPU, one model: packed jobs in, option log-probabilities out. The scoring half of the reference's Scorer
(spinf_serve/scorer.py) behind the same entry points and result types, with the GPU work on the library's kernels:

    score_grouped(items)   scorer.py:383-418   items = (key, first prompt index, GroupedTree) -> {key: [per prompt: log-probs]}
    score_trees(jobs)      scorer.py:366-381   the v0 format after tokenisation: (job id, prompt token ids, option token ids)

How a call runs here (the reference's _execute / _run / _readback, scorer.py:432-510, 263-281, 357-363, do the same job with a
bounded queue, two staging buffers and a fixed one-forward read-back lag):

  * a packing thread turns the items into Batches and does every piece of host work a forward needs ahead of the GPU: the stack's
    plan, the option columns, the tile lists of both layer types (the library's C++ builder), and lays all of a forward's input
    arrays (ids, pos, art, end, tile lists, read rows, option columns, whatever the stack adds) out in ONE pinned staging block;
  * staging blocks come from a small free list; a block returns to the list when the GPU loop has queued its upload, and the
    packing thread reuses it once the copy's CUDA event has completed. The free list is the only back-pressure: no queue depth,
    no polling;
  * the GPU loop uploads a block with one host-to-device copy, launches the forward and the option read, and queues the
    device-to-host copy of the [read rows, option columns] result into a pinned result buffer with an event; finished results
    are harvested whenever their event has completed (at most `readback_lag` forwards stay unharvested while more work waits),
    so the host never blocks on a forward it does not yet need;
  * a failure on either thread closes the flow: the other side wakes, the call raises the original exception, the scorer stays
    usable.

Tokenisation, media, extraction and decoding are outside this path. Differences that follow from the kernels: the lm head reads
only the option columns and needs no padding to lm_rows (a row's result does not depend on the number of rows)."""

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np
import torch

from spinf_serve_b200 import _lib, attention, ops
from spinf_serve_b200.extraction import Extractor
from spinf_serve_b200.packer import Batch, Packer, split_trees


@dataclass(frozen=True)
class EngineConfig:
    """the fields of the reference's EngineConfig the hot path reads (spinf_serve/config.py:29-80), same names and defaults;
    readback_lag is this build's: how many launched forwards may stay unharvested while the packing thread has more ready"""

    token_budget: int = 16384
    max_tokens: int = 65536
    prefetch: int = 6
    pack_window: int = 96  # contents the packer holds back before it packs them first-fit-decreasing (the reference's Packer.push default)
    align_jobs: bool = True
    min_stream: int = 1024
    layers: int | None = None
    fp8s_monitor_every: int = 0
    readback_lag: int = 1
    # extraction branches read on the scoring pass (spinf_serve/config.py:35-49)
    decode_budget_gib: float = 4.0    # captures held between forwards before they are decoded
    decoder_budget_gib: float = 4.0   # one decoder's working set
    capture_budget_gib: float = 2.0   # what one stream's forward may capture (the packer's cost budget)
    x_cuda_graphs: bool = False       # decoding steps replayed from a CUDA graph


@dataclass
class JobResult:
    """a v0 job's scores: logprobs[prompt][option] = log P(option | prompt), and what the job cost"""

    logprobs: list
    packed_tokens: int = 0
    trees: int = 0


@dataclass
class Stats:
    """running totals over the scorer's calls. tokens / forwards / busy_s / wall_s as the reference keeps them; the rest is what
    the staging design makes countable: bytes copied each way and the time the GPU loop spent waiting for the packing thread"""

    tokens: int = 0
    forwards: int = 0
    busy_s: float = 0.0
    wall_s: float = 0.0
    stall_s: float = 0.0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    _spans: list = field(default_factory=list, repr=False)


def option_columns(b: Batch) -> list:
    """the sorted distinct option token ids a batch reads: only these columns leave the lm head (Scorer._cols, scorer.py:420-430)"""
    ids = [np.fromiter((t for _, t, _, _ in o.plan), np.int64) for o in b.owners if o.plan]
    plans = {id(p): p for o in b.owners for p in (o.plans or ())}
    ids += [np.asarray(p.entry_tok, np.int64) for p in plans.values()]
    return np.unique(np.concatenate(ids)).tolist() if ids else []


def read_grouped(lp: np.ndarray, cols, b: Batch, out: dict) -> None:
    """one batch's result lp [read rows, len(cols)] -> out[key][prompt] = float64 log-prob per option of the prompt's ReadPlan:
    an option's score is the sum of its tokens' entries (read_grouped, scorer.py:57-71)"""
    cols = np.asarray(cols, np.int64)
    first_row = np.concatenate(([0], np.cumsum([o.n_rows for o in b.owners]))) if b.owners else np.zeros(1, np.int64)
    column_of = {}
    for o, row0 in zip(b.owners, first_row):
        key, first = o.job_id
        for c, plan in enumerate(o.plans or ()):
            if id(plan) not in column_of:
                column_of[id(plan)] = np.searchsorted(cols, plan.entry_tok)
            picked = lp[row0 + o.row_start[c] + plan.entry_row, column_of[id(plan)]]
            out[key][first + c] = np.bincount(plan.entry_opt, weights=picked.astype(np.float64), minlength=plan.n_opts)


def read_trees(lp: np.ndarray, cols, b: Batch, results: dict) -> None:
    """one batch's result -> the v0 jobs' JobResults: every (row, token, prompt, option) entry of an owner's plan adds its log-prob
    to that option (Scorer._drain, scorer.py:521-535)"""
    cols = np.asarray(cols, np.int64)
    row0 = 0
    for o in b.owners:
        jid, first = o.job_id
        res = results[jid]
        res.packed_tokens += o.n_tokens
        if o.plan:
            ent = np.asarray(o.plan, np.int64).reshape(-1, 4)
            vals = lp[row0 + ent[:, 0], np.searchsorted(cols, ent[:, 1])]
            for v, c, side in zip(vals.tolist(), ent[:, 2].tolist(), ent[:, 3].tolist()):
                res.logprobs[first + c][side] += v
        row0 += o.n_rows


class StagingBlock:
    """all host arrays of one forward in one pinned allocation, mirrored by one device allocation: `pack` lays the arrays out at
    256-byte offsets, `upload` is a single copy and returns typed device views. Both allocations grow on demand and are kept."""

    ALIGN = 256

    def __init__(self, device):
        self.device = device
        self.host = None
        self.dev = None
        self.layout = {}
        self.used = 0
        self.copied = None  # CUDA event of the last upload; the host side may be rewritten once it has completed

    def pack(self, arrays: dict) -> None:
        if self.copied is not None:
            self.copied.synchronize()
            self.copied = None
        layout, off = {}, 0
        for name, a in arrays.items():
            a = np.ascontiguousarray(a)
            layout[name] = (off, a.dtype, a.shape, a)
            off += -(-max(a.nbytes, 1) // self.ALIGN) * self.ALIGN
        if self.host is None or self.host.numel() < off:
            self.host = torch.empty(int(off * 1.25) + self.ALIGN, dtype=torch.uint8).pin_memory()
        view = self.host.numpy()
        for name, (o, dt, shape, a) in layout.items():
            view[o : o + a.nbytes] = a.reshape(-1).view(np.uint8)
            layout[name] = (o, dt, shape, a.nbytes)
        self.layout, self.used = layout, off

    def upload(self) -> dict:
        """queues the copy on the current stream -> {name: device tensor}"""
        if self.dev is None or self.dev.numel() < self.used:
            self.dev = torch.empty(self.host.numel(), dtype=torch.uint8, device=self.device)
        if self.used:
            self.dev[: self.used].copy_(self.host[: self.used], non_blocking=True)
        self.copied = torch.cuda.Event()
        self.copied.record()
        out = {}
        for name, (o, dt, shape, nbytes) in self.layout.items():
            t = self.dev[o : o + nbytes].view(getattr(torch, np.dtype(dt).name))
            out[name] = t.view(shape) if nbytes else t.new_empty(shape)
        return out


class _Flow:
    """what the packing thread and the GPU loop share: the free staging blocks, the prepared forwards, and how the call ended"""

    END = object()

    def __init__(self, blocks):
        self.cv = threading.Condition()
        self.free = deque(blocks)
        self.ready = deque()
        self.closed = False   # no more forwards will be posted
        self.error = None     # the packing thread's exception
        self.cancelled = False

    # packing thread
    def take_block(self):
        with self.cv:
            self.cv.wait_for(lambda: self.free or self.cancelled)
            return None if self.cancelled else self.free.popleft()

    def post(self, ticket) -> None:
        with self.cv:
            self.ready.append(ticket)
            self.cv.notify_all()

    def close(self, error=None) -> None:
        with self.cv:
            self.closed, self.error = True, error
            self.cv.notify_all()

    # GPU loop
    def next(self):
        with self.cv:
            self.cv.wait_for(lambda: self.ready or self.closed)
            if self.ready:
                return self.ready.popleft()
            if self.error is not None:
                raise self.error
            return self.END

    def give_block(self, block) -> None:
        with self.cv:
            self.free.append(block)
            self.cv.notify_all()

    def cancel(self) -> None:
        with self.cv:
            self.cancelled = True
            self.ready.clear()
            self.cv.notify_all()


@dataclass
class _Ticket:
    batch: Batch
    cols: list
    tiles: object          # attention.HostTiles
    block: StagingBlock


@dataclass
class _Flight:
    batch: Batch
    cols: list
    host: torch.Tensor | None   # pinned [read rows, len(cols)] fp32, a view of `buffer`
    done: object                # CUDA event after the device-to-host copy
    buffer: torch.Tensor | None = None


def stage_arrays(stack, sc, b: Batch, cols) -> tuple:
    """host work of one forward: the stack's plan, the tile lists, -> (HostTiles, {name: array}) ready for a StagingBlock"""
    stack.plan(sc, b)
    grp = b.grp if getattr(stack, "bidirectional_images", True) else None  # else image tokens attend causally, as text
    tiles = attention.host_tiles(b.art, b.end, b.pos, getattr(stack, "window", None), always_window=sc.cfg.align_jobs, grp=grp,
                                 bidir_all=getattr(stack, "vision_bidir_all", True))
    arrays = {"ids": b.ids, "sel": np.asarray(b.sel, np.int64), "cols": np.asarray(cols, np.int32)}
    arrays.update(tiles.arrays())
    arrays.update(getattr(b, "staged", None) or {})
    xo = Extractor.owners(b)
    if xo:  # the templates' last tokens: their final hidden states start the decoding
        arrays["xends"] = np.asarray(Extractor.ends(xo), np.int64)
    return tiles, arrays


def stage_one(stack, b: Batch, device, cfg: EngineConfig | None = None):
    """one batch staged outside a scoring call (tests, calibration, a device-resident benchmark loop) -> (sc, inputs, masks, st):
    `sc` is the minimal scorer view the stack methods take, `st` the staged device arrays (st["sel"], st["cols"] among them)"""
    sc = SimpleNamespace(device=torch.device(device), cfg=cfg or EngineConfig(), torch=torch)
    _lib.init(sc.device)
    tiles, arrays = stage_arrays(stack, sc, b, option_columns(b))
    block = StagingBlock(sc.device)
    block.pack(arrays)
    st = block.upload()
    st["_block"] = block  # keeps the device allocation alive as long as the views
    return sc, stack.stage(sc, b, st), attention.device_masks(tiles, st, sc.device), st


def forward_one(stack, b: Batch, device, rows=None, taps=None, cfg: EngineConfig | None = None):
    """stage_one + the stack's forward: [1, n, hidden], or [len(rows), hidden] for the stream positions `rows` (an int64 device
    tensor, or True for the batch's own read rows)"""
    sc, inputs, masks, st = stage_one(stack, b, device, cfg)
    return stack.forward(sc, b, inputs, masks, rows=st["sel"] if rows is True else rows, taps=taps)


class Scorer:
    extractor = None  # extraction.Extractor when the scorer was given stop_ids

    def __init__(self, stack, cfg: EngineConfig | None = None, device="cuda:0", stop_ids=None, banned_ids=(), beam: int | None = None):
        """stack: a built family stack (gemma_stack.GemmaStack, qwen_stack.QwenStack): plan(sc, b), stage(sc, b, st),
        forward(sc, b, inputs, masks, rows=...), .w.lm_weight, .window. stop_ids: the token ids that end a generated answer
        (with them the scorer also decodes the extraction branches of the trees it reads: extraction.Extractor, answers in
        x_found); banned_ids: ids an answer never contains; beam: sequences kept per extraction prompt"""
        self.cfg = cfg or EngineConfig()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the scorer runs on a CUDA device only")
        self.torch = torch
        torch.cuda.set_device(self.device)
        _lib.init(self.device)
        self.stack = stack
        self.softcap = getattr(stack.cfg, "softcap", None)
        pk = Packer(self.cfg.token_budget, self.cfg.max_tokens)
        self.budget, self.max_tokens = pk.budget, pk.max_tokens
        self.min_stream = self.cfg.min_stream
        self.stats = Stats()
        self._blocks = [StagingBlock(self.device) for _ in range(max(self.cfg.prefetch, 1) + 1)]
        self._results = []     # pinned result buffers not in flight
        self._workspace = None
        self.extractor = None
        if stop_ids:
            self.extractor = Extractor(stack, self.device, tuple(stop_ids), tuple(banned_ids), softcap=self.softcap, graphs=self.cfg.x_cuda_graphs,
                                       hold_budget=self.cfg.decode_budget_gib * 2**30, chunk_budget=self.cfg.decoder_budget_gib * 2**30,
                                       **({"beam": beam} if beam else {}))

    # ------------------------------------------------------------------ one forward
    def _launch(self, t: _Ticket, flow: _Flow | None) -> _Flight:
        b, cols = t.batch, t.cols
        xo = Extractor.owners(b)
        if xo and self.extractor is None:
            raise RuntimeError("a tree carries extraction branches but the scorer was built without stop_ids")
        reads = bool(len(b.sel)) and bool(cols)
        if not reads and not xo:
            if flow is not None:
                flow.give_block(t.block)
            return _Flight(b, cols, None, None)
        if getattr(self.stack.w, "scheme", "") == "fp8s":  # sampled forwards only (spinf_serve/scorer.py:270-275)
            from spinf_serve_b200.linears import MONITOR

            k = self.cfg.fp8s_monitor_every
            MONITOR["on"] = bool(k) and self.stats.forwards % k == 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st = t.block.upload()
        self.stats.h2d_bytes += t.block.used
        if flow is not None:
            flow.give_block(t.block)  # reusable by the packing thread once the copy's event has completed
        masks = attention.device_masks(t.tiles, st, self.device)
        inputs = self.stack.stage(self, b, st)
        if xo:  # the forward keeps what decoding needs; the answers are generated between forwards (extraction.Extractor)
            n_sel = st["sel"].numel()
            with self.stack.capture(self, b, xo) as cap:
                rows = self.stack.forward(self, b, inputs, masks, rows=torch.cat([st["sel"], st["xends"]]))
            self.extractor.collect(xo, cap, rows[n_sel:].clone())
            rows = rows[:n_sel]
            if not reads:
                e1.record()
                self.stats._spans.append((e0, e1))
                return _Flight(b, cols, None, None)
        else:
            rows = self.stack.forward(self, b, inputs, masks, rows=st["sel"])
        W = self.stack.w.lm_weight
        need = _lib.lib().spinf_option_logprobs_workspace_bytes(rows.shape[0], W.shape[0], len(cols))
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(int(need * 1.5), dtype=torch.uint8, device=self.device)
        lp = ops.option_logprobs(rows, W, st["cols"], self.softcap, self._workspace)
        buffer = self._result_buffer(lp.numel())
        host = buffer[: lp.numel()].view(lp.shape)
        host.copy_(lp, non_blocking=True)
        e1.record()
        self.stats.d2h_bytes += lp.numel() * 4
        self.stats._spans.append((e0, e1))
        return _Flight(b, cols, host, e1, buffer)

    def _result_buffer(self, n: int):
        for i, r in enumerate(self._results):
            if r.numel() >= n:
                return self._results.pop(i)
        return torch.empty(max(int(n * 1.25), 4096), dtype=torch.float32).pin_memory()

    def _harvest(self, flights: deque, sink, keep: int) -> None:
        """hands finished forwards to `sink`, oldest first: everything whose copy has completed, and, blocking, everything beyond
        the `keep` newest"""
        while flights and (len(flights) > keep or flights[0].done is None or flights[0].done.query()):
            f = flights.popleft()
            if f.host is None:
                sink(np.zeros((len(f.batch.sel), len(f.cols)), np.float32), f.cols, f.batch)
                continue
            f.done.synchronize()
            sink(f.host.numpy(), f.cols, f.batch)
            self._results.append(f.buffer)

    # ------------------------------------------------------------------ one call
    def _prepare(self, batches, flow: _Flow) -> None:
        """the packing thread"""
        try:
            for b in batches():
                cols = option_columns(b)
                tiles, arrays = stage_arrays(self.stack, self, b, cols)
                block = flow.take_block()
                if block is None:
                    return
                block.pack(arrays)
                flow.post(_Ticket(b, cols, tiles, block))
        except BaseException as e:  # noqa: BLE001 - re-raised by the GPU loop, on the caller's thread
            flow.close(e)
            return
        flow.close()

    def _execute(self, batches, sink) -> None:
        """batches: a generator function of Batches (run on the packing thread); sink(lp, cols, batch) receives every forward's
        [read rows, option columns] result on the calling thread, in launch order"""
        flow = _Flow(self._blocks)
        worker = threading.Thread(target=self._prepare, args=(batches, flow), name="spinf-pack", daemon=True)
        t0 = time.perf_counter()
        worker.start()
        flights: deque = deque()
        try:
            while True:
                w0 = time.perf_counter()
                ticket = flow.next()
                self.stats.stall_s += time.perf_counter() - w0
                if ticket is _Flow.END:
                    break
                flights.append(self._launch(ticket, flow))
                self.stats.tokens += ticket.batch.n_tokens
                self.stats.forwards += 1
                self._harvest(flights, sink, self.cfg.readback_lag)
            self._harvest(flights, sink, 0)
            if self.extractor is not None:
                self.extractor.flush()
            self._settle(check=True)
        except BaseException:
            flow.cancel()
            self._settle(check=False)  # nothing of the failed call stays in flight over the staging blocks
            self.stats._spans = []
            if self.extractor is not None:  # nor do its captures (spinf_serve/scorer.py:493-507)
                self.extractor.drop()
                self.stack.abandon(self)
            raise
        finally:
            worker.join()
            for blk in self._blocks:  # a cancelled call may leave blocks with the packing thread or in the ready list
                blk.copied = None
        self.stats.busy_s += sum(a.elapsed_time(c) for a, c in self.stats._spans) / 1000
        self.stats._spans = []
        self.stats.wall_s += time.perf_counter() - t0

    def _settle(self, check: bool) -> None:
        """waits for the device; check: a bounded wait that gave up inside any kernel of the call raises here"""
        torch.cuda.synchronize(self.device)
        if check:
            _lib.last_status()

    # ------------------------------------------------------------------ public
    def _packer(self):
        if self.extractor is None:
            return Packer(self.cfg.token_budget, self.cfg.max_tokens, self.cfg.align_jobs, self.min_stream)
        return Packer(self.cfg.token_budget, self.cfg.max_tokens, self.cfg.align_jobs, self.min_stream, cost=self.extractor.tree_bytes,
                      cost_budget=int(self.cfg.capture_budget_gib * 2**30))

    @property
    def x_found(self) -> dict:
        """answers of the extraction branches read so far: {prompt key: [(token ids, log-prob)] best first} (Scorer.x_found)"""
        return self.extractor.found if self.extractor is not None else {}

    def score_grouped(self, items) -> dict:
        """items: an iterable of (key, first prompt index, GroupedTree); several items may share a key (a job split over the
        budget). It is consumed lazily on the packing thread, so a generator that pulls work from a shared queue is fine.
        -> {key: per prompt the float64 log-probs of its plan's options}"""
        out: dict = {}

        def batches():
            packer = self._packer()
            for key, first, tree in items:
                slots = out.setdefault(key, [])
                slots.extend([None] * (first + len(tree.plans) - len(slots)))
                yield from packer.push((key, first), tree, self.cfg.pack_window)
            yield from packer.flush()

        self._execute(batches, lambda lp, cols, b: read_grouped(lp, cols, b, out))
        return out

    def extract(self, jobs) -> dict:
        """extraction jobs (extraction.ExtractJob) -> {prompt key: [(token ids, log-prob)] best first}: each job's prefix read once
        through the packed path with its prompts as extraction branches (a prompt without template tokens: a zero-length branch at
        the prefix's end), all decoded together; the form the reference uses for its hybrid models (Scorer._extract_hybrid,
        spinf_serve/scorer.py:748-766), here for both families"""
        from spinf_serve_b200.packer import GroupedTree

        if self.extractor is None:
            raise RuntimeError("extract needs a scorer built with stop_ids")
        items = []
        for n, job in enumerate(jobs):
            branches, xb = [], []
            for pr in job.prompts:
                if pr.kind != "text":
                    raise ValueError(f"prompt {pr.key}: only text slots are searched here")
                if pr.ids:
                    xb.append((len(branches), pr))
                    branches.append(list(pr.ids))
                else:
                    xb.append((-1, pr))
            items.append((("x", n), 0, GroupedTree(list(job.prefix), branches, [], [], media=list(job.media), xbranches=xb, parents=[-1] * len(branches))))
        self.score_grouped(items)
        return {pr.key: self.extractor.found.pop(pr.key) for job in jobs for pr in job.prompts}

    def score_trees(self, jobs) -> dict:
        """jobs: (job id, prompt token ids, option token ids per prompt), the reference's Scorer.score after tokenisation ->
        {job id: JobResult}"""
        results = {jid: JobResult([[0.0] * len(o) for o in opts]) for jid, _, opts in jobs}
        if len(results) != len(jobs):
            raise ValueError("job ids must be unique within a call")

        def batches():
            packer = self._packer()
            for jid, prompts, opts in jobs:
                try:
                    runs = split_trees(prompts, opts, self.budget)
                except ValueError as e:
                    raise ValueError(f"job {jid}: {e}") from None
                for first, tree in runs:
                    results[jid].trees += 1
                    yield from packer.push((jid, first), tree, self.cfg.pack_window)
            yield from packer.flush()

        self._execute(batches, lambda lp, cols, b: read_trees(lp, cols, b, results))
        return results

    def fp8s_peak(self):
        """fp8s with the monitor on: (the largest input / clip level over the linears since load, (layer, linear name)), else
        None (spinf_serve/scorer.py:308-317); above 1 an input was clipped: the scale table did not cover it"""
        if getattr(self.stack.w, "scheme", "") != "fp8s" or not self.cfg.fp8s_monitor_every:
            return None
        peaks = self.stack.peaks()
        k = max(peaks, key=peaks.get)
        return peaks[k], k

    # names the reference's callers know
    _cols = staticmethod(option_columns)
