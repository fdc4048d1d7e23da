"""One GPU, one model: packed jobs in, option log-probabilities out. The scoring half of the reference's Scorer
(spinf_serve/scorer.py) behind the same entry points, with the GPU work on the library's kernels:

    score_grouped(items)   scorer.py:383-418   items = (key, first prompt index, GroupedTree) -> {key: [per prompt: log-probs]}
    score_trees(jobs)      scorer.py:366-381   the v0 format after tokenisation: (job id, prompt token ids, option token ids)
    _cols / _forward / _execute / _readback / read_grouped / _drain     scorer.py:420-430, 241-261, 432-510, 357-363, 57-71, 521-535

As in the reference a producer thread packs (and plans) batches ahead of the GPU loop through a bounded queue, the inputs go up
through pinned memory, and each forward's log-probs are read back one forward late. Tokenisation, media, extraction and decoding
are outside this path. Differences that follow from the kernels: the lm head reads only the option columns and needs no padding to
lm_rows (a row's result does not depend on the number of rows)."""

import queue
import threading
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from spinf_serve_b200 import _lib, ops
from spinf_serve_b200.packer import Batch, Packer, split_trees


@dataclass(frozen=True)
class EngineConfig:
    """the fields of the reference's EngineConfig the hot path reads (spinf_serve/config.py:29-80), same names and defaults"""

    token_budget: int = 16384
    max_tokens: int = 65536
    prefetch: int = 6
    align_jobs: bool = True
    min_stream: int = 1024
    layers: int | None = None  # debug: run the first n layers only
    fp8s_monitor_every: int = 0  # fp8s: check every k-th forward's linear inputs against their scales (0 = never)


@dataclass
class JobResult:
    logprobs: list  # per prompt, per option: log P(option | prompt)
    packed_tokens: int = 0
    trees: int = 0


@dataclass
class Stats:
    tokens: int = 0
    forwards: int = 0
    busy_s: float = 0.0  # CUDA-event time of the forwards
    wall_s: float = 0.0
    _events: list = field(default_factory=list, repr=False)


def read_grouped(lp: np.ndarray, cols, b: Batch, out: dict) -> None:
    """lp [read rows, len(cols)] of one batch -> out[key][prompt] = float64 log-probs of the prompt's options, each the sum of
    its tokens' entries as its ReadPlan lists them"""
    cols_arr = np.asarray(cols, np.int64)
    col_of_plan = {}
    base = 0
    for o in b.owners:
        key, first = o.job_id
        for c, plan in enumerate(o.plans or ()):
            ci = col_of_plan.get(id(plan))
            if ci is None:
                ci = col_of_plan[id(plan)] = np.searchsorted(cols_arr, plan.entry_tok)
            vals = lp[base + o.row_start[c] + plan.entry_row, ci].astype(np.float64)
            out[key][first + c] = np.bincount(plan.entry_opt, weights=vals, minlength=plan.n_opts)
        base += o.n_rows


class Scorer:
    def __init__(self, stack, cfg: EngineConfig | None = None, device="cuda:0"):
        """stack: a built family stack (gemma_stack.GemmaStack): plan(b), stage(b, device), forward(inputs, rows), .w.lm_weight"""
        self.cfg = cfg or EngineConfig()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the scorer runs on a CUDA device only")
        torch.cuda.set_device(self.device)
        _lib.init(self.device)
        self.stack = stack
        self.softcap = getattr(stack.cfg, "softcap", None)
        pk = Packer(self.cfg.token_budget, self.cfg.max_tokens)
        self.budget, self.max_tokens = pk.budget, pk.max_tokens
        self.min_stream = self.cfg.min_stream
        self.stats = Stats()
        self._workspace = None

    # ------------------------------------------------------------------ forward
    @staticmethod
    def _cols(b: Batch) -> list:
        """the sorted distinct option token ids a batch reads"""
        cols = {t for o in b.owners for _, t, _, _ in o.plan}
        seen = set()
        for o in b.owners:
            for plan in o.plans or ():
                if id(plan) not in seen:
                    seen.add(id(plan))
                    cols.update(plan.entry_tok.tolist())
        return sorted(cols)

    def _forward(self, b: Batch, cols: list):
        """batch -> log-probs [n_sel, len(cols)] fp32 on the device"""
        dev = self.device
        if not len(b.sel) or not cols:
            return torch.zeros((len(b.sel), len(cols)), dtype=torch.float32, device=dev)
        if getattr(self.stack.w, "scheme", "") == "fp8s":  # sampled forwards only (spinf_serve/scorer.py:270-275)
            from spinf_serve_b200.linears import MONITOR

            k = self.cfg.fp8s_monitor_every
            MONITOR["on"] = bool(k) and self.stats.forwards % k == 0
        inputs = self.stack.stage(b, dev)
        sel = torch.from_numpy(b.sel).pin_memory().to(dev, non_blocking=True)
        ci = torch.tensor(cols, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        rows = self.stack.forward(inputs, rows=sel)
        W = self.stack.w.lm_weight
        need = _lib.lib().spinf_option_logprobs_workspace_bytes(rows.shape[0], W.shape[0], len(cols))
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(int(need * 1.5), dtype=torch.uint8, device=dev)
        return ops.option_logprobs(rows, W, ci, self.softcap, self._workspace)

    def fp8s_peak(self):
        """fp8s with the monitor on: (the largest input / clip level over the linears since load, (layer, linear name)), else
        None (spinf_serve/scorer.py:308-317); above 1 an input was clipped: the scale table did not cover it"""
        if getattr(self.stack.w, "scheme", "") != "fp8s" or not self.cfg.fp8s_monitor_every:
            return None
        peaks = self.stack.peaks()
        k = max(peaks, key=peaks.get)
        return peaks[k], k

    def _readback(self, lp):
        host = torch.empty(lp.shape, dtype=lp.dtype).pin_memory()
        host.copy_(lp, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(lp.device))
        return host, ev

    # ------------------------------------------------------------------ the GPU loop
    def _execute(self, batches, drain) -> None:
        q: queue.Queue = queue.Queue(self.cfg.prefetch)
        stop = threading.Event()

        def put(x) -> bool:
            while not stop.is_set():
                try:
                    q.put(x, timeout=0.2)
                    return True
                except queue.Full:
                    pass
            return False

        def producer():
            try:
                for b in batches():
                    if stop.is_set():
                        return
                    self.stack.plan(b)
                    if not put(b):
                        return
            except BaseException as e:  # handed to the GPU loop, which re-raises it
                put(e)
            put(None)

        threading.Thread(target=producer, daemon=True).start()
        t0 = time.perf_counter()
        pending = []
        try:
            while True:
                b = q.get()
                if b is None:
                    break
                if isinstance(b, BaseException):
                    raise b
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                cols = self._cols(b)
                e0.record()
                lp = self._forward(b, cols)
                e1.record()
                self.stats._events.append((e0, e1))
                pending.append((self._readback(lp), cols, b))
                self.stats.tokens += b.n_tokens
                self.stats.forwards += 1
                if len(pending) > 1:
                    drain(pending.pop(0))
            for item in pending:
                drain(item)
        except BaseException:
            stop.set()
            pending.clear()
            while True:
                try:
                    q.get_nowait()
                except queue.Empty:
                    break
            self.stats._events = []
            raise
        torch.cuda.synchronize(self.device)
        _lib.last_status()  # a bounded wait that gave up inside any kernel of the call raises here
        self.stats.busy_s += sum(a.elapsed_time(c) for a, c in self.stats._events) / 1000
        self.stats._events = []
        self.stats.wall_s += time.perf_counter() - t0

    # ------------------------------------------------------------------ public
    def _packer(self):
        return Packer(self.cfg.token_budget, self.cfg.max_tokens, self.cfg.align_jobs, self.min_stream)

    def score_grouped(self, items) -> dict:
        out: dict = {}
        for key, first, tree in items:
            slots = out.setdefault(key, [])
            need = first + len(tree.plans)
            if len(slots) < need:
                slots.extend([None] * (need - len(slots)))

        def batches():
            packer = self._packer()
            for key, first, tree in items:
                yield from packer.push((key, first), tree)
            yield from packer.flush()

        def drain(item):
            (host, ev), cols, b = item
            ev.synchronize()
            read_grouped(host.numpy(), cols, b, out)

        self._execute(batches, drain)
        return out

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
                    yield from packer.push((jid, first), tree)
            yield from packer.flush()

        self._execute(batches, lambda item: self._drain(item, results))
        return results

    @staticmethod
    def _drain(item, results: dict) -> None:
        (host, ev), cols, b = item
        ev.synchronize()
        lp = host.numpy()
        col = {c: i for i, c in enumerate(cols)}
        base = 0
        for o in b.owners:
            jid, first = o.job_id
            res = results[jid]
            res.packed_tokens += o.n_tokens
            for r, t, c, side in o.plan:
                res.logprobs[first + c][side] += float(lp[base + r, col[t]])
            base += o.n_rows
