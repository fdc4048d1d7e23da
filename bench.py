"""Throughput of the packed-prefill scoring path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Headline workload (benchmark configuration 2, at every N): one step = one pass of the hot path over one batch, the 24 contents x
56 two-option questions (1344 questions, 27408 real tokens) packed into one 27648-token stream and scored by the synthetic
Gemma-style 12B with fp8 row-wise linears (random-init weights, uniform random token ids; the reference's benchmark text is not
reproduced). Rank r of N scores its own 24 contents (replicas, no collective on the data path): weak scaling.

  value      questions/s with the packed inputs already resident in HBM (stack forward + option log-prob read), K steps between
             CUDA events, max over ranks
  e2e        the same through the public call Scorer.score_grouped with host inputs: one call over the K steps' contents, which
             the packer turns into K forwards of the same 27648-token shape; packing, tile lists, the pinned host->device copy,
             forward and device->host read of every forward's log-probs inside the timed region (the packing thread prepares the
             next forward while the GPU runs this one). forwards / tokens report what actually ran.
  roofline   the row-wise fp8 GEMM (dominant kernel): algorithmic FLOPs / CUDA-event time of its launches in the timed region,
             against an fp8 peak measured in this run (torch._scaled_mm per-tensor 8192^3, burst and sustained)
  attention  the tree attention alone on configuration 1 (2 contents x (470 + 8 x 16) tokens, H16 / Hkv8 / D256, N(0,1) inputs
             with scale 1/16): time per launch (L2 flushed between launches), TFLOP/s on the unmasked pairs, tiles visited; and
             its share and rate inside the configuration-2 step
  bulk       benchmark configuration 3 in small: a seeded slice of the bulk workload (trunks U[200, 2000], 56 questions, branches
             U[8, 24], 2-5 options, 32768-token passes) scored through the replica runner, the N replicas drawing content chunks
             from one shared host-side queue: strong scaling (the slice is the same at every N), with per-rank busy fractions
             and a bit-equality check of sampled contents scored alone
  cpu_baseline   the CPU oracle (a port of the reference's arithmetic; the reference has no CPU forward) on a bounded sample

--impl reference times that CPU oracle alone, with all host threads, on the same sample, and prints the line with "impl": "reference"."""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "questions scored/sec"
UNIT = "questions/s"
WORKLOAD = "cfg2: gemma-style 12B fp8 row-wise, 24 contents x (470-token trunk + 56 questions x 12 tokens, 2 single-token options), one 27648-token forward"
CPU_SAMPLE = {"n_contents": 2, "layers": 2}  # the one sample both CPU legs time


def _peaks():
    """measured peaks of this pool (driver-written file), else the stated fallback"""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons while the timed region runs"""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU arm (the oracle, a port)
def cpu_sample(threads: int, n_contents: int, layers: int):
    """the CPU oracle on a bounded sample of the workload: n_contents of the 24 contents (1142 tokens, 56 questions each) through
    `layers` of the 48 layers plus the lm-head read of their rows; -> (a closure that runs the sample once and returns
    (seconds in the layers, seconds in the head read), the sample's workload)"""
    import numpy as np
    import torch

    from oracle import gemma as OG
    from oracle import head as OH
    from spinf_serve_b200 import packer as P
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.scorer import option_columns

    torch.set_num_threads(threads)
    cfg = OG.GemmaConfig(layers=layers)
    g = torch.Generator().manual_seed(0)

    def lin(o, i):
        return torch.empty((o, i), dtype=torch.bfloat16).normal_(0.0, 0.02, generator=g)

    H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    ones = lambda d: torch.ones(d, dtype=torch.bfloat16)  # noqa: E731
    L = {
        "q": lin(H * D, cfg.hidden), "k": lin(K * D, cfg.hidden), "v": lin(K * D, cfg.hidden), "o": lin(cfg.hidden, H * D),
        "gate": lin(cfg.ffn, cfg.hidden), "up": lin(cfg.ffn, cfg.hidden), "down": lin(cfg.hidden, cfg.ffn),
        "q_norm": ones(D), "k_norm": ones(D), "input_ln": ones(cfg.hidden), "post_attn_ln": ones(cfg.hidden),
        "pre_ffn_ln": ones(cfg.hidden), "post_ffn_ln": ones(cfg.hidden),
    }
    W = {"embed": lin(cfg.vocab, cfg.hidden), "norm": ones(cfg.hidden), "layers": [L] * layers}  # the same weights in every layer
    Q = OG.quantize(W)
    wl = workloads.config2(seed=0, n_contents=n_contents)
    pk = P.Packer(32768, 65536, True, 1024)
    batches = [b for key, first, t in wl.items for b in pk.push((key, first), t)] + list(pk.flush())
    (b,) = batches
    cols = option_columns(b)

    def run():
        t0 = time.perf_counter()
        hf = OG.forward(cfg, W, Q, b.ids, b.art, b.end, b.pos)
        t1 = time.perf_counter()
        OH.option_logprobs(hf[torch.as_tensor(b.sel)], W["embed"], np.asarray(cols), None)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    return run, wl


def cpu_extrapolate(layer_s: float, head_s: float, wl, layers: int, threads: int):
    """the sample's times scaled to the full step (linear in layers x tokens for the forward, in rows for the head read)
    -> (questions/s, the words that say what was timed and how it was scaled)"""
    kl, kt, kr = 48 / layers, 27408 / wl.n_tokens, 1344 / wl.n_questions
    full = layer_s * kl * kt + head_s * kr
    words = (
        f"CPU oracle port (torch fp32, {threads} threads) on {CPU_SAMPLE['n_contents']} of 24 contents ({wl.n_tokens} tokens, {wl.n_questions} questions) "
        f"through {layers} of 48 layers ({layer_s:.2f} s) + the lm-head read of their rows ({head_s:.2f} s); extrapolated x{kl:.0f} in layers, "
        f"x{kt:.1f} in tokens, x{kr:.0f} in read rows to the full step ({full:.0f} s)"
    )
    return 1344 / full, words


def cpu_baseline(threads: int, repeats: int = 4):
    run, wl = cpu_sample(threads, **CPU_SAMPLE)
    run()
    times = [run() for _ in range(repeats)]
    layer_s = sum(t[0] for t in times) / repeats
    head_s = sum(t[1] for t in times) / repeats
    qps, words = cpu_extrapolate(layer_s, head_s, wl, CPU_SAMPLE["layers"], threads)
    return {"value": qps, "unit": UNIT, "cores": threads, "kind": "port", "sample": words + f"; mean of {repeats} runs after one warm-up"}


def reference_arm(args):
    """--impl reference: the reference has no CPU forward of its own (its Scorer is CUDA-only), so this arm times the CPU oracle
    assembled from its arithmetic, on the host cores, each step one run of the bounded sample; no GPU is used"""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    run, wl = cpu_sample(threads, **CPU_SAMPLE)
    for _ in range(min(args.warmup, 1)):
        run()
    t0 = time.perf_counter()
    times = [run() for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    layer_s = sum(t[0] for t in times) / len(times)
    head_s = sum(t[1] for t in times) / len(times)
    qps, words = cpu_extrapolate(layer_s, head_s, wl, CPU_SAMPLE["layers"], threads)
    line = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": UNIT, "n_gpus": 0, "n_gpus_requested": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000 * wall / max(args.steps, 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic", "config": {"workload": WORKLOAD, "l2": "inputs larger than L2", "step": "one run of the CPU sample"},
        "cpu_baseline": {"value": qps, "unit": UNIT, "cores": threads, "kind": "port", "sample": words + f"; mean of {args.steps} steps"},
        "e2e": {"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ GPU arm
def measure_fp8_peak(dev, seconds: float = 2.0):
    """a library fp8 GEMM of the size the bf16 figures of MEASURED_PEAKS.json were taken at (8192^3, per-tensor scales, bf16 out):
    best of 10 (burst) and back to back for `seconds` (sustained) -> TFLOP/s. The denominator of the fp8 roofline fraction."""
    import torch

    n = 8192
    a = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn)
    b = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn).t()
    one = torch.ones((), dtype=torch.float32, device=dev)
    flops = 2.0 * n**3

    def mm():
        return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

    for _ in range(3):
        mm()
    best = 0.0
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mm()
        e1.record()
        e1.synchronize()
        best = max(best, flops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(int(seconds / (flops / (best * 1e12))), 10)
    e0.record()
    for _ in range(reps):
        mm()
    e1.record()
    e1.synchronize()
    return {"burst": best, "sustained": reps * flops / (e0.elapsed_time(e1) * 1e-3) / 1e12}


def attention_alone(dev, peaks, repeats: int = 30):
    """benchmark configuration 1: the tree attention on 2 contents x (470-token trunk + 8 branches of 16), H16 / Hkv8 / D256,
    Q K V ~ N(0,1) bf16 seed 0 with scale 1/16; L2 flushed (a 256 MB write) before every timed launch"""
    import torch

    from spinf_serve_b200 import attention, workloads
    from spinf_serve_b200.packer import Packer

    wl = workloads.config1(seed=0)
    pk = Packer(16384, 65536, True, 1024)
    (b,) = [x for key, first, t in wl.items for x in pk.push((key, first), t)] + list(pk.flush())
    n, H, K, D = b.length, 16, 8, 256
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((n, h, D), generator=g).to(torch.bfloat16).to(dev) for h in (H, K, K))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name, window in (("full", None), ("sliding_1024", 1024)):
        mask = attention.stream_masks(b.art, b.end, b.pos, window, dev, always_window=True)["sliding_attention" if window else "full_attention"]
        pairs = workloads.attended_pairs(b, window)
        flops = 4.0 * D * H * pairs
        for _ in range(3):
            attention.tree_attention(q, k, v, mask, 1.0 / 16)
        ms = []
        for _ in range(repeats):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            attention.tree_attention(q, k, v, mask, 1.0 / 16)
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        ms.sort()
        med = ms[len(ms) // 2]
        nb = n // 128
        out[name] = {
            "ms": med, "ms_min": ms[0], "unmasked_pairs": pairs, "unmasked_gflop": flops / 1e9, "tflops_unmasked": flops / (med * 1e-3) / 1e12,
            "frac_of_bf16_burst": flops / (med * 1e-3) / 1e12 / peaks["bf16_burst"], "tiles_visited": mask.visited, "tiles_causal": nb * (nb + 1) // 2,
            "tiles_total": nb * nb,
        }
    return {"workload": "cfg1: 2 contents x (470 + 8 x 16) tokens in a 1280-row stream, H16/Hkv8/D256, N(0,1) bf16 inputs, scale 1/16", "l2": "flushed before every launch", **out}


def bulk_leg(args, stack, dev, rank, world, sync, host_group):
    """benchmark configuration 3 in small, through the replica runner with a shared content queue (strong scaling)"""
    import numpy as np
    import torch
    import torch.distributed as dist

    from spinf_serve_b200 import replicas, workloads
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    n = args.bulk_contents
    t0 = time.perf_counter()
    wl = workloads.bulk_slice(seed=0, n_contents=n)
    gen_s = time.perf_counter() - t0
    # several replicas on one queue: a replica's packer holds back 24 contents instead of 96 before it packs, so that no replica sits
    # on six passes' worth of drawn contents when the queue runs dry (one more pass in 167 on this slice; 96 for a single replica)
    window = 96 if world == 1 else 24
    scorer = Scorer(stack, EngineConfig(token_budget=32768, max_tokens=65536, prefetch=2, pack_window=window), dev)
    scorer.score_grouped(wl.items[: min(n, 32)])  # warm-up: two passes of this shape
    s0 = (scorer.stats.forwards, scorer.stats.tokens, scorer.stats.busy_s, scorer.stats.stall_s)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    merged, queue = replicas.score_queued(scorer, wl.items, chunk=8, group=host_group, name=f"spinf/bulk/{args.steps}/{n}")
    e1.record()
    sync()
    wall = time.perf_counter() - w0
    ms = e0.elapsed_time(e1)
    mine = [scorer.stats.forwards - s0[0], scorer.stats.tokens - s0[1], scorer.stats.busy_s - s0[2], scorer.stats.stall_s - s0[3], wall, float(len(queue.taken))]
    per_rank = [mine]
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        parts = [None] * world if rank == 0 else None
        dist.gather_object(mine, parts, dst=0, group=host_group)
        per_rank = parts
    if rank != 0:
        return None
    # contents scored alone must equal, bit for bit, what the replicas returned for them (whatever they were packed with)
    sample = sorted({0, 1, n // 3, n // 2, n - 1})
    same = True
    for c in sample:
        alone = scorer.score_grouped([wl.items[c]])
        key = wl.items[c][0]
        same &= all(np.array_equal(a, m) for a, m in zip(alone[key], merged[key]))
    missing = sum(1 for key, _, _ in wl.items if key not in merged or any(v is None for v in merged[key]))
    return {
        "workload": f"cfg3 slice: {n} contents (trunks U[200,2000], 56 questions, branches U[8,24], 2-5 options; seed 0, per-content streams), 32768-token passes",
        "scaling": "strong", "value": wl.n_questions / (ms * 1e-3), "unit": UNIT, "tokens_per_s": wl.n_tokens / (ms * 1e-3), "ms": ms, "questions": wl.n_questions,
        "tokens": wl.n_tokens, "queue": f"shared counter in the process group's host-side store, chunks of 8 contents, packer window {window}; no collective on the data path",
        "per_rank": [
            {"forwards": int(p[0]), "tokens": int(p[1]), "gpu_busy_fraction": round(p[2] / p[4], 4), "waited_for_packing_s": round(p[3], 3), "chunks": int(p[5])}
            for p in per_rank
        ],
        "contents_missing": missing, "alone_equals_packed_bitwise": bool(same), "sampled_contents": sample, "host_generation_s": round(gen_s, 2),
    }


def gpu_arm(args):
    import torch
    import torch.distributed as dist

    from spinf_serve_b200 import _lib, ops, workloads
    from spinf_serve_b200.gemma_stack import CONFIGS, GemmaConfig, GemmaStack, GemmaWeights
    from spinf_serve_b200.packer import Packer
    from spinf_serve_b200.scorer import EngineConfig, Scorer, stage_one

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the scoring path has no CPU fallback (use --impl reference for the CPU arm)")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")  # host objects (results, counters) travel over gloo, never over the GPUs
    _lib.init(dev)

    cfg = GemmaConfig(**CONFIGS["gemma12b"])
    stack = GemmaStack(GemmaWeights.random(cfg, seed=0, device=dev))  # every replica regenerates the same weights from the seed
    wl = workloads.config2(seed=rank, first_id=24 * rank)             # and scores its own 24 contents
    ecfg = EngineConfig(token_budget=wl.token_budget, max_tokens=65536)
    scorer = Scorer(stack, ecfg, dev)

    # ---- device-resident leg: the packed batch, its masks, the read rows and the option columns are staged once
    pk = Packer(ecfg.token_budget, ecfg.max_tokens, ecfg.align_jobs, ecfg.min_stream)
    batches = [b for key, first, t in wl.items for b in pk.push((key, first), t)] + list(pk.flush())
    if len(batches) != 1 or batches[0].length != 27648:
        raise RuntimeError(f"configuration 2 should pack into one 27648-token forward, got {[b.length for b in batches]}")
    b = batches[0]
    sc, inputs, masks, st = stage_one(stack, b, dev, ecfg)
    W = stack.w.lm_weight
    ws = torch.empty(int(_lib.lib().spinf_option_logprobs_workspace_bytes(len(b.sel), W.shape[0], st["cols"].numel())), dtype=torch.uint8, device=dev)

    def step():
        rows = stack.forward(sc, b, inputs, masks, rows=st["sel"])
        return ops.option_logprobs(rows, W, st["cols"], None, ws)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    sync()
    _lib.last_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ops.PROFILE = []
    launches0 = ops.COUNTS["launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        lp = step()
    e1.record()
    sync()
    launches = ops.COUNTS["launches"] - launches0
    prof, ops.PROFILE = ops.PROFILE, None
    ms = e0.elapsed_time(e1)
    _lib.last_status()
    if not bool(torch.isfinite(lp).all()):
        raise RuntimeError("non-finite log-probs")

    # ---- end-to-end leg: ONE public call with host inputs over the contents of all the steps (a bulk request of `steps` x 24
    # contents; the 27648-token budget makes every forward the shape of the resident leg's step)
    for _ in range(min(args.warmup, 2)):
        scorer.score_grouped(wl.items)
    bulk = [((s,) + tuple(key), first, tree) for s in range(args.steps) for key, first, tree in wl.items]
    s0 = (scorer.stats.forwards, scorer.stats.tokens, scorer.stats.h2d_bytes, scorer.stats.d2h_bytes, scorer.stats.stall_s)
    sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    out = scorer.score_grouped(bulk)
    f1.record()
    sync()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    forwards = scorer.stats.forwards - s0[0]
    e2e_tokens = scorer.stats.tokens - s0[1]
    h2d, d2h = scorer.stats.h2d_bytes - s0[2], scorer.stats.d2h_bytes - s0[3]
    scored = sum(1 for v in out.values() for x in v if x is not None)

    attn1 = attention_alone(dev, _peaks()) if rank == 0 and not args.no_attention else None
    bulk_block = bulk_leg(args, stack, dev, rank, world, sync, host_group) if args.bulk_contents > 0 else None

    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        peaks = _peaks()
        fp8 = measure_fp8_peak(dev)
        gemm = [(a.elapsed_time(c), f) for a, c, f, kind in prof if kind == "fp8_gemm"]
        gemm_ms, gemm_flops = sum(t for t, _ in gemm), sum(f for _, f in gemm)
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        attn_ms = {w: sum(a.elapsed_time(c) for a, c, _, kind in prof if kind == f"attn:{w}") for w in (0, cfg.window)}
        n_full = sum(1 for t in cfg.layer_types if t == "full_attention")
        pairs = {0: workloads.attended_pairs(b), cfg.window: workloads.attended_pairs(b, cfg.window)}
        attn_flops = 4.0 * cfg.head_dim * cfg.heads * (pairs[0] * n_full + pairs[cfg.window] * (cfg.layers - n_full)) * args.steps
        attn_total_ms = sum(attn_ms.values())
        step_flops = workloads.gemm_flops(cfg, wl.n_tokens) + workloads.head_flops(cfg, wl.n_questions)
        line = {
            "metric": METRIC, "value": world * wl.n_questions * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {
                "workload": WORKLOAD, "per_gpu": "24 contents / 1344 questions / 27408 tokens per step", "parallelism": f"{world} replicas, content-sharded",
                "l2": "inputs larger than L2 (10.8 GB of weights and >2 GB of activations per step)",
                "tiles_visited": masks["full_attention"].visited, "tiles_skipped_fraction": round(masks["full_attention"].skipped_fraction, 4),
            },
            "e2e": {
                "value": world * scored / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / max(forwards, 1),
                "h2d_bytes_per_step": int(h2d // max(forwards, 1)), "d2h_bytes_per_step": int(d2h // max(forwards, 1)),
                "forwards": forwards, "tokens": e2e_tokens, "questions_scored_per_gpu": scored, "forwards_match_steps": forwards == args.steps,
                "waited_for_packing_s": round(scorer.stats.stall_s - s0[4], 3),
            },
            "gpu_launches": int(launches),
            "roofline": {
                "kernel": "gemm_tc_kernel<fp8, 256, *> (row-wise fp8 linear: q|k|v, o, gate|up with the GeGLU epilogue, down)", "bound": "tensor",
                "achieved": achieved, "peak": fp8["sustained"], "unit": "TFLOP/s", "frac": achieved / fp8["sustained"],
                "peak_source": "library per-tensor fp8 GEMM 8192^3 measured in this run, back to back for 2 s (the kernel is timed inside a long step)",
                "peak_burst": fp8["burst"], "frac_of_burst": achieved / fp8["burst"], "frac_of_nominal_4500": achieved / 4500.0,
                "bf16_peaks": {"burst": peaks["bf16_burst"], "sustained": peaks["bf16_sustained"], "source": peaks["source"]},
                "traffic": 588.8e6 / 966.4e9 * (gemm_flops / max(len(gemm), 1)),
                "traffic_source": "not measured in this run: DRAM bytes of an ncu capture of the down-projection shape at M = 8192 (588.8 MB per 966.4 GFLOP), scaled by FLOPs to this run's average launch",
                "launches": len(gemm), "share_of_step": gemm_ms / ms if ms > 0 else None,
                "step_tflops_all_kernels": step_flops * args.steps / (ms * 1e-3) / 1e12,
            },
            "attention": {
                "in_step": {
                    "ms_per_step": attn_total_ms / args.steps, "share_of_step": attn_total_ms / ms if ms > 0 else None,
                    "unmasked_tflop_per_step": attn_flops / args.steps / 1e12,
                    "tflops_unmasked": attn_flops / (attn_total_ms * 1e-3) / 1e12 if attn_total_ms > 0 else None,
                    "frac_of_bf16_sustained": attn_flops / (attn_total_ms * 1e-3) / 1e12 / peaks["bf16_sustained"] if attn_total_ms > 0 else None,
                },
                "alone_cfg1": attn1,
            },
            "bulk": bulk_block,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(os.cpu_count() or 1)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def other_config_arm(args):
    """--config 4 / 5: the same two legs (resident and end to end) on the other single-GPU benchmark configurations, full models at
    full depth: 4 = the Gemma-style 31B-class fp8 model over contents of a 1000-token trunk + 32 questions of 16 tokens with 5
    options (21 contents = 672 questions per 32256-token forward); 5 = the Qwen-style 27B hybrid with int4 weights over contents of a
    2000-token trunk + 32 questions of 20 tokens with 5 options (12 contents = 384 questions per 32256-token forward)"""
    import torch
    import torch.distributed as dist

    from spinf_serve_b200 import _lib, ops, workloads
    from spinf_serve_b200.packer import Packer
    from spinf_serve_b200.scorer import EngineConfig, Scorer, stage_one

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the scoring path has no CPU fallback")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.init(dev)
    if args.config == 4:
        from spinf_serve_b200.gemma_stack import CONFIGS, GemmaConfig, GemmaStack, GemmaWeights

        cfg = GemmaConfig(**CONFIGS["gemma31b"])
        stack = GemmaStack(GemmaWeights.random(cfg, seed=0, device=dev))
        per, name = 21, "cfg4: gemma-style 31B-class fp8 row-wise (60 layers, hidden 5376, 32 / 16 heads of 128), 21 contents x (1000-token trunk + 32 questions x 16 tokens, 5 single-token options), one 32256-token forward"
        wl = workloads.fixed("cfg4", per, 1000, 32, 16, 5, 262144, per * 1536, seed=rank, first_id=per * rank)
        kernel, kind, dtype = "gemm_tc_kernel<fp8, 256, *> (row-wise fp8 linears)", "fp8_gemm", "fp8_e4m3"
    else:
        from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights

        cfg = QwenConfig()
        stack = QwenStack(QwenWeights.random(cfg, seed=0, device=dev))
        per, name = 12, "cfg5: qwen-style 27B hybrid, int4 group-128 weights (64 layers, 3 Gated DeltaNet : 1 attention, hidden 5120), 12 contents x (2000-token trunk + 32 questions x 20 tokens, 5 single-token options), one 32256-token forward"
        wl = workloads.fixed("cfg5", per, 2000, 32, 20, 5, 248320, per * 2688, seed=rank, first_id=per * rank)
        kernel, kind, dtype = "w4_gemm_kernel (int4 group-128 weight-only linears, bf16 tensor cores)", "w4_gemm", "int4_w_bf16_a"
    ecfg = EngineConfig(token_budget=wl.token_budget, max_tokens=65536)
    scorer = Scorer(stack, ecfg, dev)
    pk = Packer(ecfg.token_budget, ecfg.max_tokens, ecfg.align_jobs, ecfg.min_stream)
    (b,) = [x for key, first, t in wl.items for x in pk.push((key, first), t)] + list(pk.flush())
    sc, inputs, masks, st = stage_one(stack, b, dev, ecfg)
    W = stack.w.lm_weight
    ws = torch.empty(int(_lib.lib().spinf_option_logprobs_workspace_bytes(len(b.sel), W.shape[0], st["cols"].numel())), dtype=torch.uint8, device=dev)

    def step():
        rows = stack.forward(sc, b, inputs, masks, rows=st["sel"])
        return ops.option_logprobs(rows, W, st["cols"], None, ws)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    sync()
    _lib.last_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ops.PROFILE = []
    launches0 = ops.COUNTS["launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        lp = step()
    e1.record()
    sync()
    launches = ops.COUNTS["launches"] - launches0
    prof, ops.PROFILE = ops.PROFILE, None
    ms = e0.elapsed_time(e1)
    _lib.last_status()
    if not bool(torch.isfinite(lp).all()):
        raise RuntimeError("non-finite log-probs")
    for _ in range(min(args.warmup, 2)):
        scorer.score_grouped(wl.items)
    bulk = [((s,) + tuple(key), first, tree) for s in range(args.steps) for key, first, tree in wl.items]
    s0 = (scorer.stats.forwards, scorer.stats.tokens, scorer.stats.h2d_bytes, scorer.stats.d2h_bytes)
    sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    out = scorer.score_grouped(bulk)
    f1.record()
    sync()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    forwards = scorer.stats.forwards - s0[0]
    scored = sum(1 for v in out.values() for x in v if x is not None)
    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        peaks = _peaks()
        gemm = [(x.elapsed_time(y), f) for x, y, f, k in prof if k == kind]
        gemm_ms, gemm_flops = sum(t for t, _ in gemm), sum(f for _, f in gemm)
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        if args.config == 4:
            fp8 = measure_fp8_peak(dev)
            peak, src = fp8["sustained"], "library per-tensor fp8 GEMM 8192^3 measured in this run, back to back for 2 s"
        else:
            peak, src = peaks["bf16_sustained"], f"bf16 matmul 8192^3 back to back, {peaks['source']} (MEASURED_PEAKS.json)"
        line = {
            "metric": METRIC, "value": world * wl.n_questions * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype,
            "data": "synthetic",
            "config": {"workload": name, "per_gpu": f"{per} contents / {wl.n_questions} questions / {wl.n_tokens} tokens per step",
                       "parallelism": f"{world} replicas, content-sharded", "l2": "inputs larger than L2 (weights and activations of a full-depth forward)"},
            "e2e": {"value": world * scored / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / max(forwards, 1),
                    "h2d_bytes_per_step": int((scorer.stats.h2d_bytes - s0[2]) // max(forwards, 1)),
                    "d2h_bytes_per_step": int((scorer.stats.d2h_bytes - s0[3]) // max(forwards, 1)), "forwards": forwards,
                    "tokens": scorer.stats.tokens - s0[1], "forwards_match_steps": forwards == args.steps},
            "gpu_launches": int(launches),
            "roofline": {"kernel": kernel, "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": src, "traffic": None, "launches": len(gemm), "share_of_step": gemm_ms / ms if ms > 0 else None},
            "clocks": clocks,
        }
        attn_ms = sum(x.elapsed_time(y) for x, y, _, k in prof if k.startswith("attn:"))
        line["attention"] = {"ms_per_step": attn_ms / args.steps, "share_of_step": attn_ms / ms}
        gdn = [(x.elapsed_time(y), f) for x, y, f, k in prof if k == "gdn"]
        if gdn:
            g_ms, g_bytes = sum(t for t, _ in gdn), sum(f for _, f in gdn)
            line["recurrence"] = {
                "kernel": "gdn_tree_prep + gdn_tree_scan_tc (one layer pass = one preparation launch + one scan launch per level)", "bound": "hbm",
                "ms_per_layer_pass": g_ms / len(gdn), "achieved": g_bytes / (g_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": g_bytes / (g_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "share_of_step": g_ms / ms, "layer_passes": len(gdn),
            }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 4, 5], help="benchmark configuration: 2 (the headline, default), 4 (31B-class fp8), 5 (27B hybrid int4)")
    ap.add_argument("--bulk-contents", type=int, default=2624, help="contents of the bulk (configuration-3) leg, about 160 passes; 0 skips the leg")
    ap.add_argument("--no-attention", action="store_true", help="skip the attention-alone (configuration-1) block")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle timing (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.config != 2:
        other_config_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
