"""Size-independent properties at the benchmark configurations' full layer shapes and stream sizes (depth reduced to keep the test
short): a content scores bit-identically alone and inside a 32 768-token bulk pass whose trunks run past the sliding window, on the
12B shapes (head_dim 256) and the 31B-class shapes (head_dim 128); every option log-prob is a log-probability."""

import numpy as np
import pytest
import torch

from oracle import head as OH

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,layers", [("gemma12b", 2), ("gemma31b", 1)])
def test_bulk_pass_at_full_width_is_batch_invariant(dev, name, layers):
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.gemma_stack import CONFIGS, GemmaConfig, GemmaStack, GemmaWeights
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    cfg = GemmaConfig(**{**CONFIGS[name], "layers": layers, "pattern": 2})  # one sliding and one full layer on the 12B shapes
    stack = GemmaStack(GemmaWeights.random(cfg, seed=1, device=dev))
    wl = workloads.config3(seed=0, n_contents=20)  # trunks 200-2000 tokens, 56 questions, 2-5 options: ~1.2 passes of 32 768
    sc = Scorer(stack, EngineConfig(token_budget=32768, max_tokens=65536), dev)
    bulk = sc.score_grouped(wl.items)
    assert sc.stats.forwards >= 2 and sc.stats.tokens == wl.n_tokens
    for key, _, tree in (wl.items[0], wl.items[7], wl.items[-1]):
        alone = sc.score_grouped([(key, 0, tree)])[key]
        assert len(alone) == 56
        for a, b in zip(alone, bulk[key]):
            assert np.array_equal(a, b)
    n_q = 0
    for key, _, tree in wl.items:
        for lp in bulk[key]:
            n_q += 1
            assert np.isfinite(lp).all() and (lp <= 0).all()
            p, residual = OH.read_probs(lp)
            assert abs(p.sum() - 1) < 1e-9 and 0.0 <= residual <= 1.0
    assert n_q == wl.n_questions
    del stack, sc
    torch.cuda.empty_cache()


def test_attention_at_full_stream_size_by_properties(dev):
    """the tree attention over a whole configuration-2 stream (27 648 tokens, 16 query / 8 KV heads of 256) through properties
    that need no oracle: with every value row of a KV head equal to one vector the output is that vector (the weights of a row sum
    to one, whatever the mask); the per-token output maxima match the stored output; and the first content's rows are bit-identical
    to the same content run alone"""
    from spinf_serve_b200 import attention as A
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.packer import Packer

    def batches(wl):
        pk = Packer(32768, 65536, True, 1024)
        return [b for key, first, t in wl.items for b in pk.push((key, first), t)] + list(pk.flush())

    (b,) = batches(workloads.config2(seed=0))
    (b1,) = batches(workloads.config2(seed=0, n_contents=1))
    n, H, Hkv, D = b.length, 16, 8, 256
    g = torch.Generator().manual_seed(0)
    q = torch.randn((n, H, D), generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
    masks = A.stream_masks(b.art, b.end, b.pos, 1024, dev, always_window=True)
    for kind in ("full_attention", "sliding_attention"):
        const = torch.randn((1, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
        out = A.tree_attention(q, k, const.expand(n, Hkv, D).contiguous(), masks[kind], D**-0.5)
        want = const.repeat_interleave(H // Hkv, dim=1).expand(n, H, D)
        assert (out.float() - want.float()).abs().max() <= 2.0**-7 * want.float().abs().max()
        amax = torch.zeros(n, dtype=torch.float32, device=dev)
        full = A.tree_attention(q, k, v, masks[kind], D**-0.5, row_amax=amax)
        assert torch.equal(amax, full.float().abs().amax(dim=(1, 2)))
        m1 = A.stream_masks(b1.art, b1.end, b1.pos, 1024, dev, always_window=True)
        n1 = b1.length
        alone = A.tree_attention(q[:n1].contiguous(), k[:n1].contiguous(), v[:n1].contiguous(), m1[kind], D**-0.5)
        assert torch.equal(alone, full[:n1])


def _rand_bf16(shape, seed, dev, std=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=dev) * std).to(torch.bfloat16)


def test_fp8_linears_with_fused_epilogues_at_layer_shapes(dev):
    """configuration 2's layer shapes at M = 8192 rows: the q|k|v projection with norm + rotary in its epilogue and the gate|up
    projection with the GeGLU epilogue against the plain row-wise GEMM followed by the separate kernels (bit-equal for GeGLU and
    its quantisation; for q|k|v up to last-bit flips from the order of the fp32 sums of squares), and rows independent of M"""
    from spinf_serve_b200 import ops

    M, hidden, H, Hkv, D, F = 8192, 3840, 16, 8, 256, 15360
    x8, xs = ops.fp8_rowwise_quant(_rand_bf16((M, hidden), 1, dev))
    # q|k|v
    w8, ws = ops.fp8_rowwise_quant(_rand_bf16(((H + 2 * Hkv) * D, hidden), 2, dev, 0.02))
    wq, wk = 1 + 0.1 * _rand_bf16((D,), 3, dev).float(), 1 + 0.1 * _rand_bf16((D,), 4, dev).float()
    wq, wk = wq.to(torch.bfloat16), wk.to(torch.bfloat16)
    pos = torch.arange(M, dtype=torch.int32, device=dev) % 1500
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(dev)
    cos, sin = ops.rope_table(pos, inv_freq)
    ref = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    ops.qkv_norm_rope(ref, H, Hkv, D, wq, wk, cos, sin, 1e-6)
    got = ops.fp8_gemm_qkv(x8, xs, w8, ws, H, Hkv, D, wq, wk, cos, sin, 1e-6)
    assert (got.float() != ref.float()).float().mean().item() < 2e-3
    assert (got.float() - ref.float()).abs().max() <= 2.0**-6 * ref.float().abs().max()
    part = ops.fp8_gemm_qkv(x8[:1000].contiguous(), xs[:1000].contiguous(), w8, ws, H, Hkv, D, wq, wk, cos[:1000].contiguous(),
                            sin[:1000].contiguous(), 1e-6)
    assert torch.equal(part, got[:1000])
    del ref, got, part, w8
    # gate|up
    g8, gs = ops.fp8_rowwise_quant(_rand_bf16((2 * F, hidden), 5, dev, 0.02))
    gu = ops.fp8_rowwise_gemm(x8, xs, g8, gs)
    u8, us, y_ref = ops.glu_quant(gu, "gelu_tanh", want_fp8=True, want_y=True)
    del gu
    order = ops.glu_tile_order(F).to(dev)
    f8, fs, y = ops.fp8_gemm_glu(x8, xs, g8.view(torch.uint8)[order].view(torch.float8_e4m3fn).contiguous(), gs.reshape(-1)[order].contiguous())
    assert torch.equal(y, y_ref) and torch.equal(fs, us) and torch.equal(f8.view(torch.uint8), u8.view(torch.uint8))


def test_fused_norm_at_full_stream_size(dev):
    """the post-attention chain (norm, residual add, norm, row-wise fp8) over a whole 27 648 x 3840 stream: rows sampled across the
    stream against the oracle's module arithmetic, every row's scale equal to its quantised maximum / 448, and the result
    independent of how many rows the call covers"""
    from oracle import gemma as OG
    from oracle import linears as OL
    from spinf_serve_b200 import ops

    n, hidden = 27648, 3840
    y, res = _rand_bf16((n, hidden), 1, dev, 2.0), _rand_bf16((n, hidden), 2, dev, 30.0)
    w1 = (1 + 0.1 * _rand_bf16((hidden,), 3, dev).float()).to(torch.bfloat16)
    w2 = (1 + 0.1 * _rand_bf16((hidden,), 4, dev).float()).to(torch.bfloat16)
    r = ops.fused_norm(y, w1=w1, residual=res, w2=w2, eps=1e-6, want_h=True, want_norm=True, want_fp8=True)
    # (the quotient on the CPU: a division by a scalar on the GPU becomes a multiplication by its reciprocal)
    assert torch.equal(r["xs"].reshape(-1).cpu(), r["norm"].float().abs().amax(1).clamp_min(1e-12).cpu() / 448.0)
    rows = torch.arange(0, n, 431, device=dev)
    h_ref = res[rows].cpu() + OG.rmsnorm(y[rows].cpu(), w1.cpu(), 1e-6)
    x_ref = OG.rmsnorm(h_ref, w2.cpu(), 1e-6)
    assert (r["h"][rows].cpu().float() != h_ref.float()).float().mean() < 1e-3
    assert (r["norm"][rows].cpu().float() != x_ref.float()).float().mean() < 2e-3
    k8, ks = OL.quant_act_row(r["norm"][rows].cpu())
    assert torch.equal(r["xs"][rows].cpu(), ks) and torch.equal(r["x8"][rows].cpu().view(torch.uint8), k8.view(torch.uint8))
    few = ops.fused_norm(y[:300].contiguous(), w1=w1, residual=res[:300].contiguous(), w2=w2, eps=1e-6, want_h=True, want_fp8=True)
    assert torch.equal(few["h"], r["h"][:300]) and torch.equal(few["x8"].view(torch.uint8), r["x8"][:300].view(torch.uint8))


def test_int4_linear_at_the_hybrid_models_widest_shape(dev):
    """the gate|up projection of configuration 5 (5120 -> 34 816, group 128) at M = 8192: against the bf16 GEMM on the dequantised
    weight (the same products, the weight rounded to bf16 once in both), and rows independent of M"""
    from spinf_serve_b200 import ops

    M, K, N, G = 8192, 5120, 34816, 128
    g = torch.Generator(device=dev).manual_seed(0)
    qw = torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8)
    sc = (torch.rand((N, K // G), generator=g, device=dev) * 0.02 + 0.005).to(torch.float16)
    x = _rand_bf16((M, K), 1, dev)
    qk = ops.w4_repack(qw)
    y = ops.w4_gemm(x, qk, sc, G)
    nib = torch.stack([qw & 15, qw >> 4], dim=-1).reshape(N, K).float() - 8.0
    wd = (nib.view(N, K // G, G) * sc.float()[:, :, None]).reshape(N, K).to(torch.bfloat16)
    ref = ops.bf16_gemm(x, wd)
    assert (y.float() - ref.float()).abs().max() <= 2.0**-6 * ref.float().abs().max()
    assert torch.equal(ops.w4_gemm(x[:777].contiguous(), qk, sc, G), y[:777])


def test_recurrence_forms_agree_at_the_hybrid_models_shape(dev):
    """configuration 5's recurrent layer (16 key / 32 value heads of 128) over a stream of 2 000-token trunks with 32 branches of
    20 tokens: the whole plan through the one-launch-per-level kernels, the plan's long segments through the per-call chunked kernels,
    and everything through the token-serial kernel agree to the chunk pipeline's bf16 operand roundings; rows outside every segment
    stay zero"""
    from spinf_serve_b200 import gdn, workloads
    from spinf_serve_b200.gdn_plan import tree_plan
    from spinf_serve_b200.packer import Packer

    wl = workloads.fixed("cfg5", 6, 2000, 32, 20, 2, 248320, 16384, 0)
    pk = Packer(16384, 65536, True, 1024)
    (b,) = [x for key, first, t in wl.items for x in pk.push((key, first), t)] + list(pk.flush())
    T, Hk, Hv, D = b.length, 16, 32, 128
    q = torch.nn.functional.normalize(_rand_bf16((T, Hk, D), 1, dev).float(), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(_rand_bf16((T, Hk, D), 2, dev).float(), dim=-1).to(torch.bfloat16)
    v = _rand_bf16((T, Hv, D), 3, dev)
    gl = -torch.rand((T, Hv), device=dev) * 0.1
    beta = torch.rand((T, Hv), device=dev).to(torch.bfloat16)
    real = b.art >= 0
    plan = tree_plan(b.prev, real, dev)
    assert any(c.kind == "chunked" for lv in plan.levels for c in lv) and any(c.kind == "recurrent" for lv in plan.levels for c in lv)
    fused = gdn.gdn_tree(q, k, v, gl, beta, plan)  # the one-launch-per-level kernels (every segment in the chunked form)
    serial_plan = tree_plan(b.prev, real, dev)
    for lv in serial_plan.levels:
        for c in lv:
            c.kind = "recurrent"
    gdn.FUSED = False
    try:
        mixed = gdn.gdn_tree(q, k, v, gl, beta, plan)          # the per-call kernels as the reference dispatches them
        serial = gdn.gdn_tree(q, k, v, gl, beta, serial_plan)  # everything token by token
    finally:
        gdn.FUSED = True
    r = torch.from_numpy(real).to(dev)
    big = serial[r].float().abs().max()
    assert (mixed[r].float() - serial[r].float()).abs().max() <= 2e-2 * big
    assert (fused[r].float() - serial[r].float()).abs().max() <= 2e-2 * big
    assert bool((mixed[~r] == 0).all()) and bool((fused[~r] == 0).all())


def test_option_read_at_full_vocabulary(dev):
    """configuration 2's read: 1 344 rows against the 262 144 x 3840 tied head, two option columns per question among the batch's
    union: sampled rows against torch's log_softmax of the same logits, every value a log-probability, rows independent of R"""
    from spinf_serve_b200 import ops

    R, hidden, vocab = 1344, 3840, 262144
    h = _rand_bf16((R, hidden), 1, dev)
    W = _rand_bf16((vocab, hidden), 2, dev, 0.02)
    cols = torch.sort(torch.randperm(vocab, device=dev)[:2688]).values.to(torch.int32)
    lp = ops.option_logprobs(h, W, cols, None)
    assert lp.shape == (R, 2688) and bool((lp <= 0).all()) and bool(torch.isfinite(lp).all())
    rows = torch.arange(0, R, 97, device=dev)
    ref = torch.log_softmax(h[rows].float() @ W.float().t(), dim=-1)[:, cols.long()]
    assert (lp[rows] - ref).abs().max() < 2e-3
    assert torch.equal(ops.option_logprobs(h[:100].contiguous(), W, cols, None), lp[:100])


def test_down_projection_shape_rows_and_exact_product(dev):
    """configuration 2's down projection (15 360 -> 3 840) at M = 8192: sampled rows against the float64 product of the same
    quantised operands, and rows independent of M"""
    from oracle import linears as OL
    from spinf_serve_b200 import ops

    M, K, N = 8192, 15360, 3840
    x8, xs = ops.fp8_rowwise_quant(_rand_bf16((M, K), 1, dev))
    w8, ws = ops.fp8_rowwise_quant(_rand_bf16((N, K), 2, dev, 0.02))
    y = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    rows = torch.arange(0, M, 521, device=dev)
    ref = OL.scaled_mm_rowwise(x8[rows].cpu(), xs[rows].cpu(), w8.cpu(), ws.cpu().reshape(1, -1), exact=True)
    err = (y[rows].cpu().double() - ref.double()).abs()
    assert bool((err <= 2.0**-7 * ref.double().abs() + 2.0**-14 * ref.double().abs().max()).all())
    assert torch.equal(ops.fp8_rowwise_gemm(x8[:1000].contiguous(), xs[:1000].contiguous(), w8, ws), y[:1000])


def test_decoding_step_at_the_12b_shapes(dev):
    """the extraction decoder at full width and depth: 4 groups x 1 500-token prefixes, 5 prompts x 6 beams, 48 layers; the step
    replayed from its CUDA graph equals the step launched eagerly bit for bit, its outputs are finite, and its time is printed"""
    import types

    from spinf_serve_b200 import decode as D
    from spinf_serve_b200.gemma_stack import CONFIGS, GemmaConfig, GemmaStack, GemmaWeights

    cfg = GemmaConfig(**CONFIGS["gemma12b"])
    stack = GemmaStack(GemmaWeights.random(cfg, seed=0, device=dev))
    G, J, P, T, beam = 4, 5, 1500, 12, 6
    gen = torch.Generator(device=dev).manual_seed(1)

    def kv(n):
        return tuple(torch.randn((n, cfg.kv_heads, cfg.head_dim), generator=gen, device=dev).to(torch.bfloat16) for _ in range(2))

    proto = []
    for gi in range(G):
        pre = {li: kv(min(P, cfg.window - 1) if cfg.layer_types[li] == "sliding_attention" else P) for li in range(cfg.layers)}
        proto.append((pre, [(types.SimpleNamespace(key=(gi, j), max_tokens=16), {li: kv(T) for li in range(cfg.layers)}) for j in range(J)]))
    times, outs = {}, {}
    for graphs in (False, True):
        groups = [D.Group(dict(pre), P, [(p, dict(t), T, None) for p, t in prompts]) for pre, prompts in proto]
        dec = D.Decoder(stack, groups, dev, beam=beam, graphs=graphs)
        tok = torch.randint(5, 1000, (dec.G, dec.Q), generator=torch.Generator().manual_seed(2)).to(dev)
        for s in range(3):
            out = dec.forward(tok, s)
        outs[graphs] = out.clone()
        torch.cuda.synchronize()
        ms = []
        for s in range(3, 11):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dec.forward(tok, s)
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        times[graphs] = sorted(ms)[len(ms) // 2]
        del dec
    print(f"decoding step, {G * J * beam} rows, {cfg.layers} layers: {times[True]:.2f} ms from its graph, {times[False]:.2f} ms launched eagerly")
    assert torch.equal(outs[False], outs[True]) and bool(torch.isfinite(outs[True].float()).all())


def test_hybrid_decoding_step_at_the_27b_shapes(dev):
    """the hybrid family's extraction decoder at full width and depth (64 layers, 48 of them recurrent, int4 linears): 2 groups x
    1 000-token prefixes, 3 prompts x 6 beams; graph replay equals eager bit for bit, outputs finite, time printed"""
    import types

    from spinf_serve_b200 import decode as D
    from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights

    cfg = QwenConfig()
    stack = QwenStack(QwenWeights.random(cfg, seed=0, device=dev))
    G, J, P, T, beam = 2, 3, 1000, 12, 6
    gen = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *s: torch.randn(s, generator=gen, device=dev).to(torch.bfloat16)  # noqa: E731
    unit = lambda *s: torch.nn.functional.normalize(torch.randn(s, generator=gen, device=dev), dim=-1).to(torch.bfloat16)  # noqa: E731
    att = [i for i in range(cfg.layers) if cfg.layer_types[i] == "full_attention"]
    rec = [i for i in range(cfg.layers) if i not in att]
    cd = 2 * cfg.hk * cfg.dk + cfg.hv * cfg.dv

    def make_groups():
        g2 = torch.Generator(device=dev).manual_seed(2)
        groups = []
        for gi in range(G):
            grp = D.Group({li: (rnd(P, cfg.kv_heads, cfg.head_dim), rnd(P, cfg.kv_heads, cfg.head_dim)) for li in att}, P)
            grp.extra = {"state": {li: torch.randn((cfg.hv, cfg.dk, cfg.dv), generator=g2, device=dev) * 0.05 for li in rec}, "tmpl": []}
            for j in range(J):
                grp.prompts.append((types.SimpleNamespace(key=(gi, j), max_tokens=8), {li: (rnd(T, cfg.kv_heads, cfg.head_dim), rnd(T, cfg.kv_heads, cfg.head_dim)) for li in att}, T, None))
                tok = {li: (unit(T, cfg.hk, cfg.dk), unit(T, cfg.hk, cfg.dk), rnd(T, cfg.hv, cfg.dv), -torch.rand((T, cfg.hv), generator=g2, device=dev) * 0.1,
                            torch.rand((T, cfg.hv), generator=g2, device=dev).to(torch.bfloat16)) for li in rec}
                grp.extra["tmpl"].append({"tok": tok, "pre": {li: rnd(3, cd) for li in rec}})
            groups.append(grp)
        return groups

    times, outs = {}, {}
    for graphs in (False, True):
        gen.manual_seed(1)
        dec = D.HybridDecoder(stack, make_groups(), dev, beam=beam, graphs=graphs)
        tok = torch.randint(5, 1000, (dec.G, dec.Q), generator=torch.Generator().manual_seed(2)).to(dev)
        for s in range(3):
            out = dec.forward(tok, s)
        outs[graphs] = out.clone()
        torch.cuda.synchronize()
        ms = []
        for s in range(3, 8):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dec.forward(tok, s)
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        times[graphs] = sorted(ms)[len(ms) // 2]
        del dec
    print(f"hybrid decoding step, {G * J * beam} rows, {cfg.layers} layers: {times[True]:.2f} ms from its graph, {times[False]:.2f} ms launched eagerly")
    assert torch.equal(outs[False], outs[True]) and bool(torch.isfinite(outs[True].float()).all())
