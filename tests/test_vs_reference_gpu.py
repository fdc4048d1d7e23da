"""Same-box comparison with the reference's own GPU operators: parity and speed, operator by operator, on this GPU.

The reference package is installed (unmodified) under baseline/_ref by the build container; where it is absent every test here
skips. Each test runs one reference operator exactly as the reference's modules call it, the library's counterpart on the same
tensors, compares the results and times both sides with CUDA events (20 repeats after warm-up). The numbers are collected in
vs_reference.json in the run's scratch output folder (the committed summary is made from it). A reference operator that does not run on
this GPU with the installed torch / triton / fla is recorded there as "reference GPU path unavailable on this box" with the error,
and its test skips: nothing here retries or works around a failing reference kernel.

    Fp8RowLinear          spinf_serve/quant/linears.py:29-33,84-96      torch.compile'd quantiser + row-wise torch._scaled_mm
    tree_flex_forward     spinf_serve/models/gemma4.py:99-119            compiled FlexAttention with the scorer's BlockMask
    gdn.recurrent/chunked spinf_serve/models/qwen35/gdn.py:109,197       Triton / fla kernels
    Scorer._logprobs      spinf_serve/scorer.py:340-355 (f32out)         torch.mm(out_dtype=float32) + log_softmax, 1024 rows at a time
    Int4Linear (bf16)     spinf_serve/models/qwen35/qwen.py:326-330,455-458   dq_bf16 + a bf16 matmul (a closure: its two lines are run here)"""

import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "spinf_serve")), reason="the reference is not installed under baseline/_ref")]

RESULTS = {}


@pytest.fixture(scope="module", autouse=True)
def _reference_on_path():
    sys.path.insert(0, REF)
    yield
    sys.path.remove(REF)
    out = os.environ.get("SPINF_VS_REFERENCE_OUT")  # a folder: the timings and parity figures of this run as vs_reference.json
    if out:
        os.makedirs(out, exist_ok=True)
        with open(os.path.join(out, "vs_reference.json"), "w") as f:
            json.dump(RESULTS, f, indent=1)


def timed(fn, repeats=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    ms.sort()
    return ms[len(ms) // 2]


def reference(op, fn):
    """runs a reference operator; a failure is recorded and skips the test"""
    try:
        out = fn()
        torch.cuda.synchronize()
        return out
    except Exception as e:  # noqa: BLE001
        RESULTS[op] = {"reference": "reference GPU path unavailable on this box", "error": f"{type(e).__name__}: {str(e)[:400]}"}
        pytest.skip(f"reference GPU path unavailable on this box for {op}: {type(e).__name__}")


def freevar(fn, name):
    return fn.__closure__[fn.__code__.co_freevars.index(name)].cell_contents


# ------------------------------------------------------------------------------------------------ a6: row-wise fp8 linear
@pytest.mark.parametrize("name,M,K,N", [("qkv", 27648, 3840, 8192), ("down", 27648, 15360, 3840)])
def test_fp8_rowwise_linear(dev, name, M, K, N):
    from spinf_serve.quant.linears import quant_linears

    from spinf_serve_b200 import ops
    from spinf_serve_b200.linears import quantize_weight_rowwise

    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    op = f"fp8_rowwise_linear_{name}_M{M}_K{K}_N{N}"
    lin = reference(op, lambda: quant_linears(None, dev).Fp8RowLinear(w))
    y_ref = reference(op, lambda: lin(x))
    quant_ref = freevar(type(lin).forward, "quant_act_row")
    x8_ref, xs_ref = quant_ref(x)

    w8, ws = quantize_weight_rowwise(w)
    x8, xs = ops.fp8_rowwise_quant(x)
    y = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    torch.cuda.synchronize()
    # weights: the same eager ops on the same device
    assert torch.equal(lin.w8t.t().contiguous().view(torch.uint8), w8.view(torch.uint8)) and torch.equal(lin.ws.reshape(-1), ws.reshape(-1))
    # activations: the reference's compiled quantiser may divide by a reciprocal; count what differs
    scale_same = float((xs_ref.reshape(-1) == xs.reshape(-1)).float().mean())
    scale_ulp = float(((xs_ref.reshape(-1).view(torch.int32) - xs.reshape(-1).view(torch.int32)).abs()).max())
    byte_same = float((x8_ref.view(torch.uint8) == x8.view(torch.uint8)).float().mean())
    d = (y.float() - y_ref.float()).abs()
    same = float((y == y_ref).float().mean())
    rel = float(d.max() / y_ref.float().abs().max())
    t_ref = timed(lambda: lin(x))
    t_ref_mm = timed(lambda: torch._scaled_mm(x8_ref, lin.w8t, scale_a=xs_ref, scale_b=lin.ws, out_dtype=torch.bfloat16))
    t_mine = timed(lambda: ops.fp8_rowwise_gemm(*ops.fp8_rowwise_quant(x), w8, ws))
    t_mine_mm = timed(lambda: ops.fp8_rowwise_gemm(x8, xs, w8, ws))
    RESULTS[op] = {
        "weights_bit_equal": True, "act_scale_equal_fraction": scale_same, "act_scale_max_ulp": scale_ulp, "act_bytes_equal_fraction": byte_same,
        "out_equal_fraction": same, "out_max_abs_over_max": rel, "ms_reference_linear": t_ref, "ms_reference_gemm_only": t_ref_mm,
        "ms_here_linear": t_mine, "ms_here_gemm_only": t_mine_mm, "tflops_reference_gemm": 2.0 * M * N * K / t_ref_mm / 1e9,
        "tflops_here_gemm": 2.0 * M * N * K / t_mine_mm / 1e9,
    }
    assert scale_ulp <= 1 and byte_same > 0.999  # a reciprocal multiply may move a scale by one ulp and a few bytes with it
    assert rel < 2.0**-6 and same > 0.98


# ------------------------------------------------------------------------------------------------ a5: tree attention
def _ref_flex():
    """the reference's registered attention callable, taken without disturbing this process's own "tree_flex" registration"""
    from spinf_serve.models.gemma4 import register_flex
    from transformers import AttentionInterface

    mine = AttentionInterface._global_mapping.pop("tree_flex", None)
    try:
        register_flex(None)
        return AttentionInterface._global_mapping.pop("tree_flex")
    finally:
        if mine is not None:
            AttentionInterface._global_mapping["tree_flex"] = mine


def _block_mask(b, window, dev, always_window=True):
    """Scorer._init_flex + _block_masks (spinf_serve/scorer.py:163-238) for one stream: the mask closures over device copies of
    art / end / pos and the reference packer's block tables"""
    from spinf_serve.packer import BLOCK, block_tables
    from torch.nn.attention.flex_attention import BlockMask

    art, end, pos = (torch.from_numpy(np.ascontiguousarray(a, np.int32)).to(dev) for a in (b.art, b.end, b.pos))

    def full(bb, h, q, k):
        return ((k <= q) & (art[q] >= 0) & (art[k] == art[q]) & (q < end[k])) | (q == k)

    def sliding(bb, h, q, k):
        return full(bb, h, q, k) & (pos[q] - pos[k] < window)

    tabs = block_tables(b.art, b.end, b.pos, window, None, always_window)
    n = b.length
    out = {}
    for name, ts, mod in (("full_attention", tabs[0], full), ("sliding_attention", tabs[1] or tabs[0], sliding if tabs[1] is not None else full)):
        pn, pi, fn, fi = [torch.from_numpy(t).to(dev) for t in ts]
        out[name] = BlockMask.from_kv_blocks(pn[None, None], pi[None, None], fn[None, None], fi[None, None], BLOCK_SIZE=BLOCK, mask_mod=mod,
                                             seq_lengths=(n, n), compute_q_blocks=False)
    return out


@pytest.mark.parametrize("case", ["cfg1", "cfg2_stream"])
def test_tree_attention(dev, case):
    from spinf_serve_b200 import attention as A
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.packer import Packer

    H, K, D = 16, 8, 256
    wl, budget = (workloads.config1(0), 16384) if case == "cfg1" else (workloads.config2(0), 27648)
    pk = Packer(budget, 65536, True, 1024)
    (b,) = [x for key, first, t in wl.items for x in pk.push((key, first), t)] + list(pk.flush())
    n = b.length
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((n, h, D), generator=g).to(torch.bfloat16).to(dev) for h in (H, K, K))
    op = f"tree_attention_{case}_n{n}"
    fn = reference(op, _ref_flex)
    masks_ref = reference(op, lambda: _block_mask(b, 1024, dev))
    masks = A.stream_masks(b.art, b.end, b.pos, 1024, dev, always_window=True)
    res = {}
    real = torch.from_numpy(b.art >= 0).to(dev)
    for kind in ("full_attention", "sliding_attention"):
        call = lambda kind=kind: fn(None, q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], masks_ref[kind], scaling=1.0 / 16)[0]  # noqa: E731
        o_ref = reference(op, call)[0]
        o = A.tree_attention(q, k, v, masks[kind], 1.0 / 16)
        torch.cuda.synchronize()
        d = (o.float() - o_ref.float())[real].abs()
        pairs = workloads.attended_pairs(b, 1024 if kind == "sliding_attention" else None)
        t_ref, t_mine = timed(call), timed(lambda kind=kind: A.tree_attention(q, k, v, masks[kind], 1.0 / 16))
        res[kind] = {
            "max_abs": float(d.max()), "mean_abs": float(d.mean()), "ref_abs_max": float(o_ref.float().abs().max()), "ms_reference": t_ref, "ms_here": t_mine,
            "speedup": t_ref / t_mine, "tflops_unmasked_reference": 4.0 * D * H * pairs / t_ref / 1e9, "tflops_unmasked_here": 4.0 * D * H * pairs / t_mine / 1e9,
        }
        # both sides round P to bf16 before P V and accumulate in fp32, in different tile orders
        assert float(d.max()) <= 2.0**-7 * float(o_ref.float().abs().max()) + 2e-3
    RESULTS[op] = res


# ------------------------------------------------------------------------------------------------ a8: gated delta rule
def _gdn_case(dev, seg_lens, Hk=16, Hv=32, seed=3):
    g = torch.Generator(device=dev).manual_seed(seed)
    T = int(sum(seg_lens))
    q = torch.nn.functional.normalize(torch.randn((1, T, Hk, 128), generator=g, device=dev), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn((1, T, Hk, 128), generator=g, device=dev), dim=-1).to(torch.bfloat16)
    v = torch.randn((1, T, Hv, 128), generator=g, device=dev).to(torch.bfloat16)
    gl = (-torch.rand((1, T, Hv), generator=g, device=dev) * 0.2).float()
    beta = torch.rand((1, T, Hv), generator=g, device=dev).to(torch.bfloat16)
    cu = torch.tensor(np.concatenate(([0], np.cumsum(seg_lens))), dtype=torch.int64)
    return q, k, v, gl, beta, cu


def test_gdn_recurrent(dev):
    """32 x 12 branches of 20 tokens, each forking one of 12 trunk states (the configuration-5 branch level)"""
    from spinf_serve.models.qwen35 import gdn as RG

    from spinf_serve_b200 import gdn as G

    n_seg, Hv = 384, 32
    q, k, v, gl, beta, cu = _gdn_case(dev, [20] * n_seg)
    h0 = torch.randn((12, Hv, 128, 128), generator=torch.Generator(device=dev).manual_seed(1), device=dev) * 0.1
    h0_idx = (torch.arange(n_seg, device=dev) // 32).to(torch.int64)
    cu_d = cu.to(dev)
    op = "gdn_recurrent_384x20_Hv32"
    o_ref = reference(op, lambda: RG.recurrent(q, k, v, gl, beta, 128**-0.5, cu_d, n_seg, h0, h0_idx))
    o = G.recurrent(q, k, v, gl, beta, 128**-0.5, cu_d, n_seg, h0, h0_idx)
    torch.cuda.synchronize()
    d = (o.float() - o_ref.float()).abs()
    t_ref = timed(lambda: RG.recurrent(q, k, v, gl, beta, 128**-0.5, cu_d, n_seg, h0, h0_idx))
    t_mine = timed(lambda: G.recurrent(q, k, v, gl, beta, 128**-0.5, cu_d, n_seg, h0, h0_idx))
    RESULTS[op] = {"max_abs": float(d.max()), "ref_abs_max": float(o_ref.float().abs().max()), "ms_reference": t_ref, "ms_here": t_mine, "speedup": t_ref / t_mine}
    assert float(d.max()) <= 2.0**-7 * float(o_ref.float().abs().max()) + 1e-3  # fp32 state both sides, bf16 outputs


def test_gdn_chunked(dev):
    """12 trunks of 2000 tokens (the configuration-5 trunk level), final states kept"""
    from spinf_serve.models.qwen35 import gdn as RG

    from spinf_serve_b200 import gdn as G

    n_seg, Hv = 12, 32
    q, k, v, gl, beta, cu = _gdn_case(dev, [2000] * n_seg)
    cu_d = cu.to(dev)
    ht_idx = torch.arange(n_seg, device=dev, dtype=torch.int64)
    op = "gdn_chunked_12x2000_Hv32"

    def ref():
        ht = torch.zeros((n_seg, Hv, 128, 128), dtype=torch.float32, device=dev)
        return RG.chunked(q, k, v, gl, beta, 128**-0.5, cu_d, cu, None, None, ht, ht_idx), ht

    def mine():
        ht = torch.zeros((n_seg, Hv, 128, 128), dtype=torch.float32, device=dev)
        return G.chunked(q, k, v, gl, beta, 128**-0.5, cu_d, cu, None, None, ht, ht_idx), ht

    o_ref, ht_ref = reference(op, ref)
    o, ht = mine()
    # the token-serial kernel (checked against the reference's own token-serial kernel above) as the third opinion
    ht_ser = torch.zeros((n_seg, Hv, 128, 128), dtype=torch.float32, device=dev)
    o_ser = G.recurrent(q, k, v, gl, beta, 128**-0.5, cu_d, n_seg, None, None, ht_ser, ht_idx)
    torch.cuda.synchronize()
    big = float(o_ser.float().abs().max())
    e_mine, e_ref = float((o.float() - o_ser.float()).abs().max()), float((o_ref.float() - o_ser.float()).abs().max())
    s_mine, s_ref = float((ht - ht_ser).abs().max()), float((ht_ref - ht_ser).abs().max())
    t_ref, t_mine = timed(ref, repeats=10), timed(mine, repeats=10)
    RESULTS[op] = {
        "out_abs_max": big, "here_vs_token_serial": e_mine, "reference_vs_token_serial": e_ref, "here_vs_reference": float((o.float() - o_ref.float()).abs().max()),
        "state_abs_max": float(ht_ser.abs().max()), "state_here_vs_token_serial": s_mine, "state_reference_vs_token_serial": s_ref,
        "ms_reference": t_ref, "ms_here": t_mine, "speedup": t_ref / t_mine,
    }
    # chunked forms carry bf16 operand roundings: the reference reports 4.9e-4 between its own two kernels on unit-scale data
    assert e_mine <= 2e-2 * big and s_mine <= 2e-2 * float(ht_ser.abs().max())
    if e_ref > 2e-2 * big:
        RESULTS[op]["note"] = "the reference's chunked path (installed fla, not the pinned 0.5.2) is off the token recurrence on this box"


def test_gdn_layer_pass_cfg5(dev):
    """one recurrent layer's pass over a configuration-5 stream (12 contents x (2000-token trunk + 32 branches of 20), 16 key /
    32 value heads): the reference's gdn_indexed loop (spinf_serve/models/qwen35/qwen.py:550-590) over its own kernels, against
    the fused kernels and the per-call kernels of this library, on the same plan"""
    from spinf_serve.models.qwen35 import gdn as RG

    from spinf_serve_b200 import gdn as G
    from spinf_serve_b200 import workloads
    from spinf_serve_b200.gdn_plan import tree_plan
    from spinf_serve_b200.packer import Packer

    wl = workloads.fixed("cfg5", 12, 2000, 32, 20, 2, 248320, 32768, 0)
    pk = Packer(32768, 65536, True, 1024)
    (b,) = [x for key, first, t in wl.items for x in pk.push((key, first), t)] + list(pk.flush())
    T, Hk, Hv = b.length, 16, 32
    g0 = torch.Generator(device=dev).manual_seed(7)
    q = torch.nn.functional.normalize(torch.randn((T, Hk, 128), generator=g0, device=dev), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn((T, Hk, 128), generator=g0, device=dev), dim=-1).to(torch.bfloat16)
    v = torch.randn((T, Hv, 128), generator=g0, device=dev).to(torch.bfloat16)
    gl = (-torch.rand((T, Hv), generator=g0, device=dev) * 0.1).float()
    beta = torch.rand((T, Hv), generator=g0, device=dev).to(torch.bfloat16)
    plan = tree_plan(b.prev, b.art >= 0, dev)
    real = torch.from_numpy(b.art >= 0).to(dev)
    op = f"gdn_layer_pass_cfg5_T{T}"

    def ref():  # gdn_indexed with rec_idx (the reference's production path)
        scale = 128**-0.5
        o = torch.zeros_like(v)
        prev = None
        for calls, nk in zip(plan.levels, plan.n_keep):
            states = q.new_empty((nk, Hv, 128, 128), dtype=torch.float32) if nk else None
            for c in calls:
                kw = dict(h0=prev if c.h0_idx is not None else None, h0_idx=c.h0_idx, ht=states if c.ht_idx is not None else None, ht_idx=c.ht_idx)
                if c.kind == "recurrent":
                    RG.recurrent(q[None], k[None], v[None], gl[None], beta[None], scale, c.cu, len(c.cu_cpu) - 1, idx=c.idx, o=o[None], **kw)
                    continue
                a = [x.index_select(0, c.idx)[None] for x in (q, k, v, gl, beta)]
                o.index_copy_(0, c.idx, RG.chunked(*a, scale, c.cu, c.cu_cpu, **kw)[0])
            prev = states
        return o

    def per_call():
        G.FUSED = False
        try:
            return G.gdn_tree(q, k, v, gl, beta, plan)
        finally:
            G.FUSED = True

    o_ref = reference(op, ref)
    o_fused = G.gdn_tree(q, k, v, gl, beta, plan)
    o_calls = per_call()
    torch.cuda.synchronize()
    big = float(o_calls[real].float().abs().max())
    t_ref, t_fused, t_calls = timed(ref, repeats=10), timed(lambda: G.gdn_tree(q, k, v, gl, beta, plan), repeats=10), timed(per_call, repeats=10)
    n_real = int(real.sum())
    alg_bytes = n_real * (2 * Hk * 128 * 2 + 2 * Hv * 128 * 2 + Hv * 6)  # q, k, v in, o out (bf16), g fp32, beta bf16
    RESULTS[op] = {
        "out_abs_max": big, "fused_vs_reference": float((o_fused - o_ref)[real].float().abs().max()), "fused_vs_per_call": float((o_fused - o_calls)[real].float().abs().max()),
        "reference_vs_per_call": float((o_ref - o_calls)[real].float().abs().max()), "ms_reference": t_ref, "ms_fused": t_fused, "ms_per_call_kernels": t_calls,
        "speedup_vs_reference": t_ref / t_fused, "algorithmic_mb": alg_bytes / 1e6, "gbs_fused": alg_bytes / t_fused / 1e6,
    }
    assert float((o_fused - o_calls)[real].float().abs().max()) <= 2e-2 * big
    assert bool((o_fused[~real] == 0).all())


# ------------------------------------------------------------------------------------------------ a10: lm-head read
def test_option_logprobs(dev):
    from spinf_serve_b200 import ops

    R, hidden, vocab = 1344, 3840, 262144
    g = torch.Generator(device=dev).manual_seed(2)
    h = torch.randn((R, hidden), generator=g, device=dev).to(torch.bfloat16)
    W = (torch.randn((vocab, hidden), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    cols = torch.from_numpy(np.sort(np.random.default_rng(0).choice(vocab, size=48, replace=False)).astype(np.int32)).to(dev)
    ci = cols.long()
    op = "option_logprobs_R1344_vocab262144"

    def ref():  # Scorer._forward's read with lm_head "f32out", lm_rows 1024, lm_fixed_rows (scorer.py:248-254, 327-355)
        out = []
        for s in range(0, R, 1024):
            x = h[s : s + 1024]
            m = x.shape[0]
            x = torch.nn.functional.pad(x, (0, 0, 0, 1024 - m))
            out.append(torch.log_softmax(torch.mm(x, W.t(), out_dtype=torch.float32).float(), dim=-1)[:m][:, ci])
        return torch.cat(out)

    lp_ref = reference(op, ref)
    lp = ops.option_logprobs(h, W, cols, None)
    torch.cuda.synchronize()
    d = float((lp - lp_ref).abs().max())
    t_ref, t_mine = timed(ref, repeats=10), timed(lambda: ops.option_logprobs(h, W, cols, None), repeats=10)
    RESULTS[op] = {"max_abs": d, "ms_reference": t_ref, "ms_here": t_mine, "speedup": t_ref / t_mine}
    assert d < 2e-3


# ------------------------------------------------------------------------------------------------ a7: int4 linear, bf16 mode
def test_int4_linear_bf16_mode(dev):
    """Int4Linear lives in a closure of the reference's build_model (it needs a checkpoint directory), so its bf16 branch is run
    here line by line: the unpacking of Int4Linear.__init__ (qwen.py:386-392), dq_bf16 (qwen.py:326-330) and the matmul of
    forward (qwen.py:455-458), in eager torch on the GPU"""
    from spinf_serve_b200.linears import Int4Linear

    M, K, N, G = 8192, 5120, 34816, 128
    g = torch.Generator(device=dev).manual_seed(4)
    qweight = torch.randint(-(2**31), 2**31 - 1, (K // 8, N), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
    scales = (torch.rand((K // G, N), generator=g, device=dev) * 0.01 + 0.002).to(torch.float16)
    x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
    sh = torch.arange(0, 32, 4, dtype=torch.int32, device=dev)
    qq = ((qweight[:, None, :] >> sh[None, :, None]) & 15).reshape(-1, N).t()
    q8 = (qq[:, 0::2] | (qq[:, 1::2] << 4)).to(torch.uint8).contiguous()
    s = scales.t().contiguous()

    def dq_bf16(q, s):
        o = q.shape[0]
        w = torch.stack([(q & 15), (q >> 4)], -1).view(o, -1, G).float() - 8.0
        return (w * s.float()[:, :, None]).view(o, -1).to(torch.bfloat16)

    op = f"int4_linear_bf16_M{M}_K{K}_N{N}"
    y_ref = reference(op, lambda: x @ dq_bf16(q8, s).t())
    lin = Int4Linear(qweight, scales)
    y = lin(x)
    torch.cuda.synchronize()
    d = (y.float() - y_ref.float()).abs()
    same = float((y == y_ref).float().mean())
    t_ref = timed(lambda: x @ dq_bf16(q8, s).t(), repeats=10)
    w_dense = dq_bf16(q8, s)
    t_ref_mm = timed(lambda: x @ w_dense.t(), repeats=10)
    t_mine = timed(lambda: lin(x), repeats=10)
    RESULTS[op] = {
        "out_equal_fraction": same, "max_abs_over_max": float(d.max() / y_ref.float().abs().max()), "ms_reference_dq_plus_gemm": t_ref, "ms_reference_gemm_only": t_ref_mm,
        "ms_here": t_mine, "speedup": t_ref / t_mine, "tflops_here": 2.0 * M * N * K / t_mine / 1e9, "tflops_reference": 2.0 * M * N * K / t_ref / 1e9,
    }
    assert float(d.max()) <= 2.0**-7 * float(y_ref.float().abs().max()) and same > 0.98


@pytest.mark.parametrize("M,N,K", [(36, 5120, 5120), (36, 34816, 5120), (36, 5120, 17408)])
def test_w4_small_linear(dev, M, N, K):
    """the decoding steps' W4A16 linear (spinf_serve/quant/w4gemm.py:44-66, a Triton kernel) at the hybrid model's widths"""
    from spinf_serve_b200 import ops

    g = torch.Generator().manual_seed(N + K)
    q = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g).to(dev)
    s = (torch.rand((N, K // 32), generator=g) * 0.02 + 0.001).to(torch.float16).to(dev)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(dev)

    def ref_fn():
        from spinf_serve.quant import w4gemm

        return w4gemm.linear(x, q, s)

    ref = reference("w4_small", ref_fn)
    got = ops.w4_small(x, q, s, 32)
    same = float((got == ref).float().mean())
    worst = float(((got.float() - ref.float()).abs() / (ref.float().abs() + 1e-2)).max())
    from spinf_serve.quant import w4gemm

    ws = torch.empty(int(ops._lib.lib().spinf_w4_small_workspace_bytes(M, N, K)), dtype=torch.uint8, device=dev)
    t_ref, t_mine = timed(lambda: w4gemm.linear(x, q, s)), timed(lambda: ops.w4_small(x, q, s, 32, workspace=ws))
    gbs = N * K / 2 / (t_mine * 1e-3) / 1e9
    RESULTS[f"w4_small_{N}x{K}"] = {"equal_share": same, "max_rel": worst, "ref_ms": t_ref, "mine_ms": t_mine, "weight_GBs": gbs}
    print(f"w4 small M {M} N {N} K {K}: equal {same:.4%}, max rel {worst:.2e}; reference {t_ref:.3f} ms, here {t_mine:.3f} ms ({gbs:.0f} GB/s of int4 weights)")
    assert same > 0.99 and worst < 2.0**-6


def test_x_attention(dev):
    """the decoding step's attention as the reference runs it on the GPU (eager einsums, spinf_serve/decode.py:71-104) against the
    library's three kernels, at a 12B-like layer: 4 groups of 1 500-token prefixes, 5 prompts x 6 beams, 17 generated tokens"""
    import types

    from spinf_serve import decode as RD
    from spinf_serve_b200 import ops

    G, H, h, Dh, beam, J, Lp, T, S, step = 4, 16, 8, 256, 6, 5, 1500, 12, 17, 9
    Q, Tt = J * beam, J * T
    g = torch.Generator().manual_seed(77)
    rnd = lambda *s: torch.randn(s, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    q, kp, vp, kt, vt, gk, gv = rnd(G, Q, H, Dh), rnd(G, Lp, h, Dh), rnd(G, Lp, h, Dh), rnd(G, Tt, h, Dh), rnd(G, Tt, h, Dh), rnd(G, Q, S, h, Dh), rnd(G, Q, S, h, Dh)
    pos_p = torch.arange(Lp, device=dev)[None].expand(G, Lp).contiguous()
    pos_t = (Lp + torch.arange(Tt, device=dev) % T)[None].expand(G, Tt).contiguous()
    own_t = (torch.arange(Tt, device=dev) // T)[None].expand(G, Tt).contiguous()
    qpos = torch.full((G, Q), Lp + T + step, device=dev)
    d = types.SimpleNamespace()
    li = 0
    d.kp, d.vp, d.kt, d.vt = ({li: t.permute(0, 2, 1, 3).contiguous()} for t in (kp, vp, kt, vt))
    d.gk, d.gv = ({li: t.permute(0, 3, 1, 2, 4).contiguous()} for t in (gk, gv))
    d.pos_p, d.mask_p = {li: pos_p}, {li: (pos_p >= 0)[:, None, :].expand(G, Q, Lp)}
    d.pos_t, d.mask_t = pos_t, own_t[:, None, :] == (torch.arange(Q, device=dev) // beam)[None, :, None]
    d.step_t, d.gen_idx, d.qpos = torch.tensor([step], device=dev), torch.arange(S, device=dev), qpos
    qr = q.permute(0, 2, 1, 3).contiguous()
    res = {}
    for window in (None, 1024):
        def ref_fn(window=window):
            RD._CURRENT[0] = d
            try:
                return RD._x_attention(None, qr, ("x", li), ("x", li), None, scaling=1.0, sliding_window=window)[0]
            finally:
                RD._CURRENT[0] = None

        ref = reference("x_attention", ref_fn)
        i32 = lambda t: t.to(torch.int32).contiguous()  # noqa: E731
        st = torch.tensor([step], dtype=torch.int32, device=dev)
        mine = lambda window=window: ops.x_attention(q, kp, vp, i32(pos_p), kt, vt, i32(pos_t), i32(own_t), gk, gv, i32(qpos), st, beam, 1.0, window)  # noqa: E731
        got = mine()
        diff = (got.float() - ref.float()).abs()
        res[str(window)] = {"max_abs": float(diff.max()), "equal_share": float((diff == 0).float().mean()), "ref_ms": timed(ref_fn), "mine_ms": timed(mine)}
        print(f"x_attention window {window}: {res[str(window)]}")
        assert float(diff.max()) <= 2.0**-6 * float(ref.float().abs().max()) + 2e-3
    RESULTS["x_attention"] = res
