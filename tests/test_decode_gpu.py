"""GPU parity of the extraction decoder's pieces: the three-range attention kernel against the reference's own outputs (golden) and
the oracle, the few-row W4A16 linear against its oracle, the K/V capture and the decoding step against the oracle's step, a
decoded token against the packed forward of the same sequence, CUDA-graph replay against eager, and the beam search."""

import types

import numpy as np
import pytest
import torch

from oracle import decode as OD
from oracle import gemma as OG
from oracle import linears as OL
from spinf_serve_b200 import decode as D
from spinf_serve_b200 import ops
from spinf_serve_b200 import packer as P
from spinf_serve_b200.scorer import forward_one
from tests.golden.make_decode_golden import CASES
from tests.test_decode_host import golden_case

pytestmark = pytest.mark.gpu


def _to_dev(kw, dev):
    out = {}
    for k, v in kw.items():
        if isinstance(v, torch.Tensor):
            out[k] = v.to(dev).to(torch.int32 if v.dtype in (torch.int64, torch.int32) else v.dtype).contiguous()
        else:
            out[k] = v
    out["step"] = torch.tensor([kw["step"]], dtype=torch.int32, device=dev)
    return out


def _steps(mine, ref):
    """(share of differing elements, largest difference in bf16 steps of the reference value)"""
    d = (mine.float() - ref.float()).abs()
    return float((d > 0).float().mean()), float((d / (ref.float().abs() * 2.0**-8 + 1e-30)).max())


@pytest.mark.parametrize("i", range(len(CASES)))
def test_x_attention_against_the_reference_s_outputs(dev, i):
    kw, ref = golden_case(i)
    got = ops.x_attention(**_to_dev(kw, dev)).cpu()
    share, steps = _steps(got, ref)
    print(f"case {i}: {share:.3%} of elements differ, at most {steps:.1f} bf16 half-steps")
    # the products are summed in another order than the CPU's: a score or probability on a rounding boundary moves one bf16 step
    assert share < 0.02 and bool(((got.float() - ref.float()).abs() <= ref.float().abs() * 2.0**-6 + 2e-3).all())


@pytest.mark.parametrize("G,H,h,Dh,beam,J,Lp,Tt,S,step,window,softcap", [
    (2, 16, 8, 256, 6, 5, 700, 90, 17, 9, 512, None),   # 60 rows per kv head, sliding
    (1, 32, 16, 128, 6, 6, 300, 200, 9, 0, None, 30.0),  # 72 rows per kv head: two row passes
    (3, 4, 4, 64, 1, 3, 0, 10, 3, 2, None, None),       # no prefix at all
    (2, 8, 2, 128, 2, 2, 90, 0, 4, 1, None, None),      # no templates: prefix and generated tokens only
])
def test_x_attention_against_the_oracle(dev, G, H, h, Dh, beam, J, Lp, Tt, S, step, window, softcap):
    g = torch.Generator().manual_seed(G * 1000 + Lp)
    Q = J * beam
    rnd = lambda *s: torch.randn(s, generator=g).to(torch.bfloat16)  # noqa: E731
    pos_p = torch.full((G, Lp), -1, dtype=torch.int64)
    pos_t = torch.full((G, Tt), -1, dtype=torch.int64)
    own_t = torch.full((G, Tt), -1, dtype=torch.int64)
    base = torch.zeros((G, Q), dtype=torch.int64)
    for gi in range(G):
        n = Lp - 13 * gi if Lp else 0
        Pn = n + 5
        pos_p[gi, :n] = torch.arange(Pn - n, Pn)
        per = max(Tt - gi, 0) // J
        for j in range(J):
            pos_t[gi, j * per : (j + 1) * per] = torch.arange(Pn, Pn + per)
            own_t[gi, j * per : (j + 1) * per] = j
            base[gi, j * beam : (j + 1) * beam] = Pn + per
    kw = dict(q=rnd(G, Q, H, Dh), kp=rnd(G, Lp, h, Dh), vp=rnd(G, Lp, h, Dh), pos_p=pos_p, kt=rnd(G, Tt, h, Dh), vt=rnd(G, Tt, h, Dh), pos_t=pos_t,
              own_t=own_t, gk=rnd(G, Q, S, h, Dh), gv=rnd(G, Q, S, h, Dh), qpos=base + step, step=step, beam=beam, scaling=Dh**-0.5, window=window,
              softcap=softcap)
    ref = OD.x_attention(**kw)
    got = ops.x_attention(**_to_dev(kw, dev)).cpu()
    share, steps = _steps(got, ref)
    print(f"{share:.3%} of elements differ, at most {steps:.1f} bf16 half-steps")
    assert share < 0.02 and bool(((got.float() - ref.float()).abs() <= ref.float().abs() * 2.0**-6 + 2e-3).all())


@pytest.mark.parametrize("M,N,K,group,E", [(5, 96, 512, 32, 0), (40, 1024, 5120, 32, 48), (128, 200, 1024, 128, 0), (17, 6144, 2048, 64, 0)])
def test_w4_small_against_the_oracle(dev, M, N, K, group, E):
    g = torch.Generator().manual_seed(M + N)
    q = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    s = (torch.rand((N, K // group), generator=g) * 0.02 + 0.001).to(torch.float16)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    extra = (torch.randn((E, K), generator=g) * 0.05).to(torch.bfloat16) if E else None
    ref = OL.w4_small_linear(x, q, s, group, extra)
    exact = OL.w4_small_linear(x, q, s, group, extra, exact=True)
    got = ops.w4_small(x.to(dev), q.to(dev), s.to(dev), group, None if extra is None else extra.to(dev)).cpu()
    share, _ = _steps(got, ref)
    err = float(((got.double() - exact).abs() / (exact.abs() + 1e-2)).max())
    print(f"M {M} N {N} K {K}: {share:.3%} of elements differ from the oracle; largest error against the exact product {err:.2e}")
    # fp32 partial sums added in another order inside a K slice: a sum on a bf16 rounding boundary moves one step
    assert share < 0.01 and err < 2.0**-7


# ------------------------------------------------------------------------------------------------ capture + decoding steps
def _cfg(layers=4):
    return dict(layers=layers, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=4096, window=64, pattern=2)


def _trees(rng, spec):
    """spec: per group (prefix length, template lengths) -> GroupedTrees whose branches are extraction templates"""
    trees = []
    for gi, (n_prefix, Ts) in enumerate(spec):
        prefix = rng.integers(5, 4096, n_prefix).tolist()
        branches = [[20 + j] + rng.integers(5, 4096, T - 1).tolist() for j, T in enumerate(Ts)]  # distinct first tokens
        prompts = [types.SimpleNamespace(key=(gi, j), max_tokens=4) for j in range(len(Ts))]
        trees.append(P.GroupedTree(prefix, branches, [], [], xbranches=list(enumerate(prompts))))
    return trees


def _pack(trees):
    pk = P.Packer(4096, 8192, align=True)
    out = [b for j, t in enumerate(trees) for b in pk.push(j, t)] + list(pk.flush())
    (b,) = out
    return b


def _groups_from_capture(b, cap, hidden, n_layers):
    groups = []
    for o in b.owners:
        g = D.Group({li: cap["kv"][("p", id(o))][li] for li in range(n_layers)}, o.prefix_len)
        for bs, bl, pr in o.xbranches:
            g.prompts.append((pr, {li: cap["kv"][("t", pr.key)][li] for li in range(n_layers)}, bl, hidden[bs + bl - 1]))
        groups.append(g)
    return groups


def _oracle_decoder(ocfg, W, Q, b, scheme, beam, S, round_p=False):
    """the decoding step restated on the oracle: its own packed forward gives the K/V (taps), padded as Decoder.__init__ pads them.
    round_p: the packed forward with one legitimate rounding change (probabilities rounded to bf16 before P V, as the kernels and
    the reference's attention do): the yardstick for how far two correct implementations drift apart"""
    from oracle import attention as OA

    taps = {}
    exact = OA.tree_attention
    try:
        if round_p:
            OA.tree_attention = lambda *a, **k: exact(*a, **{**k, "round_p": True})
        hidden = OG.forward(ocfg, W, Q, b.ids, b.art, b.end, b.pos, taps=taps, scheme=scheme)
    finally:
        OA.tree_attention = exact
    G = len(b.owners)
    J = max(len(o.xbranches) for o in b.owners)
    Qn = J * beam
    Tt = max(sum(bl for _, bl, _ in o.xbranches) for o in b.owners)
    keep = ocfg.window - 1
    st = types.SimpleNamespace(hidden=hidden, layers=[])
    pos_t = torch.full((G, Tt), -1, dtype=torch.int64)
    own_t = torch.full((G, Tt), -1, dtype=torch.int64)
    base = torch.zeros((G, Qn), dtype=torch.int64)
    for gi, o in enumerate(b.owners):
        off = 0
        for j, (_, bl, _) in enumerate(o.xbranches):
            pos_t[gi, off : off + bl] = torch.arange(o.prefix_len, o.prefix_len + bl)
            own_t[gi, off : off + bl] = j
            base[gi, j * beam : (j + 1) * beam] = o.prefix_len + bl
            off += bl
    for i in range(ocfg.layers):
        sliding = ocfg.layer_types[i] == "sliding_attention"
        ns = [min(o.prefix_len, keep) if sliding else o.prefix_len for o in b.owners]
        Lp = max(ns)
        h, Dh = ocfg.kv_heads, ocfg.head_dim
        L = types.SimpleNamespace(kp=torch.zeros((G, Lp, h, Dh), dtype=torch.bfloat16), vp=torch.zeros((G, Lp, h, Dh), dtype=torch.bfloat16),
                                  pos_p=torch.full((G, Lp), -1, dtype=torch.int64), kt=torch.zeros((G, Tt, h, Dh), dtype=torch.bfloat16),
                                  vt=torch.zeros((G, Tt, h, Dh), dtype=torch.bfloat16), gk=torch.zeros((G, Qn, S, h, Dh), dtype=torch.bfloat16),
                                  gv=torch.zeros((G, Qn, S, h, Dh), dtype=torch.bfloat16))
        for gi, o in enumerate(b.owners):
            n = ns[gi]
            a0 = o.start + o.prefix_len - n
            L.kp[gi, :n], L.vp[gi, :n] = taps[i]["k"][a0 : a0 + n], taps[i]["v"][a0 : a0 + n]
            L.pos_p[gi, :n] = torch.arange(o.prefix_len - n, o.prefix_len)
            off = 0
            for bs, bl, _ in o.xbranches:
                L.kt[gi, off : off + bl], L.vt[gi, off : off + bl] = taps[i]["k"][bs : bs + bl], taps[i]["v"][bs : bs + bl]
                off += bl
        st.layers.append(L)
    st.pos_t, st.own_t, st.base, st.G, st.Q = pos_t, own_t, base, G, Qn

    def step(tokens, s, taps_out=None):
        qpos = base + s

        def attend(i, kind, q, k, v):
            L = st.layers[i]
            h, Dh = ocfg.kv_heads, ocfg.head_dim
            L.gk[:, :, s], L.gv[:, :, s] = k.reshape(G, Qn, h, Dh), v.reshape(G, Qn, h, Dh)
            window = ocfg.window if kind == "sliding_attention" else None
            return OD.x_attention(q.reshape(G, Qn, ocfg.heads, Dh), L.kp, L.vp, L.pos_p, L.kt, L.vt, pos_t, own_t, L.gk, L.gv, qpos, s, beam, 1.0,
                                  window).reshape(G * Qn, ocfg.heads, Dh)

        return OG.forward(ocfg, W, Q, tokens.reshape(-1).numpy(), None, None, qpos.reshape(-1).numpy().astype(np.int32), scheme=scheme,
                          attend=attend, taps=taps_out).reshape(G, Qn, -1)

    st.step = step
    return st


def _setup(dev, scheme, beam=2, spec=((70, (5, 9)), (130, (7,)))):
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights

    ocfg = OG.GemmaConfig(**_cfg())
    W = OG.init_weights(ocfg, seed=4)
    Q = OG.quantize(W, scheme)
    if scheme == "bf16":
        stack = GemmaStack(GemmaWeights.from_bf16(GemmaConfig(**_cfg()), W, dev, scheme="bf16"))
    else:
        stack = GemmaStack(GemmaWeights.from_quantized(GemmaConfig(**_cfg()), W, Q, dev))
    b = _pack(_trees(np.random.default_rng(3), spec))
    with stack.capture(None, b, b.owners) as cap:
        hidden = forward_one(stack, b, dev)[0]
    groups = _groups_from_capture(b, cap, hidden, ocfg.layers)
    return ocfg, W, Q, stack, b, cap, hidden, groups


def test_capture_holds_the_stream_s_keys_and_values(dev):
    ocfg, W, Q, stack, b, cap, hidden, groups = _setup(dev, "bf16")
    taps = {}
    forward_one(stack, b, dev, taps=taps)
    for o in b.owners:
        for li in range(ocfg.layers):
            k, v = cap["kv"][("p", id(o))][li]
            n = min(o.prefix_len, ocfg.window - 1) if ocfg.layer_types[li] == "sliding_attention" else o.prefix_len
            a0 = o.start + o.prefix_len - n
            assert k.shape == (n, ocfg.kv_heads, ocfg.head_dim)
            assert torch.equal(k, taps[li]["k"][a0 : a0 + n]) and torch.equal(v, taps[li]["v"][a0 : a0 + n])
            for bs, bl, pr in o.xbranches:
                k, v = cap["kv"][("t", pr.key)][li]
                # a template branch shorter than the window is kept whole on sliding layers too
                assert torch.equal(k, taps[li]["k"][bs : bs + bl]) and torch.equal(v, taps[li]["v"][bs : bs + bl])
    assert stack._cap is None  # the capture closed with its context


def test_decoding_steps_against_the_oracle(dev):
    """bf16 linears, so that the comparison is not blurred by fp8 re-quantisation: three steps of every slot against the oracle's
    decoder built from the oracle's own packed forward"""
    beam = 2
    ocfg, W, Q, stack, b, cap, hidden, groups = _setup(dev, "bf16", beam)
    dec = D.Decoder(stack, groups, dev, beam=beam)
    ora = _oracle_decoder(ocfg, W, Q, b, "bf16", beam, dec.S)
    pert = _oracle_decoder(ocfg, W, Q, b, "bf16", beam, dec.S, round_p=True)
    assert (dec.G, dec.Q, dec.S) == (ora.G, ora.Q, 5)
    rng = np.random.default_rng(5)
    for s in range(3):
        tokens = torch.from_numpy(rng.integers(5, 4096, (dec.G, dec.Q)))
        tg, to = {}, {}
        dec.tok_buf.copy_(tokens.to(dev))
        dec.qpos.copy_(dec.base + s)
        dec.step_t.fill_(s)
        dec.step32.fill_(s)
        inputs = {"ids": dec.tok_buf.reshape(1, -1), "pos": dec.qpos.reshape(1, -1)}
        got = stack.forward(None, None, inputs, None, attend=dec._attend, taps=tg).reshape(dec.G, dec.Q, -1).cpu().float()
        want = ora.step(tokens, s, to).float()
        live = torch.zeros(dec.G, dec.Q, dtype=torch.bool)  # group 1 has one prompt: its second prompt's slots attend to nothing real
        for gi, g in enumerate(dec.groups):
            live[gi, : len(g.prompts) * beam] = True
        lv = live.reshape(-1)
        for i in range(ocfg.layers):
            for key in ("q", "k", "v", "attn", "h"):
                a, r = tg[i][key].cpu().float()[lv], to[i][key].float()[lv]
                print(f"  step {s} layer {i} {key}: rms err / rms = {float((a - r).pow(2).mean().sqrt() / r.pow(2).mean().sqrt()):.3e}")
        # the first layer's inputs are the same on both sides: its attention output differs by bf16 steps only
        a, r = tg[0]["attn"].cpu().float()[lv], to[0]["attn"].float()[lv]
        assert float((a - r).pow(2).mean().sqrt() / r.pow(2).mean().sqrt()) < 4e-3
        rel = float((got - want)[live].pow(2).mean().sqrt() / want[live].pow(2).mean().sqrt())
        floor = float((pert.step(tokens, s).float() - want)[live].pow(2).mean().sqrt() / want[live].pow(2).mean().sqrt())
        print(f"step {s}: hidden rms err / rms = {rel:.3e} (oracle's own rounding sensitivity {floor:.3e})")
        assert rel < 3 * floor + 1e-3


@pytest.mark.parametrize("scheme", ["bf16", "fp8row"])
def test_decoded_token_equals_the_packed_forward_of_the_same_sequence(dev, scheme):
    """the hidden state of a slot after three decoded tokens against the packed forward over prefix + template + those tokens as
    one plain sequence, layer by layer. The linears are row-local (per-row quantisation in the fp8 scheme), so the two differ only
    where the two attention kernels round; the first layer's attention output must agree to bf16 steps."""
    beam = 2
    ocfg, W, Q, stack, b, cap, hidden, groups = _setup(dev, scheme, beam)
    trees = _trees(np.random.default_rng(3), ((70, (5, 9)), (130, (7,))))
    dec = D.Decoder(stack, groups, dev, beam=beam)
    rng = np.random.default_rng(6)
    toks = [torch.from_numpy(rng.integers(5, 4096, (dec.G, dec.Q))) for _ in range(3)]
    for s, t in enumerate(toks[:-1]):
        dec.forward(t.to(dev), s)
    tg = {}
    dec.tok_buf.copy_(toks[2].to(dev))
    dec.qpos.copy_(dec.base + 2)
    dec.step_t.fill_(2)
    dec.step32.fill_(2)
    stack.forward(None, None, {"ids": dec.tok_buf.reshape(1, -1), "pos": dec.qpos.reshape(1, -1)}, None, attend=dec._attend, taps=tg)
    rel = lambda a, r: float((a.float() - r.float()).pow(2).mean().sqrt() / r.float().pow(2).mean().sqrt())  # noqa: E731
    for ti, j, bm in ((0, 1, 0), (1, 0, 1)):
        gi = next(k for k, g in enumerate(dec.groups) if g.prompts[0][0].key[0] == ti)  # the packer orders the jobs by size
        slot = j * beam + bm
        seq = trees[ti].prefix + trees[ti].branches[j] + [int(t[gi, slot]) for t in toks]
        line = P.build_grouped_tree([seq + [1]], [P.ReadPlan.build([[7]])])
        pk = P.Packer(4096, 8192, align=True)
        (lb,) = list(pk.push(0, line)) + list(pk.flush())
        tp = {}
        forward_one(stack, lb, dev, taps=tp)
        row, drow = lb.owners[0].start + len(seq) - 1, gi * dec.Q + slot
        errs = {key: [rel(tg[i][key][drow], tp[i][key][row]) for i in range(ocfg.layers)] for key in ("q", "attn", "h")}
        print(f"{scheme} tree {ti} prompt {j} beam {bm}: decoded vs packed, rms err / rms per layer:", {k: ["%.2e" % e for e in v] for k, v in errs.items()})
        assert errs["q"][0] == 0.0 and errs["attn"][0] < 1e-2


def test_graph_replay_equals_eager_and_reorder_moves_the_beams(dev):
    beam = 2
    ocfg, W, Q, stack, b, cap, hidden, groups = _setup(dev, "fp8row", beam)
    _, _, _, _, _, _, _, groups2 = _setup(dev, "fp8row", beam)
    eager, graph = D.Decoder(stack, groups, dev, beam=beam), D.Decoder(stack, groups2, dev, beam=beam, graphs=True)
    rng = np.random.default_rng(7)
    for s in range(3):
        t = torch.from_numpy(rng.integers(5, 4096, (eager.G, eager.Q))).to(dev)
        a, c = eager.forward(t, s), graph.forward(t, s)
        assert torch.equal(a, c), s
    assert graph.graph is not None
    # reorder: slot 1 of group 0 takes slot 0's generated tokens; the next step of the two slots on the same token is then identical
    parent = torch.arange(eager.G * eager.Q, device=dev)
    parent[1] = 0
    eager.reorder(parent)
    t = torch.from_numpy(rng.integers(5, 4096, (eager.G, eager.Q))).to(dev)
    t[0, 1] = t[0, 0]
    out = eager.forward(t, 3)
    assert torch.equal(out[0, 0], out[0, 1])


def test_beam_search_returns_scored_answers(dev):
    beam = 3
    ocfg, W, Q, stack, b, cap, hidden, groups = _setup(dev, "fp8row", beam)
    dec = D.Decoder(stack, groups, dev, beam=beam)
    stop = [1, 2, 3]
    found = D.search_text(dec, stack.w.lm_weight, stop, banned_ids=[0], min_p=1e-9)
    assert set(found) == {(0, 0), (0, 1), (1, 0)}
    for key, answers in found.items():
        assert answers, key
        lps = [lp for _, lp in answers]
        assert lps == sorted(lps, reverse=True) and all(lp <= 1e-4 for lp in lps)
        assert all(1 <= len(toks) <= 4 and not set(toks) & set(stop) for toks, _ in answers)
    # the best answer's log-prob re-derived from scratch: the packed forward of prefix + template + answer, token by token
    trees = _trees(np.random.default_rng(3), ((70, (5, 9)), (130, (7,))))
    toks, lp = found[(0, 1)][0]
    seq = trees[0].prefix + trees[0].branches[1]
    line = P.build_grouped_tree([seq + toks + [1]], [P.ReadPlan.build([[7]])])
    pk = P.Packer(4096, 8192, align=True)
    (lb,) = list(pk.push(0, line)) + list(pk.flush())
    hs = forward_one(stack, lb, dev)[0]
    s0 = lb.owners[0].start
    total = 0.0
    for t, tok in enumerate(toks + [None]):
        row = hs[s0 + len(seq) - 1 + t][None].contiguous()
        cols = torch.tensor(sorted(stop + ([tok] if tok is not None else [])), dtype=torch.int64, device=dev)
        l = ops.option_logprobs(row, stack.w.lm_weight, cols.to(torch.int32))[0]
        if tok is None:
            total += float(torch.logsumexp(l[torch.searchsorted(cols, torch.tensor(stop, device=dev))], -1))
        else:
            total += float(l[int(torch.searchsorted(cols, torch.tensor([tok], device=dev))[0])])
    print(f"best answer of prompt (0, 1): {toks}, log-prob {lp:.4f}; re-scored by the packed forward {total:.4f}")
    assert abs(total - lp) < 0.15
