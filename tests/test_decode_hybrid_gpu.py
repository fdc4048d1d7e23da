"""GPU parity of the hybrid family's extraction decoder (qwen_stack.QwenStack.capture + decode.HybridDecoder): what the capture
keeps, the decoding steps against the same steps restated on the oracle (its own packed forward gives the captures), a decoded
token against the packed forward of the same sequence, graph replay and beam reorder."""

import types

import numpy as np
import pytest
import torch

from oracle import decode as OD
from oracle import gdn as OGD
from oracle import qwen as OQ
from spinf_serve_b200 import decode as D
from spinf_serve_b200 import packer as P
from spinf_serve_b200.gdn_plan import tree_plan
from spinf_serve_b200.scorer import forward_one
from tests.test_decode_gpu import _pack, _trees
from tests.test_qwen_gpu import SMALL

pytestmark = pytest.mark.gpu

SPEC = ((70, (5, 9)), (130, (7,)))
VOCAB = 2048


def _hybrid_trees(seed):
    trees = _trees(np.random.default_rng(seed), SPEC)
    for t in trees:  # the helper draws tokens below 4096: fold them into this model's vocabulary
        t.prefix = [x % VOCAB for x in t.prefix]
        t.branches = [[x % VOCAB for x in br] for br in t.branches]
    return trees


def _setup(dev, beam=2):
    from spinf_serve_b200.qwen_stack import QwenConfig, QwenStack, QwenWeights

    ocfg = OQ.QwenConfig(**SMALL)
    W = OQ.init_weights(ocfg, seed=3)
    stack = QwenStack(QwenWeights(QwenConfig(**SMALL), W, dev))
    b = _pack(_hybrid_trees(3))
    with stack.capture(None, b, b.owners) as cap:
        hidden = forward_one(stack, b, dev)[0]
    rec = [i for i in range(ocfg.layers) if ocfg.layer_types[i] == "linear_attention"]
    att = [i for i in range(ocfg.layers) if i not in rec]
    groups = []
    for o in b.owners:
        g = D.Group({li: cap["kv"][("p", id(o))][li] for li in att}, o.prefix_len)
        g.extra = {"state": {li: cap["extra"]["state"][("p", id(o))][li] for li in rec}, "tmpl": []}
        for bs, bl, pr in o.xbranches:
            key = ("t", pr.key)
            g.prompts.append((pr, {li: cap["kv"][key][li] for li in att}, bl, hidden[bs + bl - 1]))
            g.extra["tmpl"].append({"tok": {li: cap["extra"]["tok"][key][li] for li in rec}, "pre": {li: cap["extra"]["pre"][key][li] for li in rec}})
        groups.append(g)
    return ocfg, W, stack, b, groups, rec, att


def _oracle_decoder(ocfg, W, b, beam, S, rec, att):
    """the hybrid decoding step on the oracle: captures from the oracle's own packed forward (stream rows), the caches laid out as
    decode.HybridDecoder lays them out, a step = oracle.qwen.forward with the decoding attention and the re-run recurrence"""
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    caps = {}
    OQ.forward(ocfg, W, b.ids, b.art, b.end, b.pos, plan, caps=caps)
    conv = plan.conv.numpy()
    G = len(b.owners)
    J = max(len(o.xbranches) for o in b.owners)
    Q = J * beam
    n = G * Q
    Tt = max(sum(bl for _, bl, _ in o.xbranches) for o in b.owners)
    h, Dh, H = ocfg.kv_heads, ocfg.head_dim, ocfg.heads
    hk, hv, dk, dv = ocfg.hk, ocfg.hv, ocfg.dk, ocfg.dv
    cd = 2 * hk * dk + hv * dv
    bf = torch.bfloat16
    pos_t = torch.full((G, Tt), -1, dtype=torch.int64)
    own_t = torch.full((G, Tt), -1, dtype=torch.int64)
    base = torch.zeros((G, Q), dtype=torch.int64)
    slot_T, slot_t0 = np.zeros(n, np.int64), np.zeros(n, np.int64)
    r = 0
    spans = {}
    for gi, o in enumerate(b.owners):
        off = 0
        for j, (bs, bl, _) in enumerate(o.xbranches):
            pos_t[gi, off : off + bl] = torch.arange(o.prefix_len, o.prefix_len + bl)
            own_t[gi, off : off + bl] = j
            base[gi, j * beam : (j + 1) * beam] = o.prefix_len + bl
            sl = slice(gi * Q + j * beam, gi * Q + (j + 1) * beam)
            slot_T[sl], slot_t0[sl] = bl, r
            spans[(gi, j)] = (r, bs, bl, off)
            r += bl
            off += bl
    gen0 = r
    R = gen0 + n * S
    st = types.SimpleNamespace(G=G, Q=Q, att={}, rec={})
    for i in att:
        Lp = max(o.prefix_len for o in b.owners)
        L = types.SimpleNamespace(kp=torch.zeros((G, Lp, h, Dh), dtype=bf), vp=torch.zeros((G, Lp, h, Dh), dtype=bf), pos_p=torch.full((G, Lp), -1, dtype=torch.int64),
                                  kt=torch.zeros((G, Tt, h, Dh), dtype=bf), vt=torch.zeros((G, Tt, h, Dh), dtype=bf), gk=torch.zeros((G, Q, S, h, Dh), dtype=bf),
                                  gv=torch.zeros((G, Q, S, h, Dh), dtype=bf))
        for gi, o in enumerate(b.owners):
            P0 = o.prefix_len
            L.kp[gi, :P0], L.vp[gi, :P0] = caps[i]["k"][o.start : o.start + P0], caps[i]["v"][o.start : o.start + P0]
            L.pos_p[gi, :P0] = torch.arange(P0)
            for j in range(len(o.xbranches)):
                _, bs, bl, off = spans[(gi, j)]
                L.kt[gi, off : off + bl], L.vt[gi, off : off + bl] = caps[i]["k"][bs : bs + bl], caps[i]["v"][bs : bs + bl]
        st.att[i] = L
    for i in rec:
        c = caps[i]
        L = types.SimpleNamespace(cq=torch.zeros((R, hk, dk), dtype=bf), ck=torch.zeros((R, hk, dk), dtype=bf), cv=torch.zeros((R, hv, dv), dtype=bf),
                                  cg=torch.zeros((R, hv)), cb=torch.zeros((R, hv), dtype=bf), ring=torch.zeros((n, 3, cd), dtype=bf),
                                  h0=torch.zeros((G, hv, dk, dv)))
        # the prefixes' final states: the token recurrence over the prefix rows of the oracle's own q k v g beta
        lens = [o.prefix_len for o in b.owners]
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int64)
        idx = torch.cat([torch.arange(o.start, o.start + o.prefix_len) for o in b.owners])
        OGD.recurrent(c["q"], c["k"], c["v"], c["g"], c["beta"], dk**-0.5, cu, idx=idx, ht=L.h0, ht_idx=torch.arange(G))
        for gi, o in enumerate(b.owners):
            for j in range(len(o.xbranches)):
                a, bs, bl, _ = spans[(gi, j)]
                for name, dst in (("q", L.cq), ("k", L.ck), ("v", L.cv), ("g", L.cg), ("beta", L.cb)):
                    dst[a : a + bl] = c[name][bs : bs + bl]
                taps = conv[bs + bl - 1, 1:4]
                rows = torch.stack([c["y"][t, :cd] if 0 <= t < len(b.ids) else torch.zeros(cd, dtype=bf) for t in taps])
                L.ring[gi * Q + j * beam : gi * Q + (j + 1) * beam] = rows[None]
        st.rec[i] = L

    def step(tokens, s, advance=True):
        qpos = base + s
        cur = gen0 + np.arange(n) * S + s
        new_pre = {}

        def attend(i, q, k, v):
            L = st.att[i]
            L.gk[:, :, s], L.gv[:, :, s] = k.reshape(G, Q, h, Dh), v.reshape(G, Q, h, Dh)
            return OD.x_attention(q.reshape(G, Q, H, Dh), L.kp, L.vp, L.pos_p, L.kt, L.vt, pos_t, own_t, L.gk, L.gv, qpos, s, beam, Dh**-0.5).reshape(n, H, Dh)

        def recur(i, y):
            L, Wl = st.rec[i], W["layers"][i]
            ext = torch.cat([y, torch.cat([L.ring.reshape(3 * n, cd), torch.zeros((3 * n, y.shape[1] - cd), dtype=bf)], 1)])
            cidx = np.full((4 * n, 4), 4 * n, np.int64)
            sa = np.arange(n)
            cidx[:n] = np.stack([n + 3 * sa, n + 3 * sa + 1, n + 3 * sa + 2, sa], 1)
            q, k, v, z, g, beta = OGD.prologue(ext, cidx, Wl["conv_w"], Wl["A_log"], Wl["dt_bias"], hk, dk, hv, dv)
            for name, val, dst in (("q", q, L.cq), ("k", k, L.ck), ("v", v, L.cv), ("g", g, L.cg), ("beta", beta, L.cb)):
                dst[cur] = val[:n]
            new_pre[i] = y[:, :cd].clone()
            idx = torch.cat([torch.cat([slot_t0[sl] + torch.arange(int(slot_T[sl])), gen0 + sl * S + torch.arange(s + 1)]) for sl in range(n)])
            cu = torch.tensor([0] + list(np.cumsum(slot_T + s + 1)), dtype=torch.int64)
            o = torch.zeros((R, hv, dv), dtype=bf)
            OGD.recurrent(L.cq, L.ck, L.cv, L.cg, L.cb, dk**-0.5, cu, idx=idx, h0=L.h0, h0_idx=torch.arange(n) // Q, o=o)
            return o[cur], z[:n]

        out = OQ.forward(ocfg, W, tokens.reshape(-1).numpy(), None, None, qpos.reshape(-1).numpy().astype(np.int32), None, attend=attend, recur=recur)
        if advance:
            for i, pre in new_pre.items():
                st.rec[i].ring = torch.cat([st.rec[i].ring[:, 1:], pre[:, None]], 1)
        return out.reshape(G, Q, -1)

    st.step = step
    return st


def _rel(a, r):
    return float((a.float() - r.float()).pow(2).mean().sqrt() / r.float().pow(2).mean().sqrt())


def test_capture_holds_states_rows_and_rings(dev):
    ocfg, W, stack, b, groups, rec, att = _setup(dev)
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    caps = {}
    OQ.forward(ocfg, W, b.ids, b.art, b.end, b.pos, plan, caps=caps)
    li = rec[0]  # the first layer's inputs are the same on both sides: its captures agree to bf16 steps
    for g, o in zip(groups, b.owners, strict=True):
        S = torch.zeros((1, ocfg.hv, ocfg.dk, ocfg.dv))
        c = caps[li]
        OGD.recurrent(c["q"], c["k"], c["v"], c["g"], c["beta"], ocfg.dk**-0.5, torch.tensor([0, o.prefix_len]),
                      idx=torch.arange(o.start, o.start + o.prefix_len), ht=S, ht_idx=torch.arange(1))
        err = _rel(g.extra["state"][li].cpu(), S[0])
        print(f"prefix of {o.prefix_len} tokens: captured state vs the token recurrence, rms err / rms = {err:.3e}")
        assert err < 5e-3
        for j, (bs, bl, _) in enumerate(o.xbranches):
            q, k, v, gg, bb = g.extra["tmpl"][j]["tok"][li]
            assert _rel(q.cpu(), c["q"][bs : bs + bl]) < 5e-3 and _rel(v.cpu(), c["v"][bs : bs + bl]) < 5e-3
            assert _rel(gg.cpu(), c["g"][bs : bs + bl]) < 5e-3 and q.shape == (bl, ocfg.hk, ocfg.dk)
            pre = g.extra["tmpl"][j]["pre"][li].cpu()
            cd = 2 * ocfg.hk * ocfg.dk + ocfg.hv * ocfg.dv
            want = torch.stack([c["y"][t, :cd] for t in plan.conv.numpy()[bs + bl - 1, 1:4]])
            assert pre.shape == (3, cd) and _rel(pre, want) < 5e-3
        for a in att:
            k, v = g.prefix_kv[a]
            assert k.shape == (o.prefix_len, ocfg.kv_heads, ocfg.head_dim)


def test_decoding_steps_against_the_oracle(dev):
    beam = 2
    ocfg, W, stack, b, groups, rec, att = _setup(dev, beam)
    dec = D.HybridDecoder(stack, groups, dev, beam=beam)
    ora = _oracle_decoder(ocfg, W, b, beam, dec.S, rec, att)
    assert (dec.G, dec.Q) == (ora.G, ora.Q)
    live = torch.zeros(dec.G, dec.Q, dtype=torch.bool)
    for gi, g in enumerate(dec.groups):
        live[gi, : len(g.prompts) * beam] = True
    rng = np.random.default_rng(5)
    for s in range(3):
        tokens = torch.from_numpy(rng.integers(5, VOCAB, (dec.G, dec.Q)))
        got = dec.forward(tokens.to(dev), s).cpu().float()
        want = ora.step(tokens, s).float()
        err = _rel(got[live], want[live])
        print(f"step {s}: hidden rms err / rms = {err:.3e}")
        assert err < 3e-2  # bf16 activations through four layers, as the packed forward's own test


def test_decoded_token_equals_the_packed_forward_of_the_same_sequence(dev):
    beam = 2
    ocfg, W, stack, b, groups, rec, att = _setup(dev, beam)
    trees = _hybrid_trees(3)
    dec = D.HybridDecoder(stack, groups, dev, beam=beam)
    rng = np.random.default_rng(6)
    toks = [torch.from_numpy(rng.integers(5, VOCAB, (dec.G, dec.Q))) for _ in range(3)]
    for s, t in enumerate(toks):
        got = dec.forward(t.to(dev), s)
    for ti, j, bm in ((0, 1, 0), (1, 0, 1)):
        gi = next(k for k, g in enumerate(dec.groups) if g.prompts[0][0].key[0] == ti)
        slot = j * beam + bm
        seq = trees[ti].prefix + trees[ti].branches[j] + [int(t[gi, slot]) for t in toks]
        line = P.build_grouped_tree([seq + [1]], [P.ReadPlan.build([[7]])])
        pk = P.Packer(4096, 8192, align=True)
        (lb,) = list(pk.push(0, line)) + list(pk.flush())
        ref = forward_one(stack, lb, dev)[0][lb.owners[0].start + len(seq) - 1]
        err = _rel(got[gi, slot], ref)
        print(f"tree {ti} prompt {j} beam {bm}: decoded vs packed final hidden, rms err / rms = {err:.3e}")
        assert err < 5e-2


def test_graph_replay_and_reorder(dev):
    beam = 2
    _, _, stack, _, groups, _, _ = _setup(dev, beam)
    _, _, _, _, groups2, _, _ = _setup(dev, beam)
    eager, graph = D.HybridDecoder(stack, groups, dev, beam=beam), D.HybridDecoder(stack, groups2, dev, beam=beam, graphs=True)
    rng = np.random.default_rng(7)
    for s in range(3):
        t = torch.from_numpy(rng.integers(5, VOCAB, (eager.G, eager.Q))).to(dev)
        assert torch.equal(eager.forward(t, s), graph.forward(t, s)), s
    parent = torch.arange(eager.G * eager.Q, device=dev)
    parent[1] = 0
    eager.reorder(parent)
    t = torch.from_numpy(rng.integers(5, VOCAB, (eager.G, eager.Q))).to(dev)
    t[0, 1] = t[0, 0]
    out = eager.forward(t, 3)
    assert torch.equal(out[0, 0], out[0, 1])
