"""The oracle of the extraction decoder's attention against outputs of the reference's own `_x_attention` run on the CPU
(tests/golden/decode_golden.npz, written by tests/golden/make_decode_golden.py), and the decoder's memory estimates."""

import os
import types

import numpy as np
import torch

from oracle import decode as OD
from tests.golden.make_decode_golden import CASES

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "decode_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def golden_case(i):
    """-> (keyword arguments of oracle.decode.x_attention in token-major layouts, the reference's output [G, Q, H, D])"""
    c = CASES[i]
    kw = dict(
        q=bf16(G[f"q{i}"]).permute(0, 2, 1, 3).contiguous(),  # [G, H, Q, D] -> [G, Q, H, D]
        kp=bf16(G[f"kp{i}"]).permute(0, 2, 1, 3).contiguous(), vp=bf16(G[f"vp{i}"]).permute(0, 2, 1, 3).contiguous(),
        kt=bf16(G[f"kt{i}"]).permute(0, 2, 1, 3).contiguous(), vt=bf16(G[f"vt{i}"]).permute(0, 2, 1, 3).contiguous(),
        gk=bf16(G[f"gk{i}"]).permute(0, 2, 3, 1, 4).contiguous(), gv=bf16(G[f"gv{i}"]).permute(0, 2, 3, 1, 4).contiguous(),  # -> [G, Q, S, h, D]
        pos_p=torch.from_numpy(G[f"pos_p{i}"]), pos_t=torch.from_numpy(G[f"pos_t{i}"]), own_t=torch.from_numpy(G[f"own_t{i}"]),
        qpos=torch.from_numpy(G[f"qpos{i}"]), step=c["step"], beam=c["beam"], scaling=1.0 if i != 1 else c["D"] ** -0.5,
        window=c["window"], softcap=c["softcap"],
    )
    return kw, bf16(G[f"y{i}"])


def test_oracle_attention_is_the_reference_s():
    for i in range(len(CASES)):
        kw, ref = golden_case(i)
        mine = OD.x_attention(**kw)
        # the same ops in the same order on other strides: bit-equal but for products summed in another order (a bf16 step at most)
        d = (mine.float() - ref.float()).abs()
        assert float((d > 0).float().mean()) < 0.01, i
        assert bool((d <= ref.float().abs() * 2.0**-7 + 1e-6).all()), i


def test_memory_estimates_grow_with_padding():
    from spinf_serve_b200 import decode as D

    def group(P, Ts, max_tokens):
        kv = {0: (torch.zeros(P, 2, 8), torch.zeros(P, 2, 8)), 1: (torch.zeros(min(P, 15), 2, 8), torch.zeros(min(P, 15), 2, 8))}
        return D.Group(kv, P, [(types.SimpleNamespace(key=j, max_tokens=max_tokens), {}, T, None) for j, T in enumerate(Ts)])

    per = {0: 64, 1: 64}
    a, b = group(100, [5, 7], 16), group(30, [9], 64)
    for g in (a, b):  # one group alone: the chunk estimate is the group's own
        S = max(p.max_tokens for p, *_ in g.prompts) + 1
        assert D.chunk_bytes([g], per) == D.group_bytes(g, per, S)
    Sa, Sb = 17, 65
    assert D.chunk_bytes([a, b], per) > D.group_bytes(a, per, Sa) + D.group_bytes(b, per, Sb)
    assert D.group_bytes(a, per, Sa) == 64 * (100 + 12 + 2 * D.BEAM * 17) + 64 * (15 + 12 + 2 * D.BEAM * 17)


def _fake_hybrid(beam=2):
    """a two-layer stand-in for the hybrid stack (layer 0 recurrent, layer 1 attention) and two groups with CPU tensors: enough
    for decode.HybridDecoder's constructor, its per-step tables and its beam reorder, none of which launch a kernel"""
    from spinf_serve_b200 import decode as D

    cfg = types.SimpleNamespace(heads=2, kv_heads=1, head_dim=64, hk=1, hv=2, dk=128, dv=128)
    stack = types.SimpleNamespace(cfg=cfg, n_layers=2, w=types.SimpleNamespace(layers=[{"kind": "linear_attention"}, {"kind": "full_attention"}]))
    cd = 2 * cfg.hk * cfg.dk + cfg.hv * cfg.dv
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    groups = []
    for gi, (P, Ts) in enumerate(((9, (3, 2)), (5, (4,)))):
        grp = D.Group({1: (torch.randn((P, 1, 64), generator=g).to(bf), torch.randn((P, 1, 64), generator=g).to(bf))}, P)
        grp.extra = {"state": {0: torch.full((cfg.hv, cfg.dk, cfg.dv), float(gi + 1))}, "tmpl": []}
        for j, T in enumerate(Ts):
            grp.prompts.append((types.SimpleNamespace(key=(gi, j), max_tokens=3), {1: (torch.randn((T, 1, 64), generator=g).to(bf), torch.randn((T, 1, 64), generator=g).to(bf))}, T, None))
            tok = (torch.full((T, cfg.hk, cfg.dk), 10.0 * gi + j).to(bf), torch.zeros((T, cfg.hk, cfg.dk), dtype=bf), torch.zeros((T, cfg.hv, cfg.dv), dtype=bf),
                   torch.zeros((T, cfg.hv)), torch.zeros((T, cfg.hv), dtype=bf))
            grp.extra["tmpl"].append({"tok": {0: tok}, "pre": {0: torch.full((3, cd), 100.0 * gi + j).to(bf)}})
        groups.append(grp)
    return D.HybridDecoder(stack, groups, "cpu", beam=beam), cd


def test_hybrid_decoder_tables_and_reorder():
    beam = 2
    dec, cd = _fake_hybrid(beam)
    n, S = dec.n, dec.S
    assert (dec.G, dec.Q, S, n) == (2, 4, 4, 8) and dec.gen0 == 9 and dec.R == 9 + n * S
    # the templates' call: one segment per prompt slot (group 1 has one prompt: its second slot has no rows and passes the
    # prefix state on), from the group's prefix state into the prompt's entry of `ht`
    assert dec.t_cu.tolist() == [0, 3, 5, 9, 9] and dec.t_h0_idx.tolist() == [0, 0, 1, 1] and dec.t_ht_idx.tolist() == [0, 1, 2, 3]
    assert dec.ht.shape[0] == 4 and dec.slot_prompt.tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    # the slots' call: every slot's generated rows 0 .. step, from its prompt's entry
    for st in range(S):
        cu = dec.cu_all[st].tolist()
        assert cu == [s * (st + 1) for s in range(n + 1)]
        for s in range(n):
            assert dec.idx_all[st, cu[s] : cu[s + 1]].tolist() == [dec.gen0 + s * S + k for k in range(st + 1)]
    assert dec.h0_idx.tolist() == [0, 0, 0, 0, 1, 1, 1, 1] and float(dec.h0[0, 1, 0, 0, 0]) == 2.0
    assert dec.conv_idx[3].tolist() == [n + 9, n + 10, n + 11, 3]
    ring = dec.ybuf[0, n:].view(n, 3, -1)
    assert float(ring[2, 0, 0]) == 1.0 and float(ring[4, 2, cd - 1]) == 100.0 and float(ring[6].abs().max()) == 0.0
    assert float(dec.cq[0, 3, 0, 0]) == 1.0 and float(dec.cq[0, 5, 0, 0]) == 10.0  # template rows: prompt (0, 1) at 3.., (1, 0) at 5..
    # a step's tables, then the beams: slot 1 takes slot 0's generated rows and ring, slot 5 takes slot 4's
    dec._prepare(2)
    assert dec.cur_rows.tolist() == [dec.gen0 + s * S + 2 for s in range(n)] and torch.equal(dec.idx_buf, dec.idx_all[2])
    dec.cq[0, dec.gen0 : dec.gen0 + S] = 7.0
    ring[0] = 5.0
    dec.gk[1][0, 0] = 3.0
    parent = torch.arange(n)
    parent[1] = 0
    dec.reorder(parent)
    assert float(dec.cq[0, dec.gen0 + S, 0, 0]) == 7.0 and float(dec.ybuf[0, n:].view(n, 3, -1)[1, 1, 0]) == 5.0 and float(dec.gk[1][0, 1, 0, 0, 0]) == 3.0
    assert float(dec.cq[0, dec.gen0 + 2 * S, 0, 0]) == 0.0


def test_decoder_pads_groups_as_the_reference_s_does():
    """Decoder.__init__ on CPU tensors: padded prefixes carry position -1, a sliding layer's stored tail keeps its true positions,
    templates carry their owner, every slot starts right after its own template (decode.py:123-177)"""
    from spinf_serve_b200 import decode as D

    cfg = types.SimpleNamespace(heads=2, kv_heads=1, head_dim=64, window=8)
    stack = types.SimpleNamespace(cfg=cfg, n_layers=2)
    kv = lambda n: (torch.ones((n, 1, 64), dtype=torch.bfloat16), torch.ones((n, 1, 64), dtype=torch.bfloat16))  # noqa: E731
    groups = []
    for gi, (P, Ts) in enumerate(((20, (3, 2)), (5, (4,)))):
        g = D.Group({0: kv(min(P, cfg.window - 1)), 1: kv(P)}, P)  # layer 0 sliding: the last window - 1 tokens
        for j, T in enumerate(Ts):
            g.prompts.append((types.SimpleNamespace(key=(gi, j), max_tokens=5), {0: kv(T), 1: kv(T)}, T, None))
        groups.append(g)
    dec = D.Decoder(stack, groups, "cpu", beam=2)
    assert (dec.G, dec.Q, dec.S, dec.Tt) == (2, 4, 6, 5)
    assert dec.pos_p[0][0].tolist() == list(range(13, 20)) and dec.pos_p[0][1].tolist() == [0, 1, 2, 3, 4, -1, -1]
    assert dec.pos_p[1][1].tolist() == list(range(5)) + [-1] * 15 and float(dec.kp[1][1, 5:].abs().max()) == 0.0
    assert dec.pos_t[0].tolist() == [20, 21, 22, 20, 21] and dec.own_t[0].tolist() == [0, 0, 0, 1, 1]
    assert dec.pos_t[1].tolist() == [5, 6, 7, 8, -1] and dec.own_t[1].tolist() == [0, 0, 0, 0, -1]
    assert dec.base.tolist() == [[23, 23, 22, 22], [9, 9, 0, 0]]
    assert dec.gk[0].shape == (2, 4, 6, 1, 64) and groups[0].prefix_kv[0] is None  # the captures were let go
