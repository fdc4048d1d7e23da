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
