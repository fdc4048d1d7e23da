"""Writes tests/golden/decode_golden.npz: inputs and outputs of the reference's own decoding-step attention run on the CPU.

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_decode_golden.py <path of the reference checkout>

`_x_attention` (spinf_serve/decode.py:71-104) reads the running decoder's tensors through the module's `_CURRENT` slot; here a plain
object with those attributes stands in for the decoder (its constructor needs a scorer and a model), filled as Decoder.__init__
fills them (decode.py:123-177): padded prefixes with position -1, templates with their owners, the generated range written up to
the current step. The function is called exactly as transformers' attention interface calls it (key = ("x", layer)). Tensors are
recorded in the reference's layouts ([G, kv heads, tokens, dim]); the test moves them to token-major."""

import sys
import types

import numpy as np
import torch


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


CASES = [
    # G, H, h, D, beam, J, Lp (per group), templates (per group: lengths), S, step, window, softcap
    dict(G=2, H=4, h=2, D=64, beam=3, J=2, Lp=[37, 20], T=[[5, 9], [7]], S=6, step=3, window=None, softcap=None),
    dict(G=1, H=8, h=2, D=128, beam=6, J=3, Lp=[150], T=[[12, 3, 30]], S=17, step=0, window=64, softcap=None),
    dict(G=3, H=2, h=2, D=64, beam=2, J=1, Lp=[70, 0, 129], T=[[66], [4], [1]], S=5, step=4, window=40, softcap=30.0),
]


def build(case, seed):
    g = torch.Generator().manual_seed(seed)
    G, H, h, D, beam, J, S = (case[k] for k in ("G", "H", "h", "D", "beam", "J", "S"))
    Q = J * beam
    Lp = max(max(case["Lp"]), 1)
    Tt = max(sum(t) for t in case["T"])
    rnd = lambda *s: torch.randn(s, generator=g).to(torch.bfloat16)  # noqa: E731
    kp, vp = rnd(G, h, Lp, D), rnd(G, h, Lp, D)
    kt, vt = rnd(G, h, Tt, D), rnd(G, h, Tt, D)
    gk, gv = rnd(G, h, Q, S, D), rnd(G, h, Q, S, D)
    q = rnd(G, H, Q, D)
    pos_p = torch.full((G, Lp), -1, dtype=torch.int64)
    pos_t = torch.full((G, Tt), -1, dtype=torch.int64)
    own_t = torch.full((G, Tt), -1, dtype=torch.int64)
    base = torch.zeros((G, Q), dtype=torch.int64)
    for gi in range(G):
        P = case["Lp"][gi] + 11  # the stored prefix is the tail of a longer one, as on sliding layers
        n = case["Lp"][gi]
        pos_p[gi, :n] = torch.arange(P - n, P)
        o = 0
        for j, T in enumerate(case["T"][gi]):
            pos_t[gi, o : o + T] = torch.arange(P, P + T)
            own_t[gi, o : o + T] = j
            base[gi, j * beam : (j + 1) * beam] = P + T
            o += T
    return dict(q=q, kp=kp, vp=vp, kt=kt, vt=vt, gk=gk, gv=gv, pos_p=pos_p, pos_t=pos_t, own_t=own_t, base=base, Q=Q)


def main(ref_root):
    sys.path.insert(0, ref_root)
    from spinf_serve import decode as RD

    out = {}
    for i, case in enumerate(CASES):
        t = build(case, 500 + i)
        Q, G = t["Q"], case["G"]
        d = types.SimpleNamespace()
        li = 7
        d.kp, d.vp, d.kt, d.vt, d.gk, d.gv = ({li: t[k]} for k in ("kp", "vp", "kt", "vt", "gk", "gv"))
        d.pos_p = {li: t["pos_p"]}
        d.mask_p = {li: (t["pos_p"] >= 0)[:, None, :].expand(G, Q, t["pos_p"].shape[1])}
        d.pos_t = t["pos_t"]
        d.mask_t = t["own_t"][:, None, :] == (torch.arange(Q) // case["beam"])[None, :, None]
        d.step_t = torch.tensor([case["step"]])
        d.gen_idx = torch.arange(case["S"])
        d.qpos = t["base"] + case["step"]
        RD._CURRENT[0] = d
        try:
            y, _ = RD._x_attention(None, t["q"], ("x", li), ("x", li), None, scaling=1.0 if i != 1 else case["D"] ** -0.5,
                                   sliding_window=case["window"], softcap=case["softcap"])
        finally:
            RD._CURRENT[0] = None
        for k in ("q", "kp", "vp", "kt", "vt", "gk", "gv"):
            out[f"{k}{i}"] = bits(t[k])
        for k in ("pos_p", "pos_t", "own_t"):
            out[f"{k}{i}"] = t[k].numpy().astype(np.int32)
        out[f"qpos{i}"] = d.qpos.numpy().astype(np.int32)
        out[f"y{i}"] = bits(y)  # [G, Q, H, D]
    path = __file__.replace("make_decode_golden.py", "decode_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items() if k.startswith("y")})


if __name__ == "__main__":
    main(sys.argv[1])
