"""CPU oracle of the extraction decoder's attention and of one decoding step (test infrastructure: only tests, the smoke check and
the benchmark's CPU legs import this package; the product never does).

Restates spinf_serve/decode.py: `_x_attention` (:71-104), the decoder's padded tensors (Decoder.__init__, :110-189) and the K/V
write of a step (GroupKV.update, :60-65). Layouts here are token-major ([..., tokens, kv heads, dim]) where the reference keeps
[..., kv heads, tokens, dim]; the arithmetic and its rounding points are the reference's: scores as bf16 products with fp32
accumulation rounded to bf16, scaling / soft cap / softmax in fp32 over (prefix | templates | generated), probabilities rounded to
bf16, each of the three value products rounded to bf16 and the three summed in fp32.
"""

import torch

NINF = torch.finfo(torch.float32).min


def x_attention(q, kp, vp, pos_p, kt, vt, pos_t, own_t, gk, gv, qpos, step, beam, scaling, window=None, softcap=None):
    """q [G, Q, H, d] bf16; prefix kp / vp [G, Lp, h, d] with positions pos_p [G, Lp] (-1 = padding); templates kt / vt [G, Tt, h, d]
    with positions pos_t and owning prompt own_t [G, Tt] (-1 = padding); generated gk / gv [G, Q, S, h, d] (slot-owned, tokens
    0..step written); qpos [G, Q] the queries' positions; slot s belongs to prompt s // beam -> [G, Q, H, d] bf16"""
    G, Q, H, d = q.shape
    h = kp.shape[2]
    r = H // h
    qq = q.reshape(G, Q, h, r, d)
    sp = torch.einsum("gqhrd,gkhd->ghrqk", qq, kp).float() * scaling
    st = torch.einsum("gqhrd,gkhd->ghrqk", qq, kt).float() * scaling
    sg = torch.einsum("gqhrd,gqshd->ghrqs", qq, gk).float() * scaling
    if softcap:
        sp, st, sg = (torch.tanh(x / softcap) * softcap for x in (sp, st, sg))
    mp = (pos_p >= 0)[:, None, :].expand(G, Q, -1)
    mt = own_t[:, None, :] == (torch.arange(Q) // beam)[None, :, None]
    if window is not None:
        mp = mp & ((qpos[:, :, None] - pos_p[:, None, :]) < window)
        mt = mt & ((qpos[:, :, None] - pos_t[:, None, :]) < window)
    sp = sp.masked_fill(~mp[:, None, None], NINF)
    st = st.masked_fill(~mt[:, None, None], NINF)
    sg = sg.masked_fill(torch.arange(gk.shape[2]) > step, NINF)
    a = torch.softmax(torch.cat([sp, st, sg], -1), -1).to(vp.dtype)
    Lp, Lt = sp.shape[-1], st.shape[-1]
    out = torch.einsum("ghrqk,gkhd->gqhrd", a[..., :Lp], vp).float()
    out = out + torch.einsum("ghrqk,gkhd->gqhrd", a[..., Lp : Lp + Lt], vt).float()
    out = out + torch.einsum("ghrqs,gqshd->gqhrd", a[..., Lp + Lt :], gv).float()
    return out.reshape(G, Q, H, d).to(q.dtype)
