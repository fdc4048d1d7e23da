"""Oracle of the Gated DeltaNet layer pieces (CPU torch; test infrastructure only, never imported by the product).

recurrent() restates the reference's token-by-token kernel (spinf_serve/models/qwen35/gdn.py:163-190) with its calling contract
(gdn.py:197-235): per segment and value head, state S [K, V] fp32 starting from h0[h0_idx] (or zero), per token
    S *= exp(g);  v' = (v - sum_k S[k, :] k[k]) * beta;  S += k (x) v';  o = sum_k S[k, :] (q[k] * scale)
and the final state written to ht[ht_idx] where ht_idx >= 0. The reference's chunked form (gdn.py:109-133, built on the third-party
fla kernels) computes the same recurrence in 64-token chunks; the reference measured the two forms 4.9e-4 apart in bf16.
gdn_tree() follows gdn_indexed (spinf_serve/models/qwen35/qwen.py:550-590): levels of a TreePlan, children start from their
parent's kept state. prologue() / epilogue() follow GatedDeltaNet.forward (qwen.py:640-673)."""

import numpy as np
import torch
import torch.nn.functional as F


def recurrent(q, k, v, g, beta, scale, cu, idx=None, h0=None, h0_idx=None, ht=None, ht_idx=None, o=None, dtype=torch.float32):
    """q, k [rows, Hk, K], v [rows, Hv, V], g, beta [rows, Hv]; cu [n + 1]; idx [sum of lengths] rows of the call's tokens (None:
    rows 0.. in call order) -> o [rows, Hv, V] (the rows touched are overwritten, in v's dtype). dtype: accumulation type."""
    rows, Hk, K = k.shape
    Hv, V = v.shape[1], v.shape[2]
    rep = Hv // Hk
    if o is None:
        o = torch.zeros_like(v)
    cu = [int(x) for x in cu]
    for n in range(len(cu) - 1):
        S = torch.zeros((Hv, K, V), dtype=dtype)
        if h0 is not None and h0_idx is not None and int(h0_idx[n]) >= 0:
            S = h0[int(h0_idx[n])].to(dtype).clone()
        for t in range(cu[n], cu[n + 1]):
            r = int(idx[t]) if idx is not None else t
            qt = q[r].to(dtype).repeat_interleave(rep, 0) * scale  # [Hv, K]
            kt = k[r].to(dtype).repeat_interleave(rep, 0)
            vt = v[r].to(dtype)
            S = S * torch.exp(g[r].to(dtype))[:, None, None]
            vn = (vt - torch.einsum("hkv,hk->hv", S, kt)) * beta[r].to(dtype)[:, None]
            S = S + kt[:, :, None] * vn[:, None, :]
            o[r] = torch.einsum("hkv,hk->hv", S, qt).to(o.dtype)
        if ht is not None and ht_idx is not None and int(ht_idx[n]) >= 0:
            ht[int(ht_idx[n])] = S.to(ht.dtype)
    return o


def chunked(q, k, v, g, beta, scale, cu, idx=None, h0=None, h0_idx=None, ht=None, ht_idx=None, o=None, chunk=64):
    """The same recurrence in the chunked (WY) form of the reference's gdn.chunked (spinf_serve/models/qwen35/gdn.py:109-133). That
    function runs kernels of a third-party dependency that is not part of the reference tree (flash-linear-attention, pinned 0.5.2:
    chunk_local_cumsum, chunk_scaled_dot_kkt_fwd, solve_tril, recompute_w_u_fwd, chunk_fwd_o) around the reference's own state
    kernel (gdn.py:21-106); this restates their published algorithm (Yang et al., Gated Delta Networks, the WY form) with their
    rounding points: bf16 operands into every product, fp32 accumulation and state. With G the running sum of g inside a chunk in
    log2 units:  A[t,s] = beta_t (k_t.k_s) 2^(G_t-G_s) (s < t);  T = (I+A)^-1;  W = T (beta K 2^G);  U = T (beta V);
    v' = U - W S;  o = scale ((Q S) 2^G + tril(Q K^T 2^(G_t-G_s)) v');  S <- S 2^(G_last) + K^T (v' 2^(G_last-G))."""
    rows, Hk, K = k.shape
    Hv, V = v.shape[1], v.shape[2]
    rep = Hv // Hk
    bf = lambda x: x.to(torch.bfloat16).float()
    if o is None:
        o = torch.zeros_like(v)
    cu = [int(x) for x in cu]
    for n in range(len(cu) - 1):
        S = torch.zeros((Hv, K, V), dtype=torch.float32)
        if h0 is not None and h0_idx is not None and int(h0_idx[n]) >= 0:
            S = h0[int(h0_idx[n])].float().clone()
        for c0 in range(cu[n], cu[n + 1], chunk):
            c1 = min(c0 + chunk, cu[n + 1])
            r = torch.as_tensor([int(idx[t]) if idx is not None else t for t in range(c0, c1)], dtype=torch.int64)
            C = len(r)
            Q = q[r].float().repeat_interleave(rep, 1).transpose(0, 1)  # [Hv, C, K]
            Kc = k[r].float().repeat_interleave(rep, 1).transpose(0, 1)
            Vc = v[r].float().transpose(0, 1)                           # [Hv, C, V]
            b = beta[r].float().transpose(0, 1)                         # [Hv, C]
            G = torch.cumsum(g[r].float(), 0).transpose(0, 1) * 1.4426950408889634
            dec = torch.exp2(G[:, :, None] - G[:, None, :])             # [Hv, t, s]
            lower = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
            A = torch.where(lower, (Kc @ Kc.transpose(1, 2)) * dec * b[:, :, None], torch.zeros(()))
            T = bf(torch.linalg.solve_triangular(torch.eye(C) + A, torch.eye(C).expand(Hv, C, C), upper=False))
            W = bf(T @ bf(Kc * b[:, :, None] * torch.exp2(G)[:, :, None]))
            U = bf(T @ bf(Vc * b[:, :, None]))
            Sb = bf(S)
            vn = U - W @ Sb
            P = torch.where(torch.tril(torch.ones(C, C, dtype=torch.bool)), (Q @ Kc.transpose(1, 2)) * dec, torch.zeros(()))
            out = ((Q @ Sb) * torch.exp2(G)[:, :, None] + bf(P) @ bf(vn)) * scale
            o[r] = out.transpose(0, 1).to(o.dtype)
            g_last = G[:, -1]
            S = S * torch.exp2(g_last)[:, None, None] + Kc.transpose(1, 2) @ bf(vn * torch.exp2(g_last[:, None] - G)[:, :, None])
        if ht is not None and ht_idx is not None and int(ht_idx[n]) >= 0:
            ht[int(ht_idx[n])] = S.to(ht.dtype)
    return o


def gdn_tree(q, k, v, g, beta, plan, dtype=torch.float32, form="recurrent"):
    """every segment from its parent's final state, level by level (gdn_indexed, qwen.py:550-590); plan: a TreePlan whose calls
    carry idx, cu_cpu, h0_idx, ht_idx (host or device tensors). form "chunked": every segment, short ones too, through chunked()
    (the rounding points of the kernels that run whole plans in the chunked form)"""
    scale = q.shape[-1] ** -0.5
    o = torch.zeros_like(v)
    prev_states = None
    for calls, nk in zip(plan.levels, plan.n_keep):
        states = torch.zeros((nk, v.shape[1], q.shape[-1], v.shape[-1]), dtype=torch.float32) if nk else None
        for c in calls:
            args = (
                q, k, v, g, beta, scale, np.asarray(c.cu_cpu), np.asarray(c.idx.cpu()),
                prev_states if c.h0_idx is not None else None, None if c.h0_idx is None else np.asarray(c.h0_idx.cpu()),
                states if c.ht_idx is not None else None, None if c.ht_idx is None else np.asarray(c.ht_idx.cpu()), o,
            )
            if form == "chunked":
                chunked(*args)
            else:
                recurrent(*args, dtype)
        prev_states = states
    return o


def prologue(y, conv, conv_w, A_log, dt_bias, Hk, Dk, Hv, Dv):
    """y [T, conv_dim + Hv Dv + 2 Hv] bf16 (the fused in-projection: q k v | z | b | a) -> q, k [T, Hk, Dk], v [T, Hv, Dv] bf16,
    z [T, Hv, Dv] bf16, g [T, Hv] fp32, beta [T, Hv] bf16: path convolution over 4 taps (conv [T, 4], index T = a zero row) + SiLU,
    beta = sigmoid(b), g = -exp(A_log) softplus(a + dt_bias), q and k l2-normalised per head (qwen.py:651-668)"""
    T = y.shape[0]
    kd, vd = Hk * Dk, Hv * Dv
    conv_dim = 2 * kd + vd
    qkv, z = y[:, :conv_dim], y[:, conv_dim : conv_dim + vd]
    b, a = y[:, conv_dim + vd : conv_dim + vd + Hv], y[:, conv_dim + vd + Hv :]
    ext = torch.cat([qkv, qkv.new_zeros(1, conv_dim)])
    c = (ext[torch.as_tensor(np.asarray(conv), dtype=torch.int64)].float() * conv_w.float()[None].transpose(1, 2)).sum(1)
    qkv = F.silu(c).to(y.dtype)
    q = qkv[:, :kd].reshape(T, Hk, Dk)
    k = qkv[:, kd : 2 * kd].reshape(T, Hk, Dk)
    v = qkv[:, 2 * kd :].reshape(T, Hv, Dv)
    beta = torch.sigmoid(b.float()).to(y.dtype)
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    q = (q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6)).to(y.dtype)
    k = (k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)).to(y.dtype)
    return q, k, v, z.reshape(T, Hv, Dv), g, beta


def epilogue(o, z, norm_w, eps):
    """o, z [T, Hv, Dv] bf16 -> [T, Hv Dv] bf16: per-head RMS normalisation, weight, SiLU(z) gate (qwen.py:670-673)"""
    of = o.float()
    of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    of = (norm_w * of.to(o.dtype)).float() * F.silu(z.float())
    return of.to(o.dtype).reshape(o.shape[0], -1)
