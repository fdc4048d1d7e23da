"""Oracle of the Qwen-style hybrid packed forward (CPU torch; test infrastructure only, never imported by the product): a
restatement of the reference's own model code, spinf_serve/models/qwen35/qwen.py: RMSNorm with (1 + w) (:502-510), Layer (:718-734),
GatedDeltaNet.forward (:640-673), Attention.forward (:683-697) with partial rotary embedding rope() (:699-704), MLP (:706-716),
QwenTextModel.forward (:764-775), with Int4Linear in bf16 mode (oracle.linears.int4_linear). Stream layout (no compact rows).
The reference builds this model inside a closure that needs a checkpoint directory, so it cannot be imported for a bit-for-bit
pin: this restatement is checked against the reference by reading only (parity unpinned by execution)."""

from dataclasses import dataclass, field

import numpy as np
import torch
import torch.nn.functional as F

from oracle import attention as OA
from oracle import gdn as OGD
from oracle import linears as OL


@dataclass
class QwenConfig:
    layers: int = 64
    hidden: int = 5120
    ffn: int = 17408
    vocab: int = 248320
    hk: int = 16       # Gated DeltaNet key heads
    hv: int = 32       # Gated DeltaNet value heads
    dk: int = 128
    dv: int = 128
    heads: int = 24    # full-attention layers
    kv_heads: int = 4
    head_dim: int = 256
    rotary: int = 64   # rotary dimensions (head_dim * partial_rotary_factor)
    theta: float = 10_000_000.0
    eps: float = 1e-6
    group: int = 128   # int4 group size
    every: int = 4     # every `every`-th layer is full attention, the rest Gated DeltaNet
    layer_types: list = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["full_attention" if (i + 1) % self.every == 0 else "linear_attention" for i in range(self.layers)]


def _int4(g, out_f, in_f, group):
    nib = torch.randint(0, 16, (in_f, out_f), generator=g, dtype=torch.int32)
    qweight = torch.zeros((in_f // 8, out_f), dtype=torch.int32)
    for i in range(8):
        qweight |= nib[i::8] << (4 * i)
    scales = (torch.rand((in_f // group, out_f), generator=g) * 0.01 + 0.001).to(torch.float16)
    return qweight, scales


def init_weights(cfg: QwenConfig, seed=0):
    """random GPTQ-format int4 linears (qweight int32 [K/8, N], scales fp16 [K/G, N]) and bf16 / fp32 small parameters"""
    g = torch.Generator().manual_seed(seed)
    bf = lambda *s, std=0.05: (torch.randn(s, generator=g) * std).to(torch.bfloat16)  # noqa: E731
    kd, vd = cfg.hk * cfg.dk, cfg.hv * cfg.dv
    W = {"embed": bf(cfg.vocab, cfg.hidden, std=0.5), "lm_head": bf(cfg.vocab, cfg.hidden, std=0.05), "norm": bf(cfg.hidden, std=0.1), "layers": []}
    for kind in cfg.layer_types:
        L = {"kind": kind, "input_ln": bf(cfg.hidden, std=0.1), "post_ln": bf(cfg.hidden, std=0.1),
             "gate_up": _int4(g, 2 * cfg.ffn, cfg.hidden, cfg.group), "down": _int4(g, cfg.hidden, cfg.ffn, cfg.group)}
        if kind == "linear_attention":
            L["in_proj"] = _int4(g, 2 * kd + 2 * vd, cfg.hidden, cfg.group)
            L["in_extra"] = bf(2 * cfg.hv, cfg.hidden, std=0.02)  # the b and a projections, un-quantised
            L["out_proj"] = _int4(g, cfg.hidden, vd, cfg.group)
            L["conv_w"] = bf(2 * kd + vd, 4, std=0.5)
            L["A_log"] = torch.randn(cfg.hv, generator=g) * 0.5
            L["dt_bias"] = torch.randn(cfg.hv, generator=g)
            L["gdn_norm"] = (1 + 0.1 * torch.randn(cfg.dv, generator=g)).to(torch.bfloat16)
        else:
            L["qkv_proj"] = _int4(g, (2 * cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim, cfg.hidden, cfg.group)
            L["o_proj"] = _int4(g, cfg.hidden, cfg.heads * cfg.head_dim, cfg.group)
            L["q_norm"] = bf(cfg.head_dim, std=0.1)
            L["k_norm"] = bf(cfg.head_dim, std=0.1)
        W["layers"].append(L)
    return W


def rmsnorm(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).type_as(x)


def rope(x, cos, sin):
    R = cos.shape[-1]
    xr, xp = x[..., :R], x[..., R:]
    x1, x2 = xr[..., : R // 2], xr[..., R // 2 :]
    rot = torch.cat([-x2, x1], -1)
    return torch.cat([xr * cos[:, None] + rot * sin[:, None], xp], -1)


def forward(cfg: QwenConfig, W, ids, art, end, pos, plan, n_layers=None, taps=None, caps=None, attend=None, recur=None):
    """packed forward -> final hidden states [T, hidden] bf16; plan: a TreePlan over the stream (gdn_plan.tree_plan on the CPU).
    caps: optional dict filled per layer with what an extraction capture keeps (recurrent layers: the in-projection rows y and
    q, k, v, g, beta; attention layers: k, v). attend(layer, q, k, v) -> [T, H, D] and recur(layer, y) -> (o, z) stand in for the
    tree attention and the recurrence over the plan in a decoding step (spinf_serve/models/qwen35/qwen_decode.py); art, end and
    plan are unused then."""
    T = len(ids)
    lin = lambda x, w, extra=None: OL.int4_linear(x, *OL.gptq_unpack(*w), cfg.group, extra)  # noqa: E731
    x = W["embed"][torch.as_tensor(np.asarray(ids), dtype=torch.int64)]
    inv_freq = 1.0 / (cfg.theta ** (torch.arange(0, cfg.rotary, 2, dtype=torch.float32) / cfg.rotary))
    f = torch.as_tensor(np.asarray(pos), dtype=torch.float32)[:, None] * inv_freq[None]
    e = torch.cat([f, f], -1)
    cos, sin = e.cos().to(x.dtype), e.sin().to(x.dtype)
    conv = None if plan is None else plan.conv.numpy() if hasattr(plan.conv, "numpy") else np.asarray(plan.conv)
    H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    for i, L in enumerate(W["layers"][: n_layers if n_layers is not None else cfg.layers]):
        h = rmsnorm(x, L["input_ln"], cfg.eps)
        if L["kind"] == "linear_attention":
            y = lin(h, L["in_proj"], L["in_extra"])
            if recur is not None:
                o, z = recur(i, y)
            else:
                q, k, v, z, g, beta = OGD.prologue(y, conv, L["conv_w"], L["A_log"], L["dt_bias"], cfg.hk, cfg.dk, cfg.hv, cfg.dv)
                o = OGD.gdn_tree(q, k, v, g, beta, plan)
                if caps is not None:
                    caps[i] = {"y": y, "q": q, "k": k, "v": v, "g": g, "beta": beta, "o": o}
            h = lin(OGD.epilogue(o, z, L["gdn_norm"], cfg.eps), L["out_proj"])
        else:
            y = lin(h, L["qkv_proj"])
            nq, nk = H * 2 * D, K * D
            qg = y[:, :nq].reshape(T, H, 2 * D)
            q, gate = qg[..., :D], qg[..., D:].reshape(T, -1)
            q = rmsnorm(q, L["q_norm"], cfg.eps)
            k = rmsnorm(y[:, nq : nq + nk].reshape(T, K, D), L["k_norm"], cfg.eps)
            v = y[:, nq + nk :].reshape(T, K, D)
            q, k = rope(q, cos, sin), rope(k, cos, sin)
            if caps is not None:
                caps[i] = {"k": k, "v": v}
            o = attend(i, q, k, v) if attend is not None else OA.tree_attention(q, k, v, art, end, pos, D**-0.5, None).to(x.dtype)
            h = lin(o.reshape(T, -1) * torch.sigmoid(gate), L["o_proj"])
        x = x + h
        gu = lin(rmsnorm(x, L["post_ln"], cfg.eps), L["gate_up"])
        n = gu.shape[-1] // 2
        x = x + lin(F.silu(gu[:, :n]) * gu[:, n:], L["down"])
        if taps is not None:
            taps[i] = x.clone()
    return rmsnorm(x, W["norm"], cfg.eps)
