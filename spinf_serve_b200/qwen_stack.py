"""The Qwen-style hybrid stack of the packed scoring path (Gated DeltaNet layers with a full-attention layer every few layers, int4
weight-only linears): the counterpart of Qwen35Stack and QwenTextModel (spinf_serve/models/qwen35/qwen.py:1007-1165, :737-775), in
the stream layout, on library kernels only. Per layer (qwen.py:718-734):

    x -> RMSNorm(1 + w) -> mixer -> + x -> RMSNorm(1 + w) -> SwiGLU MLP -> + x
    Gated DeltaNet mixer (qwen.py:640-673): int4 in-projection (q k v z | b a) -> path conv + SiLU, l2 norms, beta, g (one kernel)
        -> gated delta rule over the plan's segments, branches forking their trunk's state -> gated RMS norm -> int4 out-projection
    attention mixer (qwen.py:683-697): int4 projection [H x (q | gate)] | k | v -> head norms + partial rotary -> tree attention
        -> sigmoid gate -> int4 out-projection
The plan of the recurrent layers (segments, levels, conv taps) is built on the host ahead of the GPU (gdn_plan.tree_plan)."""

from dataclasses import dataclass, field

import torch

from spinf_serve_b200 import attention, gdn, ops
from spinf_serve_b200.gdn_plan import tree_plan
from spinf_serve_b200.linears import Int4Linear


@dataclass
class QwenConfig:
    layers: int = 64
    hidden: int = 5120
    ffn: int = 17408
    vocab: int = 248320
    hk: int = 16
    hv: int = 32
    dk: int = 128
    dv: int = 128
    heads: int = 24
    kv_heads: int = 4
    head_dim: int = 256
    rotary: int = 64
    theta: float = 10_000_000.0
    eps: float = 1e-6
    group: int = 128
    every: int = 4  # every `every`-th layer is full attention, the rest Gated DeltaNet
    softcap: float | None = None
    layer_types: list = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["full_attention" if (i + 1) % self.every == 0 else "linear_attention" for i in range(self.layers)]


class QwenWeights:
    """device-resident weights from GPTQ-format tensors: W = {"embed", "lm_head", "norm", "layers": [{"kind", "input_ln", "post_ln",
    "gate_up", "down", and per kind "in_proj" / "in_extra" / "out_proj" / "conv_w" / "A_log" / "dt_bias" / "gdn_norm" or
    "qkv_proj" / "o_proj" / "q_norm" / "k_norm"}]}; int4 linears are (qweight int32 [K/8, N], scales fp16 [K/G, N]) pairs"""

    def __init__(self, cfg: QwenConfig, W, device):
        self.cfg = cfg
        dev = torch.device(device)
        self.embed = W["embed"].to(dev).contiguous()
        self.lm_head = W["lm_head"].to(dev).contiguous()
        self.norm = W["norm"].to(dev).contiguous()
        self.layers = []
        for L in W["layers"]:
            out = {"kind": L["kind"]}
            for k, v in L.items():
                if k == "kind":
                    continue
                if isinstance(v, tuple):
                    out[k] = Int4Linear(v[0].to(dev), v[1].to(dev))
                elif k in ("A_log", "dt_bias"):
                    out[k] = v.to(dev, torch.float32).contiguous()
                else:
                    out[k] = v.to(dev).contiguous()
            if "in_extra" in out:
                out["in_proj"].set_extra(out.pop("in_extra"))  # the b and a rows ride in the same output (qwen.py:421-426)
            self.layers.append(out)

    @property
    def lm_weight(self):
        return self.lm_head  # untied lm head (qwen.py:809-812)


class QwenStack:
    family = "qwen"
    hybrid = True

    def __init__(self, weights: QwenWeights, n_layers: int | None = None):
        self.w = weights
        self.cfg = weights.cfg
        self.n_layers = self.cfg.layers if n_layers is None else n_layers
        R = self.cfg.rotary
        self.inv_freq = (1.0 / (self.cfg.theta ** (torch.arange(0, R, 2, dtype=torch.float32) / R))).to(weights.embed.device)

    def plan(self, b) -> None:
        """the recurrent layers' plan, on the host ahead of the GPU (the producer thread; Qwen35Stack.plan, qwen.py:1056)"""
        b.gdn_plan_host = (b.prev, b.art >= 0)

    def stage(self, b, device):
        ids = torch.from_numpy(b.ids).pin_memory().to(device, non_blocking=True)
        masks = attention.stream_masks(b.art, b.end, b.pos, None, device, always_window=False)
        prev, real = getattr(b, "gdn_plan_host", (b.prev, b.art >= 0))
        return {"ids": ids, "pos": masks["full_attention"].pos, "masks": masks, "plan": tree_plan(prev, real, device)}

    def forward(self, inputs, rows=None, taps=None):
        cfg, w = self.cfg, self.w
        ids, pos, mask, plan = inputs["ids"], inputs["pos"], inputs["masks"]["full_attention"], inputs["plan"]
        n = ids.numel()
        H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
        cos, sin = ops.rope_table(pos, self.inv_freq)
        x = ops.embed_scale(ids, w.embed, 1.0)
        h = ops.fused_norm(x, w2=w.layers[0]["input_ln"], eps=cfg.eps, plus1=True, want_norm=True)["norm"] if self.n_layers else None
        for i in range(self.n_layers):
            L = w.layers[i]
            if L["kind"] == "linear_attention":
                y = L["in_proj"](h)
                q, k, v, z, g, beta = gdn.prologue(y, plan.conv, L["conv_w"], L["A_log"], L["dt_bias"], cfg.hk, cfg.dk, cfg.hv, cfg.dv)
                o = gdn.gdn_tree(q, k, v, g, beta, plan)
                m = L["out_proj"](gdn.epilogue(o, z, L["gdn_norm"], cfg.eps))
            else:
                y = L["qkv_proj"](h)
                q = ops.qkv_norm_rope_gated(y, H, K, D, L["q_norm"], L["k_norm"], cos, sin, cfg.eps, plus1=True)
                kk = y[:, 2 * H * D : (2 * H + K) * D].view(n, K, D)
                vv = y[:, (2 * H + K) * D :].view(n, K, D)
                o = attention.tree_attention(q, kk, vv, mask, D**-0.5)
                ops.attn_gate(o, y, H, D)
                m = L["o_proj"](o.view(n, H * D))
            r = ops.fused_norm(m, residual=x, w2=L["post_ln"], eps=cfg.eps, plus1=True, want_h=True, want_norm=True)
            x = r["h"]
            _, _, act = ops.glu_quant(L["gate_up"](r["norm"]), "silu", want_fp8=False, want_y=True)
            d = L["down"](act)
            last = i == self.n_layers - 1
            r = ops.fused_norm(d, residual=x, w2=None if last else w.layers[i + 1]["input_ln"], eps=cfg.eps, plus1=True, want_h=True,
                               want_norm=not last)
            x = r["h"]
            h = None if last else r["norm"]
            if taps is not None:
                taps[i] = x
        return ops.fused_norm(x, w2=w.norm, rows=rows, eps=cfg.eps, plus1=True, want_norm=True)["norm"]
