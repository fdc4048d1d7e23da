"""The Qwen-style hybrid stack of the packed scoring path (Gated DeltaNet layers with a full-attention layer every few layers, int4
weight-only linears): the counterpart of Qwen35Stack and QwenTextModel (spinf_serve/models/qwen35/qwen.py:1007-1165, :737-775), in
the stream layout, on library kernels only. Per layer (qwen.py:718-734):

    x -> RMSNorm(1 + w) -> mixer -> + x -> RMSNorm(1 + w) -> SwiGLU MLP -> + x
    Gated DeltaNet mixer (qwen.py:640-673): int4 in-projection (q k v z | b a) -> path conv + SiLU, l2 norms, beta, g (one kernel)
        -> gated delta rule over the plan's segments, branches forking their trunk's state -> gated RMS norm -> int4 out-projection
    attention mixer (qwen.py:683-697): int4 projection [H x (q | gate)] | k | v -> head norms + partial rotary -> tree attention
        -> sigmoid gate -> int4 out-projection
The plan of the recurrent layers (segments, levels, conv taps) is built on the host ahead of the GPU (gdn_plan.tree_plan)."""

from contextlib import contextmanager
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

    def __init__(self, cfg: QwenConfig, W, device, fuse_glu: bool = True):
        """fuse_glu: the MLP's SiLU(gate) * up inside the gate|up GEMM's epilogue (the same values as the separate pass)"""
        self.cfg = cfg
        self.fuse_glu = fuse_glu
        dev = torch.device(device)
        self.embed = W["embed"].to(dev).contiguous()
        self.lm_head = W["lm_head"].to(dev).contiguous()
        self.norm = W["norm"].to(dev).contiguous()
        self.layers = [self._layer(L, dev, fuse_glu) for L in W["layers"]]

    @staticmethod
    def _layer(L, dev, fuse_glu):
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
        if fuse_glu:
            out["gate_up"].fuse_glu("silu")
        return out

    @classmethod
    def random(cls, cfg: QwenConfig, seed: int, device, fuse_glu: bool = True):
        """random-init weights of the architecture, generated on the device one layer at a time (GPTQ-format int4 linears with
        uniform random nibbles and small positive scales, bf16 / fp32 small parameters): the benchmark's synthetic hybrid model"""
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)

        def bf(*shape, std=0.05):
            return (torch.randn(shape, generator=g, device=dev) * std).to(torch.bfloat16)

        def int4(out_f, in_f):
            qweight = torch.randint(-(2**31), 2**31 - 1, (in_f // 8, out_f), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
            scales = (torch.rand((in_f // cfg.group, out_f), generator=g, device=dev) * 0.01 + 0.001).to(torch.float16)
            return qweight, scales

        self = cls.__new__(cls)
        self.cfg, self.fuse_glu = cfg, fuse_glu
        self.embed, self.lm_head, self.norm = bf(cfg.vocab, cfg.hidden, std=0.5), bf(cfg.vocab, cfg.hidden), bf(cfg.hidden, std=0.1)
        kd, vd = cfg.hk * cfg.dk, cfg.hv * cfg.dv
        self.layers = []
        for kind in cfg.layer_types:
            L = {"kind": kind, "input_ln": bf(cfg.hidden, std=0.1), "post_ln": bf(cfg.hidden, std=0.1),
                 "gate_up": int4(2 * cfg.ffn, cfg.hidden), "down": int4(cfg.hidden, cfg.ffn)}
            if kind == "linear_attention":
                L["in_proj"] = int4(2 * kd + 2 * vd, cfg.hidden)
                L["in_extra"] = bf(2 * cfg.hv, cfg.hidden, std=0.02)
                L["out_proj"] = int4(cfg.hidden, vd)
                L["conv_w"] = bf(2 * kd + vd, 4, std=0.5)
                L["A_log"] = torch.randn(cfg.hv, generator=g, device=dev) * 0.5
                L["dt_bias"] = torch.randn(cfg.hv, generator=g, device=dev)
                L["gdn_norm"] = (1 + 0.1 * torch.randn(cfg.dv, generator=g, device=dev)).to(torch.bfloat16)
            else:
                L["qkv_proj"] = int4((2 * cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim, cfg.hidden)
                L["o_proj"] = int4(cfg.hidden, cfg.heads * cfg.head_dim)
                L["q_norm"], L["k_norm"] = bf(cfg.head_dim, std=0.1), bf(cfg.head_dim, std=0.1)
            self.layers.append(cls._layer(L, dev, fuse_glu))
            del L
        return self

    @property
    def lm_weight(self):
        return self.lm_head  # untied lm head (qwen.py:809-812)


class QwenStack:
    family = "qwen"
    hybrid = True
    bidirectional_images = False  # image tokens attend causally, as text (qwen.py:1014)

    def __init__(self, weights: QwenWeights, n_layers: int | None = None, compact: bool = True, min_stream: int = 0, align_jobs: bool = True):
        """compact (QwenOptions.compact, qwen.py:86, default on): the model runs on the stream's real tokens only, in stream order,
        padded with zero rows to whole blocks; the stream layout (pads between aligned jobs) exists only around the attention"""
        self.w = weights
        self.cfg = weights.cfg
        self.n_layers = self.cfg.layers if n_layers is None else n_layers
        self.compact, self.min_stream, self.align_jobs = compact, min_stream, align_jobs
        R = self.cfg.rotary
        self.inv_freq = (1.0 / (self.cfg.theta ** (torch.arange(0, R, 2, dtype=torch.float32) / R))).to(weights.embed.device)
        self._cap = None  # capture() sets the ranges and the dicts the forward fills

    def compact_rows(self, b) -> int | None:
        """the rows the model runs on: the real tokens in whole blocks, at least the GEMM floor for aligned jobs, never more than the
        stream (Qwen35Stack.compact_rows, qwen.py:1039-1048); None = the stream layout"""
        from spinf_serve_b200.packer import BLOCK

        if not self.compact:
            return None
        R = int((b.art >= 0).sum())
        floor = self.min_stream if self.align_jobs else 0
        return min(b.length, max((R + BLOCK - 1) // BLOCK * BLOCK, floor))

    window = None  # every attention layer of the family is full attention

    # ---- capture for the extraction decoder (Qwen35Stack.capture, spinf_serve/models/qwen35/qwen.py, and what qwen_decode.Decoder
    # reads of it, qwen_decode.py:70-166): per attention layer the K/V of every owner's prefix and of every template branch; per
    # recurrent layer the prefix's final state, the templates' q k v g beta rows and the pre-convolution rows of the last three
    # tokens on the path to each template's end (the decoder's conv ring)
    @contextmanager
    def capture(self, sc, b, xo: list):
        """around the forward of a batch whose owners `xo` have extraction branches -> {"kv": {key: {layer: (k, v)}}, "extra":
        {"state": {key: {layer: S [Hv, K, V] fp32}}, "tok": {key: {layer: (q, k, v, g, beta)}}, "pre": {key: {layer: [3, conv
        dim]}}}, "pos0": None}; keys ("p", id(owner)) for prefixes, ("t", prompt key) for templates"""
        import numpy as np

        if b.media:
            raise ValueError("media in a hybrid-family stream needs the (t, h, w) rotary positions of its images, which are outside this path")
        real = b.art >= 0
        to_row = (np.cumsum(real) - 1) if self.compact_rows(b) is not None else np.arange(b.length)
        pre = [(int(to_row[o.start]), o.prefix_len, ("p", id(o))) for o in xo]
        # (first row, length, key, row of the template's last token: the prefix's last token for a slot without template tokens)
        tmpl = [(int(to_row[bs]) if bl else 0, bl, ("t", pr.key), int(to_row[bs + bl - 1])) for o in xo for bs, bl, pr in o.xbranches]
        cap = {"prefixes": pre, "templates": tmpl, "kv": {}, "state": {}, "tok": {}, "pre": {}}
        self._cap = cap
        try:
            yield {"kv": cap["kv"], "extra": {"state": cap["state"], "tok": cap["tok"], "pre": cap["pre"]}, "pos0": None}
        finally:
            self._cap = None

    def abandon(self, sc) -> None:
        self._cap = None

    def kv_bytes_per_token(self) -> dict:
        return {i: 2 * self.cfg.kv_heads * self.cfg.head_dim * 2 for i in range(self.n_layers) if self.w.layers[i]["kind"] != "linear_attention"}

    def _capture_recurrent(self, i, y, q, k, v, g, beta, plan):
        cap, cfg = self._cap, self.cfg
        cd = 2 * cfg.hk * cfg.dk + cfg.hv * cfg.dv
        dev = y.device
        if cap["prefixes"]:
            # the prefixes' final states: the chunked recurrence once more over the prefix rows alone (only batches with
            # extraction branches pay for it)
            lens = [n for _, n, _ in cap["prefixes"]]
            cu_cpu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
            idx = torch.cat([torch.arange(r0, r0 + n, dtype=torch.int64) for r0, n, _ in cap["prefixes"]]).to(dev)
            ht = torch.empty((len(lens), cfg.hv, cfg.dk, cfg.dv), dtype=torch.float32, device=dev)
            scratch = torch.empty((1, q.shape[0], cfg.hv, cfg.dv), dtype=torch.bfloat16, device=dev)
            gdn.chunked(q, k, v, g, beta, cfg.dk**-0.5, cu_cpu.to(dev), cu_cpu, ht=ht, ht_idx=torch.arange(len(lens), dtype=torch.int64, device=dev),
                        idx=idx, o=scratch)
            for j, (_, _, key) in enumerate(cap["prefixes"]):
                cap["state"].setdefault(key, {})[i] = ht[j]
        n_rows = y.shape[0]
        for r0, n, key, r_end in cap["templates"]:
            sl = slice(r0, r0 + n)
            cap["tok"].setdefault(key, {})[i] = (q[sl].clone(), k[sl].clone(), v[sl].clone(), g[sl].clone(), beta[sl].clone())
            taps = plan.conv[r_end, 1:4]  # the path's last three tokens, the template's end among them
            ok = (taps >= 0) & (taps < n_rows)
            cap["pre"].setdefault(key, {})[i] = y[taps.clamp(0, n_rows - 1), :cd] * ok[:, None].to(y.dtype)

    def plan(self, sc, b) -> None:
        """the host half of the recurrent layers' plan, ahead of the GPU (the packing thread; Qwen35Stack.plan, qwen.py:1056): the
        compact-row count and, for compact rows, the real tokens' ids / positions and the stream-position -> row map, which ride
        in the batch's staging block (b.staged)"""
        import numpy as np

        real = b.art >= 0
        rows = self.compact_rows(b)
        b.gdn_plan_host = (b.prev, real, rows)
        if rows is not None:
            R = int(real.sum())
            ids = np.zeros(rows, np.int64)
            ids[:R] = b.ids[real]
            pos = np.zeros(rows, np.int32)
            pos[:R] = b.pos[real]
            b.staged = {"compact.ids": ids, "compact.pos": pos, "compact.to_row": (np.cumsum(real) - 1).astype(np.int64)}

    def stage(self, sc, b, st: dict) -> dict:
        """what forward reads (Qwen35Stack.stage, qwen.py:1064): the staged ids / positions (compact rows: the real tokens', then
        zeros, qwen.py:1064-1090) and the recurrent layers' TreePlan, whose index arrays go up here"""
        if not hasattr(b, "gdn_plan_host"):
            self.plan(sc, b)
        prev, real, rows = b.gdn_plan_host
        plan = tree_plan(prev, real, sc.device, rows=rows)
        if rows is None:
            return {"ids": st["ids"][None], "pos": st["pos32"][None], "plan": plan, "n": b.length}
        if "compact.ids" not in st:
            raise RuntimeError("compact rows: the batch was staged without its plan (call stack.plan(sc, b) before staging)")
        return {"ids": st["compact.ids"][None], "pos": st["compact.pos"][None], "plan": plan, "n": b.length, "to_row": st["compact.to_row"]}

    def forward(self, sc, b, inputs: dict, masks: dict, rows=None, taps=None, attend=None, recur=None):
        """packed forward (Stack.forward, base.py:62-64) -> final hidden states after the last norm, [1, stream length, hidden] bf16
        in the stream layout. Beyond the reference's signature: rows (stream positions) returns only those rows, [len(rows),
        hidden]; taps: optional dict filled with the residual stream per layer, in the stream layout (tests); attend(layer, q, k, v)
        -> [n, H, D] and recur(layer, y) -> (o, z) stand in for the tree attention and the recurrence over the plan in a decoding
        step (decode.HybridDecoder): masks and inputs["plan"] are unused then"""
        cfg, w = self.cfg, self.w
        ids, pos, plan = inputs["ids"].reshape(-1), inputs["pos"].reshape(-1), inputs.get("plan")
        mask = masks["full_attention"] if masks is not None else None
        n = ids.numel()          # rows the layers run on
        T = inputs.get("n", n)   # stream length (the attention's layout)
        sidx = plan.sidx if plan is not None and plan.rows is not None else None
        R = sidx.numel() if sidx is not None else n
        H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
        cos, sin = ops.rope_table(pos, self.inv_freq)
        x = ops.embed_scale(ids, w.embed, 1.0)
        if sidx is not None and n > R:
            x[R:].zero_()  # rows past the real tokens are zero rows
        h = ops.fused_norm(x, w2=w.layers[0]["input_ln"], eps=cfg.eps, plus1=True, want_norm=True)["norm"] if self.n_layers else None

        def to_stream(t):  # compact rows -> the stream layout (pads zero)
            if sidx is None:
                return t
            return torch.zeros((T,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device).index_copy_(0, sidx, t[:R])

        few = recur is not None or attend is not None  # a decoding step: the linears' few-row form

        def lin(mod, t):
            return mod.few(t) if few and t.shape[0] <= 256 else mod(t)

        for i in range(self.n_layers):
            L = w.layers[i]
            if L["kind"] == "linear_attention":
                y = lin(L["in_proj"], h)
                if recur is not None:
                    o, z = recur(i, y)
                else:
                    q, k, v, z, g, beta = gdn.prologue(y, plan.conv, L["conv_w"], L["A_log"], L["dt_bias"], cfg.hk, cfg.dk, cfg.hv, cfg.dv)
                    o = gdn.gdn_tree(q, k, v, g, beta, plan)
                    if self._cap is not None:
                        self._capture_recurrent(i, y, q, k, v, g, beta, plan)
                m = lin(L["out_proj"], gdn.epilogue(o, z, L["gdn_norm"], cfg.eps))
            else:
                y = lin(L["qkv_proj"], h)
                q = ops.qkv_norm_rope_gated(y, H, K, D, L["q_norm"], L["k_norm"], cos, sin, cfg.eps, plus1=True)
                kk = y[:, 2 * H * D : (2 * H + K) * D].view(n, K, D)
                vv = y[:, (2 * H + K) * D :].view(n, K, D)
                if self._cap is not None:
                    for r0, cnt, key in self._cap["prefixes"] + [t[:3] for t in self._cap["templates"]]:
                        self._cap["kv"].setdefault(key, {})[i] = (kk[r0 : r0 + cnt].clone(), vv[r0 : r0 + cnt].clone())
                if attend is not None:
                    o = attend(i, q, kk, vv)
                elif sidx is None:
                    o = attention.tree_attention(q, kk, vv, mask, D**-0.5)
                else:  # the real rows scattered into the stream layout for the attention, its output gathered back (qwen.py:605-623)
                    o_s = attention.tree_attention(to_stream(q), to_stream(kk), to_stream(vv), mask, D**-0.5)
                    o = torch.zeros((n, H, D), dtype=o_s.dtype, device=o_s.device)
                    o[:R] = o_s.index_select(0, sidx)
                ops.attn_gate(o, y, H, D)
                m = lin(L["o_proj"], o.view(n, H * D))
            r = ops.fused_norm(m, residual=x, w2=L["post_ln"], eps=cfg.eps, plus1=True, want_h=True, want_norm=True)
            x = r["h"]
            if w.fuse_glu:
                act = lin(L["gate_up"], r["norm"])
            else:
                _, _, act = ops.glu_quant(L["gate_up"](r["norm"]), "silu", want_fp8=False, want_y=True)
            d = lin(L["down"], act)
            last = i == self.n_layers - 1
            r = ops.fused_norm(d, residual=x, w2=None if last else w.layers[i + 1]["input_ln"], eps=cfg.eps, plus1=True, want_h=True,
                               want_norm=not last)
            x = r["h"]
            h = None if last else r["norm"]
            if taps is not None:
                taps[i] = to_stream(x)
        if rows is not None and sidx is not None:
            rows = inputs["to_row"].index_select(0, rows)  # the read rows are stream positions
        out = ops.fused_norm(x, w2=w.norm, rows=rows, eps=cfg.eps, plus1=True, want_norm=True)["norm"]
        if rows is not None:
            return out
        return (out if sidx is None else to_stream(out))[None]
