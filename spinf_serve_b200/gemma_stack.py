"""The Gemma-style stack of the packed scoring path: the counterpart of Gemma4Stack (spinf_serve/models/gemma4.py:390-435), whose
forward (gemma4.py:407-415) runs transformers' Gemma 4 decoder layers with fp8 row-wise linears and the tree attention. Here a
layer is a fixed chain of library kernels over the packed stream [n, hidden]:

    fused_norm (post-ffn norm of the previous layer + residual + input norm + fp8 quantisation)
    fp8 GEMM q|k|v (one fused projection, head norms + rotary in its epilogue)  ->  tree attention (+ the row maxima of its output)
    ->  one-pass fp8 quantisation  ->  fp8 GEMM o  ->  fused_norm (post-attention norm + residual + pre-ffn norm + fp8 quantisation)
    fp8 GEMM gate|up with GeGLU in its epilogue (+ row maxima)  ->  one-pass fp8 quantisation  ->  fp8 GEMM down

Fusing q|k|v and gate|up is exact for this scheme: weight scales are per output channel and the activation scale is per token,
so each output element is the one the separate linears give. The final norm runs on the read rows only (Scorer._forward reads
nothing else, spinf_serve/scorer.py:248-254)."""

from contextlib import contextmanager
from dataclasses import dataclass, field

import torch

from spinf_serve_b200 import attention, ops
from spinf_serve_b200.linears import MONITOR, quantize_weight, quantize_weight_rowwise, static_scale

LINEARS = ("q", "k", "v", "o", "gate", "up", "down")  # the quantized linears of a layer
# the reference's EngineConfig.quant values for this family (spinf_serve/config.py:6, models/gemma4.py:170-235)
SCHEMES = ("fp8row", "fp8", "fp8s", "w8a8", "w8a16", "bf16")


@dataclass
class GemmaConfig:
    layers: int = 48
    hidden: int = 3840
    heads: int = 16
    kv_heads: int = 8
    head_dim: int = 256
    ffn: int = 15360
    vocab: int = 262144
    window: int = 1024
    pattern: int = 6  # every pattern-th layer is full attention, the rest sliding; the last layer is always full
    eps: float = 1e-6
    theta_sliding: float = 10_000.0
    theta_full: float = 1_000_000.0
    softcap: float | None = None
    layer_types: list = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["sliding_attention" if (i + 1) % self.pattern else "full_attention" for i in range(self.layers)]
            if self.layer_types:
                self.layer_types[-1] = "full_attention"

    @property
    def linear_params(self) -> int:
        """parameters of the quantized linears of one layer"""
        qkv = (self.heads + 2 * self.kv_heads) * self.head_dim
        return self.hidden * (qkv + self.heads * self.head_dim) + 3 * self.hidden * self.ffn


CONFIGS = {
    # benchmark configuration 2 / 3: synthetic Gemma-style 12B
    "gemma12b": dict(layers=48, hidden=3840, heads=16, kv_heads=8, head_dim=256, ffn=15360, vocab=262144, window=1024),
    # benchmark configuration 4: synthetic Gemma-style 31B-class
    "gemma31b": dict(layers=60, hidden=5376, heads=32, kv_heads=16, head_dim=128, ffn=21504, vocab=262144, window=1024),
}


class GemmaWeights:
    """device-resident weights: per layer the fused fp8 projections with their per-channel scales and the bf16 norm weights"""

    def __init__(self, cfg: GemmaConfig, embed, norm, layers, scheme="fp8row"):
        if scheme not in SCHEMES:
            raise RuntimeError(f"quant scheme {scheme} is outside the packed scoring path of this build (one of {SCHEMES})")
        self.cfg, self.embed, self.norm, self.layers, self.scheme = cfg, embed, norm, layers, scheme

    @staticmethod
    def _layer(L, pre=None, scheme="fp8row", xs=None):
        """one layer's device tensors. fp8row: per-channel weight scales, gate|up in the tiled order of the fused GeGLU GEMM.
        fp8 / fp8s (per-tensor weight scales): the same fused [out, in] storage with each linear's scalar spread over its output
        channels, gate|up in natural order; fp8s adds the calibrated activation scale and the clipping monitor of every linear
        input (`xs`: {linear name: scale}). w8a8: int8 weights with per-channel scales; w8a16 / bf16: bf16 weights (int8 values with
        the scale folded in, or the originals) and no scales."""

        def quant_int8(w):  # Int8Linear.__init__ (spinf_serve/quant/linears.py:43-46), the same eager ops
            wf = w.float()
            sc = wf.abs().amax(-1).clamp(min=1e-12) / 127.0
            return (wf / sc[:, None]).round_().clamp_(-127, 127).to(torch.int8), sc

        def fold(w):  # w8a16: the scale folded into the weight in bf16, as Int8Linear.forward folds it on every call (:63)
            w8, sc = quant_int8(w)
            return w8.to(torch.bfloat16) * sc.to(torch.bfloat16)[:, None], None

        quant = {"fp8row": quantize_weight_rowwise, "fp8": quantize_weight, "fp8s": quantize_weight, "w8a8": quant_int8,
                 "w8a16": fold, "bf16": lambda w: (w, None)}[scheme]

        def q8(*names):
            parts = [pre[k] if pre is not None else quant(L[k]) for k in names]
            if scheme == "w8a16" and pre is not None:  # int8 tensors given: fold as above
                parts = [(p[0].to(torch.bfloat16) * p[1].to(torch.bfloat16).reshape(-1)[:, None], None) for p in parts]
            if parts[0][1] is None:  # bf16 weights, no scales
                return torch.cat([p[0] for p in parts]).contiguous(), None
            w = torch.cat([p[0] for p in parts]).contiguous()
            sc = torch.cat([p[1].float().reshape(-1).expand(p[0].shape[0]) if p[1].numel() == 1 else p[1].reshape(-1) for p in parts])
            return w, sc.contiguous()

        out = {}
        out["qkv_w"], out["qkv_s"] = q8("q", "k", "v")
        out["o_w"], out["o_s"] = q8("o")
        gu_w, gu_s = q8("gate", "up")
        if scheme == "fp8row":
            order = ops.glu_tile_order(gu_w.shape[0] // 2).to(gu_w.device)  # the fused GEMM + GeGLU epilogue reads this row order
            gu_w, gu_s = gu_w.view(torch.uint8)[order].view(torch.float8_e4m3fn).contiguous(), gu_s[order].contiguous()
        out["gu_w"], out["gu_s"] = gu_w, gu_s
        out["down_w"], out["down_s"] = q8("down")
        for k in ("q_norm", "k_norm", "input_ln", "post_attn_ln", "pre_ffn_ln", "post_ffn_ln"):
            out[k] = L[k].contiguous()
        if scheme == "fp8s":
            dev = gu_w.device
            out["xs"] = {k: torch.tensor(float(xs[k]), dtype=torch.float32, device=dev) for k in LINEARS}
            out["peak"] = {k: torch.zeros((), dtype=torch.float32, device=dev) for k in LINEARS}
        return out

    @classmethod
    def from_bf16(cls, cfg: GemmaConfig, W, device, scheme="fp8row", scales=None):
        """W: {"embed", "norm", "layers": [{q,k,v,o,gate,up,down, q_norm,k_norm, input_ln,post_attn_ln,pre_ffn_ln,post_ffn_ln}]} of
        bf16 tensors (any device); quantisation runs on `device`, one layer at a time. scheme fp8s: scales[i][name] = the
        calibrated activation scale of layer i's linear `name` (the table calibrate() returns)"""
        layers = [
            cls._layer({k: v.to(device) for k, v in L.items()}, None, scheme, scales[i] if scales is not None else None)
            for i, L in enumerate(W["layers"])
        ]
        return cls(cfg, W["embed"].to(device).contiguous(), W["norm"].to(device).contiguous(), layers, scheme)

    @classmethod
    def from_quantized(cls, cfg: GemmaConfig, W, Q, device, scheme="fp8row", scales=None):
        """as from_bf16 with the linears already quantized: Q[i][name] = (w8 [out, in] e4m3, ws fp32: [1, out] row-wise, one
        element per-tensor), the tensors an fp8 checkpoint would hold (the reference's `prequantized` path,
        spinf_serve/quant/linears.py:121-131); scales as in from_bf16 (an fp8-static checkpoint's input_scale tensors)"""
        names = ("q_norm", "k_norm", "input_ln", "post_attn_ln", "pre_ffn_ln", "post_ffn_ln")
        layers = [
            cls._layer({k: L[k].to(device) for k in names}, {k: (a.to(device), None if b is None else b.to(device)) for k, (a, b) in q.items()}, scheme,
                       scales[i] if scales is not None else None)
            for i, (L, q) in enumerate(zip(W["layers"], Q))
        ]
        return cls(cfg, W["embed"].to(device).contiguous(), W["norm"].to(device).contiguous(), layers, scheme)

    @classmethod
    def random(cls, cfg: GemmaConfig, seed: int, device):
        """random-init weights of the architecture generated on the device (N(0, 0.02) linears and embedding, norm weights near 1)"""
        g = torch.Generator(device=device).manual_seed(seed)

        def lin(o, i):
            return (torch.randn((o, i), generator=g, device=device) * 0.02).to(torch.bfloat16)

        def nw(d):
            return (1.0 + 0.1 * torch.randn(d, generator=g, device=device)).to(torch.bfloat16)

        H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
        embed, norm = lin(cfg.vocab, cfg.hidden), nw(cfg.hidden)
        layers = []
        for _ in range(cfg.layers):
            L = {
                "q": lin(H * D, cfg.hidden), "k": lin(K * D, cfg.hidden), "v": lin(K * D, cfg.hidden), "o": lin(cfg.hidden, H * D),
                "gate": lin(cfg.ffn, cfg.hidden), "up": lin(cfg.ffn, cfg.hidden), "down": lin(cfg.hidden, cfg.ffn),
                "q_norm": nw(D), "k_norm": nw(D),
                "input_ln": nw(cfg.hidden), "post_attn_ln": nw(cfg.hidden), "pre_ffn_ln": nw(cfg.hidden), "post_ffn_ln": nw(cfg.hidden),
            }
            layers.append(cls._layer(L))
        return cls(cfg, embed, norm, layers)

    @property
    def lm_weight(self):
        return self.embed  # tied lm head (spinf_serve/models/gemma4.py:249)


class GemmaStack:
    """plan / stage / forward of the family (the Stack interface, spinf_serve/models/base.py:50-64), on library kernels only"""

    family = "gemma"
    hybrid = False
    bidirectional_images = True  # an image's placeholder tokens attend to each other both ways (Stack.bidirectional_images, base.py:28)

    def __init__(self, weights: GemmaWeights, n_layers: int | None = None, vision_bidir_all: bool = True):
        """vision_bidir_all (the reference's model._vision_bidir_all, gemma4.py:259): images' two-way blocks on every layer and
        past the window (the "unified" checkpoints); False: on the sliding layers only, within the window (global layers causal)"""
        self.vision_bidir_all = vision_bidir_all
        self.w = weights
        self.cfg = weights.cfg
        self.n_layers = self.cfg.layers if n_layers is None else n_layers  # the reference's EngineConfig.layers debug knob
        dev = weights.embed.device
        D = self.cfg.head_dim
        expo = torch.arange(0, D, 2, dtype=torch.int64).float() / D
        self.inv_freq = {
            "sliding_attention": (1.0 / (self.cfg.theta_sliding**expo)).to(dev),
            "full_attention": (1.0 / (self.cfg.theta_full**expo)).to(dev),
        }
        self.embed_scale = float(torch.tensor(self.cfg.hidden**0.5).to(torch.bfloat16))
        self.fuse_qkv = D in (128, 256) and ((self.cfg.heads + 2 * self.cfg.kv_heads) * D) % 256 == 0
        self.amax_log = None  # calibrate() sets a list here: (linear name, device scalar) per quantised input of a forward
        self._cap = None  # capture_ranges() sets {"window", "ranges", "kv"} here for the forwards inside it

    @property
    def window(self):
        """the sliding layers' window (the text config's sliding_window, read by the scorer when it builds the tile lists)"""
        return self.cfg.window

    def plan(self, sc, b) -> None:
        """nothing to prepare on the host for attention-only models (Stack.plan, base.py:50-51)"""

    # ---- K/V capture for the extraction decoder (Gemma4Stack.capture_ranges / capture, spinf_serve/models/gemma4.py:417-435, and
    # the hook inside the attention, :100-106)
    @contextmanager
    def capture_ranges(self, sc, ranges: list):
        """the K/V of the stream ranges [(start, n, key)] kept by the forwards inside -> the dict they fill under "kv":
        {key: {layer: (k [n', kv heads, D], v [n', kv heads, D])}}, token-major copies of the rows start .. start + n - 1 after
        head norm and rotary embedding; sliding layers keep the last window - 1 tokens of a range only"""
        cap = {"window": self.cfg.window, "ranges": list(ranges), "kv": {}}
        self._cap = cap
        try:
            yield cap
        finally:
            self._cap = None

    @contextmanager
    def capture(self, sc, b, xo: list):
        """around the forward of a batch whose owners `xo` have extraction branches (Stack.capture, base.py:66-70): every owner's
        prefix under ("p", id(owner)) and every template branch under ("t", prompt key)"""
        rs = [(o.start, o.prefix_len, ("p", id(o))) for o in xo] + [(bs, bl, ("t", pr.key)) for o in xo for bs, bl, pr in o.xbranches]
        with self.capture_ranges(sc, rs) as cap:
            yield {"kv": cap["kv"], "extra": None, "pos0": None}

    def abandon(self, sc) -> None:
        """drop a capture left open by a failed call (Stack.abandon)"""
        self._cap = None

    def kv_bytes_per_token(self) -> dict:
        """{layer: bytes of K and V one stored token takes} (what decode.group_bytes / chunk_bytes count with)"""
        return {i: 2 * self.cfg.kv_heads * self.cfg.head_dim * 2 for i in range(self.n_layers)}

    def stage(self, sc, b, st: dict) -> dict:
        """what forward reads of the staged arrays (Stack.stage, base.py:53-60, returns {"ids": [1, n], "pos": [1, n]}). `st` maps
        array names to device tensors: the scorer has laid the batch's arrays out in one pinned block and queued its single
        upload, so there is nothing left to copy here."""
        out = {"ids": st["ids"][None], "pos": st["pos32"][None]}
        if b.media:
            out["media"] = list(b.media)
        return out

    # ---- per-tensor schemes (fp8: the activation scale from the forward's own maximum; fp8s: a calibrated fixed scale). The
    # GEMMs are the row-wise kernels with every row given the tensor's one scale, so their fused epilogues stay; the reference
    # computes bf16(acc * xs * ws) with scalar scales (spinf_serve/quant/linears.py:77,114), the same product.
    def _linear(self, x, L, key, names):
        """x [n, K] bf16 through the fused linear `key` (the linears `names` of the layer) under the stack's scheme -> bf16 [n, N]"""
        sch = self.w.scheme
        if sch in ("bf16", "w8a16"):
            return ops.bf16_gemm(x, L[key + "_w"])
        if sch == "w8a8":
            x8, xs = ops.int8_rowwise_quant(x)
            return ops.int8_rowwise_gemm(x8, xs, L[key + "_w"], L[key + "_s"])
        x8, xs = self._quant_in(x, L, names)
        return ops.fp8_rowwise_gemm(x8, xs, L[key + "_w"], L[key + "_s"])

    def _quant_in(self, x, L, names):
        """x [n, K] bf16, the input of the linears `names` -> (x8, xs [n]). fp8s: the linears that share an input share its
        quantisation when their calibrated scales agree (they do when calibrate() made the table: one input, one maximum)."""
        n = x.shape[0]
        if self.w.scheme == "fp8":
            x8, s, amax = ops.fp8_tensor_quant(x, want_amax=True)
            if self.amax_log is not None:  # calibration: the largest input of each linear (quant/calibrate.py:117-124)
                for k in names:
                    self.amax_log.append((k, amax))
        else:
            vals = {float(L["xs"][k]) for k in names} if len(names) > 1 and not L.get("xs_checked") else ()
            if len(vals) > 1:
                raise RuntimeError(f"fp8s: the linears {names} read one input but carry different activation scales {sorted(vals)}")
            L["xs_checked"] = True
            x8, s = ops.fp8_tensor_quant(x, L["xs"][names[0]], L["peak"][names[0]] if MONITOR["on"] else None)
        return x8, s.reshape(1).expand(n).contiguous()

    def peaks(self):
        """fp8s: {(layer, linear name): largest |input| / (448 x scale) seen while linears.MONITOR["on"]} (above 1: clipped)"""
        out = {}
        for i, L in enumerate(self.w.layers[: self.n_layers]):
            for group in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
                for k in group:
                    out[(i, k)] = float(L["peak"][group[0]])
        return out

    def forward(self, sc, b, inputs: dict, masks: dict, rows=None, taps=None, attend=None):
        """packed forward (Stack.forward, base.py:62-64) -> final hidden states after the model's last norm, [1, n, hidden] bf16 in
        the stream layout. masks = {"full_attention": TileMask, "sliding_attention": TileMask} (attention.device_masks). Beyond the
        reference's signature: rows (int64 device tensor of stream positions) returns only those rows, [len(rows), hidden], the
        last norm running on them alone; taps: optional dict filled with per-layer intermediates (tests); attend(layer, kind, q, k,
        v) -> [n, H, D] replaces the tree attention (the extraction decoder's steps: masks is unused then)."""
        cfg, w = self.cfg, self.w
        H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
        ids, pos = inputs["ids"].reshape(-1), inputs["pos"].reshape(-1)
        n = ids.numel()
        row = w.scheme == "fp8row"
        fp8 = w.scheme in ("fp8row", "fp8", "fp8s")
        # a decoding step's few rows: the narrow projections run with their K dimension cut into slices
        row_gemm = ops.fp8_rowwise_gemm_small if attend is not None and n <= 128 else ops.fp8_rowwise_gemm
        tables = {k: ops.rope_table(pos, f) for k, f in self.inv_freq.items()}
        h = ops.embed_scale(ids, w.embed, self.embed_scale)
        for start, obj in inputs.get("media", ()):  # the media rows over their placeholders, not scaled (gemma4.py:410-413)
            if obj.embeds is not None:
                h[start : start + obj.n_tokens] = obj.embeds.to(device=h.device, dtype=h.dtype)
        if self.n_layers == 0:
            out = ops.fused_norm(h, w2=w.norm, rows=rows, eps=cfg.eps, want_norm=True)["norm"]
            return out if rows is not None else out[None]
        r = ops.fused_norm(h, w2=w.layers[0]["input_ln"], eps=cfg.eps, want_fp8=row, want_norm=not row)
        for i in range(self.n_layers):
            L = w.layers[i]
            kind = cfg.layer_types[i]
            cos, sin = tables[kind]
            if fp8:
                x8, xs = (r["x8"], r["xs"]) if row else self._quant_in(r["norm"], L, ("q", "k", "v"))
            if fp8 and self.fuse_qkv:  # head norms + rotary in the projection's epilogue
                qkv = ops.fp8_gemm_qkv(x8, xs, L["qkv_w"], L["qkv_s"], H, K, D, L["q_norm"], L["k_norm"], cos, sin, cfg.eps)
            else:
                qkv = ops.fp8_rowwise_gemm(x8, xs, L["qkv_w"], L["qkv_s"]) if fp8 else self._linear(r["norm"], L, "qkv", ("q", "k", "v"))
                ops.qkv_norm_rope(qkv, H, K, D, L["q_norm"], L["k_norm"], cos, sin, cfg.eps)
            q = qkv[:, : H * D].view(n, H, D)
            k = qkv[:, H * D : (H + K) * D].view(n, K, D)
            v = qkv[:, (H + K) * D :].view(n, K, D)
            if self._cap is not None:
                keep = self._cap["window"] - 1
                for start, cnt, key in self._cap["ranges"]:
                    a0 = start + (max(0, cnt - keep) if kind == "sliding_attention" else 0)
                    self._cap["kv"].setdefault(key, {})[i] = (k[a0 : start + cnt].clone(), v[a0 : start + cnt].clone())
            if attend is not None:
                a = attend(i, kind, q, k, v)
                amax = None
            else:
                amax = torch.zeros(n, dtype=torch.float32, device=qkv.device) if row else None
                ops.COUNTS["launches"] += 1 if row else 0
                a = attention.tree_attention(q, k, v, masks[kind], 1.0, row_amax=amax)  # scaling = 1.0: q and k are normed
            if row:  # the tree attention kernel has already found the row maxima
                a8, a_s = ops.fp8_quant_from_amax(a.view(n, H * D), amax) if amax is not None else ops.fp8_rowwise_quant(a.view(n, H * D))
                o = row_gemm(a8, a_s, L["o_w"], L["o_s"])
            else:
                o = self._linear(a.view(n, H * D), L, "o", ("o",))
            r = ops.fused_norm(o, w1=L["post_attn_ln"], residual=h, w2=L["pre_ffn_ln"], eps=cfg.eps, want_h=True, want_fp8=row,
                               want_norm=not row)
            h = r["h"]
            if row:
                g8, g_s, _ = ops.fp8_gemm_glu(r["x8"], r["xs"], L["gu_w"], L["gu_s"], "gelu_tanh")
                d = row_gemm(g8, g_s, L["down_w"], L["down_s"])
            else:
                gu = self._linear(r["norm"], L, "gu", ("gate", "up"))
                d = self._linear(ops.glu_quant(gu, "gelu_tanh", want_fp8=False, want_y=True)[2], L, "down", ("down",))
            last = i == self.n_layers - 1
            r = ops.fused_norm(
                d, w1=L["post_ffn_ln"], residual=h, w2=None if last else w.layers[i + 1]["input_ln"], eps=cfg.eps, want_h=True,
                want_fp8=row and not last, want_norm=not row and not last,
            )
            h = r["h"]
            if taps is not None:
                taps[i] = {"q": q.clone(), "k": k.clone(), "v": v.clone(), "attn": a, "h": h}
        out = ops.fused_norm(h, w2=w.norm, rows=rows, eps=cfg.eps, want_norm=True)["norm"]
        return out if rows is not None else out[None]


def calibrate(cfg: GemmaConfig, W, batches, device, headroom: float = 2.0, n_layers=None):
    """Makes an fp8s scale table as the reference's calibration does (spinf_serve/quant/calibrate.py:100-178): run the model with the
    dynamic fp8 scheme over `batches` (packer Batches covering what the model will see), record the largest |input| of every
    quantized linear, and set scale = 2^ceil(log2(headroom x amax / 448)). -> {"scheme": "fp8s", "headroom", "amax": [{name: v}],
    "scales": [{name: s}]}, one dict per layer; `scales` is what GemmaWeights.from_bf16(..., scheme="fp8s", scales=...) takes."""
    from spinf_serve_b200.scorer import stage_one

    stack = GemmaStack(GemmaWeights.from_bf16(cfg, W, device, scheme="fp8"), n_layers)
    amax = [dict.fromkeys(LINEARS, 0.0) for _ in range(stack.n_layers)]
    for b in batches:
        stack.amax_log = []
        sc, inputs, masks, _ = stage_one(stack, b, device)
        stack.forward(sc, b, inputs, masks)
        per_layer = len(LINEARS)
        logged = [(k, float(v)) for k, v in stack.amax_log]  # read back after the forward: no sync inside it
        for j, (k, v) in enumerate(logged):
            i = j // per_layer
            amax[i][k] = max(amax[i][k], v)
        stack.amax_log = None
    return {
        "scheme": "fp8s", "headroom": headroom, "amax": amax,
        "scales": [{k: static_scale(v, headroom) for k, v in a.items()} for a in amax],
    }
