"""Oracle of the Gemma-style packed forward (CPU torch; test infrastructure only, never imported by the product).

The reference builds transformers' Gemma 4 text model, swaps every nn.Linear of the decoder layers for a quantized one and
registers its attention at the "tree_flex" seam (spinf_serve/models/gemma4.py:134-143, :99-121; forward at :407-415). The layer
arithmetic therefore lives in the third-party dependency `transformers` (pinned 5.16.1 by the reference, 5.5.0 installed here):
Gemma4RMSNorm, Gemma4TextAttention, Gemma4TextMLP, Gemma4TextDecoderLayer, Gemma4TextScaledWordEmbedding. This file restates that
published layer with the reference's own pieces plugged in: row-wise fp8 linears (oracle.linears, spinf_serve/quant/linears.py:
84-96), the tree mask (oracle.attention, spinf_serve/scorer.py:173-177) and the lm-head read (oracle.head, scorer.py:340-355).
tests/test_model_host.py pins it against the installed transformers model run with the same weights.

Synthetic configuration: every layer has the same head_dim and default rotary embeddings (theta 10 000 on sliding layers, 1 000 000
on full layers); per-layer inputs, KV sharing, MoE blocks and soft-capping are off, as in the benchmark configurations."""

from dataclasses import dataclass, field

import numpy as np
import torch

from oracle import attention as OA
from oracle import head as OH
from oracle import linears as OL


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
    pattern: int = 6  # every pattern-th layer is full attention, the rest sliding
    eps: float = 1e-6
    theta_sliding: float = 10_000.0
    theta_full: float = 1_000_000.0
    softcap: float | None = None
    layer_types: list = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["sliding_attention" if (i + 1) % self.pattern else "full_attention" for i in range(self.layers)]
            if self.layer_types:
                self.layer_types[-1] = "full_attention"  # the model code forces the last layer to full attention


def init_weights(cfg: GemmaConfig, seed: int = 0, device="cpu"):
    """random-init bf16 weights of the architecture: linears N(0, 0.02), embedding N(0, 0.02), norm weights 1 + N(0, 0.1)"""
    g = torch.Generator(device=device).manual_seed(seed)

    def lin(o, i):
        return (torch.randn((o, i), generator=g, device=device) * 0.02).to(torch.bfloat16)

    def nw(d):
        return (1.0 + 0.1 * torch.randn(d, generator=g, device=device)).to(torch.bfloat16)

    H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    W = {"embed": lin(cfg.vocab, cfg.hidden), "norm": nw(cfg.hidden), "layers": []}
    for _ in range(cfg.layers):
        W["layers"].append(
            {
                "q": lin(H * D, cfg.hidden), "k": lin(K * D, cfg.hidden), "v": lin(K * D, cfg.hidden), "o": lin(cfg.hidden, H * D),
                "gate": lin(cfg.ffn, cfg.hidden), "up": lin(cfg.ffn, cfg.hidden), "down": lin(cfg.hidden, cfg.ffn),
                "q_norm": nw(D), "k_norm": nw(D),
                "input_ln": nw(cfg.hidden), "post_attn_ln": nw(cfg.hidden), "pre_ffn_ln": nw(cfg.hidden), "post_ffn_ln": nw(cfg.hidden),
            }
        )
    return W


def rmsnorm(x, w, eps):
    """Gemma4RMSNorm: x * pow(mean(x^2) + eps, -0.5) [* w], fp32, rounded to the input dtype"""
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


def rope_tables(pos, dim, theta):
    """(cos, sin) [n, dim] bf16 as Gemma4TextRotaryEmbedding.forward returns them (default rope type)"""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    freqs = torch.as_tensor(np.asarray(pos), dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


def apply_rope(x, cos, sin):
    """x [n, heads, D] bf16: (x * cos) + (rotate_half(x) * sin), every product and the sum rounded to bf16"""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos[:, None, :]) + (rot * sin[:, None, :])


LINEARS = ("q", "k", "v", "o", "gate", "up", "down")


def quantize(W, scheme="fp8row"):
    """per-linear (w8 [out, in] e4m3, ws fp32: [1, out] for fp8row, one scalar for the per-tensor schemes fp8 / fp8s) with the
    q|k|v and gate|up projections kept separate, as the reference's module swap leaves them (spinf_serve/quant/linears.py:66-106)"""
    fn = {"fp8row": OL.quantize_weight_rowwise, "fp8": OL.quantize_weight, "fp8s": OL.quantize_weight,
          "w8a8": OL.quantize_weight_int8, "w8a16": OL.quantize_weight_int8, "bf16": lambda w: (w, None)}[scheme]
    return [{k: fn(L[k]) for k in LINEARS} for L in W["layers"]]


def forward(cfg: GemmaConfig, W, Q, ids, art, end, pos, n_layers=None, taps=None, scheme="fp8row", scales=None, amax=None, peaks=None,
            attend=None, grp=None, bidir_all=True, media=()):
    """packed forward -> final hidden states [n, hidden] bf16 (after the model's last norm), the oracle of Gemma4Stack.forward
    (spinf_serve/models/gemma4.py:407-415). taps: optional dict filled with intermediate tensors for operator-level checks.
    scheme: fp8row (Fp8RowLinear), fp8 (Fp8Linear: dynamic per-tensor), fp8s (Fp8StaticLinear with scales[i][name]), w8a8 / w8a16
    (Int8Linear with int8 / bf16 activations) or bf16 (the unquantized linears).
    amax: optional list of per-layer dicts updated with the largest |input| of every linear (what the reference's calibration
    hooks record, quant/calibrate.py:117-124); peaks: the same for the static scheme's monitor (max|x| / (448 scale)).
    attend(layer, kind, q, k, v) -> [n, H, D]: another attention in place of the tree attention (a decoding step, where
    transformers' layers call the "x_decode" interface instead: spinf_serve/decode.py:359-377); art / end are unused then.
    Streams with images: grp (Batch.grp) and bidir_all select the full_img / sliding_img mask rules (spinf_serve/scorer.py:178-198);
    media = [(start, embeds [m, hidden])]: rows laid over the placeholders' embeddings, not scaled (gemma4.py:410-413)."""
    n = len(ids)
    H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    layer = [0]

    def lin(x, key, q):
        if amax is not None:
            amax[layer[0]][key] = max(amax[layer[0]][key], float(x.float().abs().max()))
        if scheme == "fp8row":
            return OL.fp8_row_linear(x, *q[key])
        if scheme == "fp8":
            return OL.fp8_linear(x, *q[key])
        if scheme in ("w8a8", "w8a16"):  # Int8Linear with int8 or bf16 activations (linears.py:55-64)
            return OL.int8_linear(x, *q[key], scheme == "w8a8")
        if scheme == "bf16":
            return torch.nn.functional.linear(x, q[key][0])
        y, pk = OL.fp8_static_linear(x, *q[key], torch.tensor(scales[layer[0]][key], dtype=torch.float32))
        if peaks is not None:
            peaks[(layer[0], key)] = max(peaks.get((layer[0], key), 0.0), float(pk))
        return y

    h = W["embed"][torch.as_tensor(np.asarray(ids), dtype=torch.int64)] * torch.tensor(cfg.hidden**0.5).to(torch.bfloat16)
    for start, e in media:
        h[start : start + len(e)] = e.to(h.dtype)
    tables = {"sliding_attention": rope_tables(pos, D, cfg.theta_sliding), "full_attention": rope_tables(pos, D, cfg.theta_full)}
    for i in range(cfg.layers if n_layers is None else n_layers):
        L, q8 = W["layers"][i], Q[i]
        layer[0] = i
        kind = cfg.layer_types[i]
        cos, sin = tables[kind]
        x = rmsnorm(h, L["input_ln"], cfg.eps)
        q = rmsnorm(lin(x, "q", q8).view(n, H, D), L["q_norm"], cfg.eps)
        k = rmsnorm(lin(x, "k", q8).view(n, K, D), L["k_norm"], cfg.eps)
        v = rmsnorm(lin(x, "v", q8).view(n, K, D), None, cfg.eps)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        window = cfg.window if kind == "sliding_attention" else None
        if attend is not None:
            a = attend(i, kind, q, k, v)
        else:
            g = grp if (bidir_all or window) else None  # global layers stay causal when the images' blocks are sliding-only
            a = OA.tree_attention(q, k, v, art, end, pos, 1.0, window, grp=g, grp_in_window=not bidir_all).to(torch.bfloat16)  # scaling = 1.0
        o = lin(a.reshape(n, H * D), "o", q8)
        h = h + rmsnorm(o, L["post_attn_ln"], cfg.eps)
        x = rmsnorm(h, L["pre_ffn_ln"], cfg.eps)
        act = torch.nn.functional.gelu(lin(x, "gate", q8), approximate="tanh") * lin(x, "up", q8)
        d = lin(act, "down", q8)
        h = h + rmsnorm(d, L["post_ffn_ln"], cfg.eps)
        if taps is not None:
            taps[i] = {"q": q, "k": k, "v": v, "attn": a, "h": h.clone()}
    return rmsnorm(h, W["norm"], cfg.eps)


def calibrate(cfg: GemmaConfig, W, batches, headroom=2.0, n_layers=None):
    """the fp8s scale table: the dynamic scheme run over `batches`, the largest input of every linear, and the power-of-two rule
    (spinf_serve/quant/calibrate.py:100-178 without the service around it) -> {"amax": [...], "scales": [...]} per layer"""
    nl = cfg.layers if n_layers is None else n_layers
    Q = quantize(W, "fp8")
    amax = [dict.fromkeys(LINEARS, 0.0) for _ in range(nl)]
    for b in batches:
        forward(cfg, W, Q, b.ids, b.art, b.end, b.pos, n_layers, scheme="fp8", amax=amax)
    return {"amax": amax, "scales": [{k: OL.static_scale(v, headroom) for k, v in a.items()} for a in amax]}


def score(cfg: GemmaConfig, W, Q, batch, cols, n_layers=None):
    """one packed batch -> option log-probs [len(sel), len(cols)] fp32: Scorer._forward (spinf_serve/scorer.py:241-261)"""
    hf = forward(cfg, W, Q, batch.ids, batch.art, batch.end, batch.pos, n_layers)
    sel = torch.as_tensor(batch.sel, dtype=torch.int64)
    return OH.option_logprobs(hf[sel], W["embed"], cols, cfg.softcap)  # tied lm head (gemma4.py:249)
