"""CPU pins of the model-level oracle and of the scorer's host logic.

(1) oracle.gemma (the restated Gemma-style layer) against the installed transformers Gemma 4 text model, the module code the
    reference instantiates (spinf_serve/models/gemma4.py:134-143): same weights, the oracle's row-wise fp8 linear swapped in for
    every nn.Linear as the reference's build_model does, the oracle's dense-mask attention registered at an attention-interface
    seam as the reference's register_flex does (gemma4.py:99-121).
(2) read geometry: _cols / read_grouped / _drain against a fake model whose log-prob is a function of (previous token, target),
    the idea of the reference's tests/test_protocol_compiler.py:216-264."""

import numpy as np
import pytest
import torch

from oracle import attention as OA
from oracle import gemma as OG
from oracle import linears as OL
from spinf_serve_b200 import packer as P


def _tiny():
    return OG.GemmaConfig(layers=3, hidden=128, heads=4, kv_heads=2, head_dim=32, ffn=256, vocab=512, window=24, pattern=2)


def _stream(seed=0, align=True):
    rng = np.random.default_rng(seed)
    pk = P.Packer(1024, 4096, align=align)
    for j in range(2):
        trunk = rng.integers(1, 500, int(rng.integers(30, 90))).tolist()
        prompts = [trunk + [400 + q] + rng.integers(1, 500, int(rng.integers(2, 9))).tolist() for q in range(3)]
        list(pk.push(j, P.build_grouped_tree(prompts, [P.ReadPlan.build([[11], [12, 13]]) for _ in prompts])))
    (b,) = list(pk.flush())
    return b


def test_oracle_layer_equals_transformers_gemma4():
    tr = pytest.importorskip("transformers")
    from transformers import AttentionInterface
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
    from transformers.models.gemma4.modeling_gemma4 import Gemma4TextModel

    cfg = _tiny()
    W = OG.init_weights(cfg, seed=1)
    Q = OG.quantize(W)
    b = _stream()

    class OracleFp8RowLinear(torch.nn.Module):
        def __init__(self, w8, ws):
            super().__init__()
            self.w8, self.ws = w8, ws

        def forward(self, x):
            return OL.fp8_row_linear(x, self.w8, self.ws)

    def oracle_attention(module, query, key, value, attention_mask, scaling=None, sliding_window=None, **kw):
        art, end, pos = attention_mask
        out = OA.tree_attention(query[0].transpose(0, 1), key[0].transpose(0, 1), value[0].transpose(0, 1), art, end, pos, scaling, sliding_window)
        return out.to(query.dtype)[None], None

    AttentionInterface.register("oracle_tree", oracle_attention)
    hf = Gemma4TextConfig(
        vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.ffn, num_hidden_layers=cfg.layers,
        num_attention_heads=cfg.heads, num_key_value_heads=cfg.kv_heads, head_dim=cfg.head_dim, global_head_dim=cfg.head_dim,
        sliding_window=cfg.window, layer_types=list(cfg.layer_types), hidden_size_per_layer_input=0, use_cache=False,
        rope_parameters={
            "sliding_attention": {"rope_type": "default", "rope_theta": cfg.theta_sliding},
            "full_attention": {"rope_type": "default", "rope_theta": cfg.theta_full},
        },
    )
    hf._attn_implementation = "oracle_tree"
    model = Gemma4TextModel(hf).to(torch.bfloat16).eval()
    model.rotary_emb = type(model.rotary_emb)(hf)  # fp32 inv_freq, as the reference rebuilds it after loading (gemma4.py:166)
    with torch.no_grad():
        model.embed_tokens.weight.copy_(W["embed"])
        model.norm.weight.copy_(W["norm"])
        for layer, L, q8 in zip(model.layers, W["layers"], Q):
            at, mlp = layer.self_attn, layer.mlp
            at.q_proj, at.k_proj, at.v_proj, at.o_proj = (OracleFp8RowLinear(*q8[k]) for k in ("q", "k", "v", "o"))
            mlp.gate_proj, mlp.up_proj, mlp.down_proj = (OracleFp8RowLinear(*q8[k]) for k in ("gate", "up", "down"))
            at.q_norm.weight.copy_(L["q_norm"])
            at.k_norm.weight.copy_(L["k_norm"])
            for name, key in (("input_layernorm", "input_ln"), ("post_attention_layernorm", "post_attn_ln"),
                              ("pre_feedforward_layernorm", "pre_ffn_ln"), ("post_feedforward_layernorm", "post_ffn_ln")):
                getattr(layer, name).weight.copy_(L[key])
        info = (b.art, b.end, b.pos)
        out = model(
            input_ids=torch.from_numpy(b.ids)[None], position_ids=torch.from_numpy(b.pos.astype(np.int64))[None],
            attention_mask={"full_attention": info, "sliding_attention": info},
        ).last_hidden_state[0]
    mine = OG.forward(cfg, W, Q, b.ids, b.art, b.end, b.pos)
    real = torch.from_numpy(b.art >= 0)
    assert torch.equal(mine[real], out[real])


def test_read_geometry_with_a_fake_model():
    """every option's log-prob is the sum over its tokens of fake_lp(token before the read row, target)"""
    from spinf_serve_b200.scorer import Scorer, read_grouped

    def fake_lp(prev, target):
        return -((prev * 31 + target * 7) % 97) / 10.0

    rng = np.random.default_rng(4)
    items, truth = [], {}
    for j in range(5):
        trunk = rng.integers(1, 300, int(rng.integers(1, 60))).tolist()
        prompts = [trunk + rng.integers(1, 300, int(rng.integers(1, 7))).tolist() for _ in range(int(rng.integers(1, 6)))]
        options = [[rng.integers(1, 40, int(rng.integers(1, 4))).tolist() for _ in range(int(rng.integers(2, 5)))] for _ in prompts]
        plans = [P.ReadPlan.build(o) for o in options]
        items.append((("job", j), 0, P.build_grouped_tree(prompts, plans)))
        truth[("job", j)] = [
            [sum(fake_lp((pr + opt)[len(pr) - 1 + i], opt[i]) for i in range(len(opt))) for opt in opts] for pr, opts in zip(prompts, options)
        ]
    pk = P.Packer(512, 4096, align=True)
    batches = [b for key, first, t in items for b in pk.push((key, first), t, window=2)] + list(pk.flush())
    out = {key: [None] * len(t.plans) for key, _, t in items}
    for b in batches:
        cols = Scorer._cols(b)
        assert cols == sorted(set(cols))
        lp = np.array([[fake_lp(int(b.ids[q]), c) for c in cols] for q in b.sel], np.float32).reshape(len(b.sel), len(cols))
        read_grouped(lp, cols, b, out)
    for key, want in truth.items():
        for got, w in zip(out[key], want):
            assert np.allclose(got, w, atol=1e-4)


def test_v0_drain_with_a_fake_model():
    from spinf_serve_b200.scorer import JobResult, Scorer, read_trees

    def fake_lp(prev, target):
        return -((prev * 13 + target * 5) % 89) / 10.0

    prompts = [[1, 2, 3, 4], [1, 2, 3, 9, 8]]
    options = [[[20], [21, 22], [21, 23]], [[30, 31, 32], [33]]]
    t = P.build_tree(prompts, options)
    pk = P.Packer(256)
    list(pk.push(("a", 0), t))
    (b,) = list(pk.flush())
    cols = Scorer._cols(b)
    lp = np.array([[fake_lp(int(b.ids[q]), c) for c in cols] for q in b.sel], np.float32)
    res = {"a": JobResult([[0.0] * len(o) for o in options])}
    read_trees(lp, cols, b, res)
    for pr, opts, got in zip(prompts, options, res["a"].logprobs):
        for opt, g in zip(opts, got):
            want = sum(fake_lp((pr + opt)[len(pr) - 1 + i], opt[i]) for i in range(len(opt)))
            assert abs(g - want) < 1e-4
