"""Writes tests/golden/qwen_golden.npz: outputs of the reference's own Qwen-style hybrid model code run on the CPU.

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_qwen_golden.py <path of the reference checkout>

The reference builds its model classes (Int4Linear, RMSNorm, GatedDeltaNet, Attention, MLP, Layer, QwenTextModel) inside
build_model (spinf_serve/models/qwen35/qwen.py:280-945), which reads a checkpoint directory. This script writes a tiny synthetic
checkpoint in that format (config.json of model type qwen3_5 with a GPTQ int4 group-128 quantization_config, safetensors shards,
index file) from the oracle's seeded weights, calls the reference's build_model(cfg, dir, "cpu", QwenOptions(mode="bf16")) and runs
its modules on seeded inputs. TORCHDYNAMO_DISABLE makes the torch.compile decorators run their functions eagerly (same ops).

Two things of the reference cannot run on a CPU and are replaced while it runs, both outside the arithmetic that is recorded:
  * torch.cuda.synchronize / empty_cache (called at the end of build_model and in tune_orientation) are no-ops here;
  * gdn_tree (qwen.py:515-590) launches Triton kernels: the closure cell GatedDeltaNet.forward reads it from is pointed at a
    stand-in that records the q, k, v, g, beta it is given and returns the oracle's token-serial recurrence, so everything before
    and after the recurrence (in-projection, path convolution, SiLU, l2 norms, beta, g; gated RMS norm, out-projection) is the
    reference's own code acting on known inputs.
Recorded: a dequantised weight; every Int4Linear of one recurrent and one attention layer on a seeded input; RMSNorm, MLP, rope; the recurrent mixer's
q k v g beta and output; the attention mixer's output (the reference's eager FlexAttention with its BlockMask); every layer's
residual stream and the final hidden states of the whole model on a packed stream."""

import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SMALL = dict(layers=4, hidden=256, ffn=512, vocab=2048, hk=2, hv=4, dk=128, dv=128, heads=4, kv_heads=2, head_dim=128, rotary=32, group=128, every=2)
SEED = 3


def bits(t):
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def stream(P):
    """the packed stream every recorded forward runs on (the test rebuilds it from the same seed)"""
    rng = np.random.default_rng(2)

    def content(n_trunk, n_q):
        trunk = rng.integers(5, SMALL["vocab"], n_trunk).tolist()
        prompts = [trunk + [10 + i] + rng.integers(5, SMALL["vocab"], int(rng.integers(3, 14))).tolist() for i in range(n_q)]
        return P.build_grouped_tree(prompts, [P.ReadPlan.build([[7], [8], [9, 11]]) for _ in prompts])

    pk = P.Packer(2048, 8192, align=True)
    for j in range(2):
        list(pk.push(j, content(int(rng.integers(30, 90)), 3)))
    (b,) = list(pk.flush())
    return b


def write_checkpoint(path, cfg, W):
    from safetensors.torch import save_file

    kd, vd = cfg.hk * cfg.dk, cfg.hv * cfg.dv
    H, K, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    T = {}
    pre = "model.language_model."

    def int4(name, qw, sc):
        T[pre + name + ".qweight"] = qw.contiguous()
        T[pre + name + ".scales"] = sc.contiguous()
        T[pre + name + ".qzeros"] = torch.full((sc.shape[0], qw.shape[1] // 8), 0x77777777, dtype=torch.int32)

    def split(name_parts, pair, widths):
        qw, sc = pair
        a = 0
        for nm, w in zip(name_parts, widths):
            int4(nm, qw[:, a : a + w], sc[:, a : a + w])
            a += w

    for i, L in enumerate(W["layers"]):
        p = f"layers.{i}."
        T[pre + p + "input_layernorm.weight"] = L["input_ln"]
        T[pre + p + "post_attention_layernorm.weight"] = L["post_ln"]
        split([p + "mlp.gate_proj", p + "mlp.up_proj"], L["gate_up"], [cfg.ffn, cfg.ffn])
        int4(p + "mlp.down_proj", *L["down"])
        if L["kind"] == "linear_attention":
            la = p + "linear_attn."
            split([la + "in_proj_qkv", la + "in_proj_z"], L["in_proj"], [2 * kd + vd, vd])
            T[pre + la + "in_proj_b.weight"] = L["in_extra"][: cfg.hv].contiguous()
            T[pre + la + "in_proj_a.weight"] = L["in_extra"][cfg.hv :].contiguous()
            int4(la + "out_proj", *L["out_proj"])
            T[pre + la + "conv1d.weight"] = L["conv_w"][:, None, :].contiguous()
            T[pre + la + "norm.weight"] = L["gdn_norm"]
            T[pre + la + "A_log"] = L["A_log"]
            T[pre + la + "dt_bias"] = L["dt_bias"]
        else:
            sa = p + "self_attn."
            split([sa + "q_proj", sa + "k_proj", sa + "v_proj"], L["qkv_proj"], [2 * H * D, K * D, K * D])
            int4(sa + "o_proj", *L["o_proj"])
            T[pre + sa + "q_norm.weight"] = L["q_norm"]
            T[pre + sa + "k_norm.weight"] = L["k_norm"]
    T[pre + "norm.weight"] = W["norm"]
    T[pre + "embed_tokens.weight"] = W["embed"]
    T["lm_head.weight"] = W["lm_head"]
    save_file(T, os.path.join(path, "model-00001-of-00001.safetensors"))
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": dict.fromkeys(T, "model-00001-of-00001.safetensors")}, f)
    text = {
        "model_type": "qwen3_5_text", "hidden_size": cfg.hidden, "intermediate_size": cfg.ffn, "num_hidden_layers": cfg.layers, "vocab_size": cfg.vocab,
        "num_attention_heads": H, "num_key_value_heads": K, "head_dim": D, "rms_norm_eps": cfg.eps, "layer_types": cfg.layer_types,
        "linear_num_key_heads": cfg.hk, "linear_num_value_heads": cfg.hv, "linear_key_head_dim": cfg.dk, "linear_value_head_dim": cfg.dv,
        "linear_conv_kernel_dim": 4, "full_attention_interval": cfg.every,
        "rope_parameters": {"rope_type": "default", "rope_theta": cfg.theta, "partial_rotary_factor": cfg.rotary / D, "mrope_section": [cfg.rotary // 4, cfg.rotary // 8, cfg.rotary // 8], "mrope_interleaved": True},
    }
    conf = {"model_type": "qwen3_5", "text_config": text,
            "quantization_config": {"quant_method": "gptq", "bits": 4, "sym": True, "desc_act": False, "group_size": cfg.group}}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(conf, f)


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, ROOT)
    from spinf_serve import packer as RP
    from spinf_serve.config import EngineConfig
    from spinf_serve.models.qwen35 import qwen as RQ
    from torch.nn.attention.flex_attention import BlockMask

    from oracle import gdn as OGD
    from oracle import qwen as OQ

    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.empty_cache = lambda *a, **k: None
    cfg = OQ.QwenConfig(**SMALL)
    W = OQ.init_weights(cfg, seed=SEED)
    with tempfile.TemporaryDirectory() as d:
        write_checkpoint(d, cfg, W)
        ecfg = EngineConfig(model_dir=d, quant="bf16", token_budget=256, media=False)
        model, tcfg = RQ.build_model(ecfg, d, "cpu", RQ.QwenOptions(mode="bf16", embed_host=False, compact=False))
    assert model._quant == "int4-bf16", model._quant

    out = {}
    g = torch.Generator().manual_seed(11)
    rec, att = model.layers[0], model.layers[1]
    assert rec.kind == "linear_attention" and att.kind == "full_attention"
    # ---- every Int4Linear of a recurrent and an attention layer, RMSNorm, MLP
    x = (torch.randn((37, cfg.hidden), generator=g) * 0.7).to(torch.bfloat16)
    out["x"] = bits(x)
    for name, lin in (("in_proj", rec.linear_attn.in_proj_qkvz), ("qkv_proj", att.self_attn.qkv_proj), ("gate_up", rec.mlp.gate_up_proj)):
        out["lin_" + name] = bits(lin(x).to(torch.bfloat16))
    for name, lin in (("out_proj", rec.linear_attn.out_proj), ("o_proj", att.self_attn.o_proj), ("down", rec.mlp.down_proj)):
        xin = (torch.randn((37, lin.in_features), generator=g) * 0.7).to(torch.bfloat16)
        out["xin_" + name] = bits(xin)
        out["lin_" + name] = bits(lin(xin))
    fwd_l = type(rec.mlp.down_proj).forward
    dq_bf16 = fwd_l.__closure__[fwd_l.__code__.co_freevars.index("dq_bf16")].cell_contents
    out["dq_down"] = bits(dq_bf16(rec.mlp.down_proj.q, rec.mlp.down_proj.s))  # the dequantised weight itself (qwen.py:326-330)
    out["rmsnorm"] = bits(rec.input_layernorm(x))
    out["mlp"] = bits(rec.mlp(x))

    # ---- the packed stream, the reference's plan and mask
    b = stream(RP)
    n = b.length
    plan = RQ.tree_plan(b.prev, b.art >= 0, "cpu", path="indexed")
    art, end = torch.from_numpy(b.art.astype(np.int32)), torch.from_numpy(b.end.astype(np.int32))

    def full(bb, h, q, k):  # Scorer._init_flex (spinf_serve/scorer.py:173-174)
        return ((k <= q) & (art[q] >= 0) & (art[k] == art[q]) & (q < end[k])) | (q == k)

    pn, pi, fn, fi = [torch.from_numpy(t) for t in RP.block_tables(b.art, b.end, b.pos, None, None, True)[0]]
    mask = BlockMask.from_kv_blocks(pn[None, None], pi[None, None], fn[None, None], fi[None, None], BLOCK_SIZE=RP.BLOCK, mask_mod=full,
                                    seq_lengths=(n, n), compute_q_blocks=False)

    # ---- the recurrence's stand-in, through the closure cell GatedDeltaNet.forward reads gdn_tree from
    seen = []

    def gdn_stand_in(q, k, v, gl, beta, plan_, mod=None):
        seen.append((q.clone(), k.clone(), v.clone(), gl.clone(), beta.clone()))
        return OGD.gdn_tree(q, k, v, gl, beta, plan_)

    fwd = type(rec.linear_attn).forward
    fwd.__closure__[fwd.__code__.co_freevars.index("gdn_tree")].cell_contents = gdn_stand_in

    ids = torch.from_numpy(b.ids)
    pos = torch.from_numpy(b.pos.astype(np.int64))
    with torch.no_grad():
        h0 = rec.input_layernorm(model.embed_tokens(ids))
        out["gdn_y"] = bits(rec.linear_attn.in_proj_qkvz(h0).to(torch.bfloat16))  # what the steps before the recurrence read
        m0 = rec.linear_attn(h0, plan)
        q, k, v, gl, beta = seen[0]
        out["gdn_o"] = bits(OGD.gdn_tree(q, k, v, gl, beta, plan))                 # what the steps after it read
        out["gdn_q"], out["gdn_k"], out["gdn_v"], out["gdn_beta"] = bits(q), bits(k), bits(v), bits(beta)
        out["gdn_g"] = gl.float().numpy()
        out["gdn_out"] = bits(m0)
        # rope and the attention mixer on a seeded input
        f = pos.float()[:, None] * model.inv_freq[None]
        e = torch.cat([f, f], -1)
        cos, sin = e.cos().to(torch.bfloat16), e.sin().to(torch.bfloat16)
        xa = (torch.randn((n, cfg.hidden), generator=g) * 0.7).to(torch.bfloat16)
        out["xa"] = bits(xa)
        out["attn_out"] = bits(att.self_attn(xa, cos, sin, mask, plan))
        # the whole model, layer by layer
        xs = model.embed_tokens(ids)
        for i, layer in enumerate(model.layers):
            xs = layer(xs, cos, sin, mask, plan)
            out[f"resid{i}"] = bits(xs)
        out["final"] = bits(model.norm(xs))
        seen.clear()
        out["final_forward"] = bits(model(ids, pos, mask, plan))
    assert np.array_equal(out["final"], out["final_forward"])
    del out["final_forward"]
    np.savez_compressed(os.path.join(HERE, "qwen_golden.npz"), **out)
    print("stream", n, "real", int((b.art >= 0).sum()), "keys", len(out), "bytes", os.path.getsize(os.path.join(HERE, "qwen_golden.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
