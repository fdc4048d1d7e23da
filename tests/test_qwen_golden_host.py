"""The oracles of the int4 linear, the hybrid layer pieces and the whole hybrid forward against outputs of the reference's own model
code run on the CPU (tests/golden/qwen_golden.npz, written by tests/golden/make_qwen_golden.py from build_model of
spinf_serve/models/qwen35/qwen.py on a synthetic GPTQ checkpoint). Element-wise steps must agree bit for bit; where a matrix
product is involved the two sides may sum in different orders, so a small fraction of elements may differ by one bf16 step."""

import os

import numpy as np
import torch

from oracle import attention as OA
from oracle import gdn as OGD
from oracle import linears as OL
from oracle import qwen as OQ
from spinf_serve_b200 import packer as P
from spinf_serve_b200.gdn_plan import tree_plan
from tests.golden.make_qwen_golden import SEED, SMALL, stream

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qwen_golden.npz"))
CFG = OQ.QwenConfig(**SMALL)
W = OQ.init_weights(CFG, seed=SEED)
REC, ATT = W["layers"][0], W["layers"][1]


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def close(mine, ref, frac=0.02, steps=1):
    """equal up to `steps` bf16 steps on at most `frac` of the elements"""
    d = (mine.float() - ref.float()).abs()
    tol = ref.float().abs() * 2.0**-7 * steps + ref.float().abs().max() * 2.0**-12  # the second term: sums that cancel to near zero
    return bool((d <= tol).all()) and (mine != ref).float().mean().item() <= frac


def lin(x, w, extra=None):
    return OL.int4_linear(x, *OL.gptq_unpack(*w), CFG.group, extra)


def test_dequantised_weight_is_the_reference_s_bit_for_bit():
    q, s = OL.gptq_unpack(*REC["down"])
    assert torch.equal(OL.dq_bf16(q, s, CFG.group), bf16(G["dq_down"]))


def test_int4_linears():
    x = bf16(G["x"])
    assert close(lin(x, REC["in_proj"], REC["in_extra"]), bf16(G["lin_in_proj"]))
    assert close(lin(x, ATT["qkv_proj"]), bf16(G["lin_qkv_proj"]))
    assert close(lin(x, REC["gate_up"]), bf16(G["lin_gate_up"]))
    for name, w in (("out_proj", REC["out_proj"]), ("o_proj", ATT["o_proj"]), ("down", REC["down"])):
        assert close(lin(bf16(G["xin_" + name]), w), bf16(G["lin_" + name]))


def test_rmsnorm_and_mlp():
    x = bf16(G["x"])
    assert torch.equal(OQ.rmsnorm(x, REC["input_ln"], CFG.eps), bf16(G["rmsnorm"]))
    gu = lin(x, REC["gate_up"])
    n = gu.shape[-1] // 2
    mlp = lin(torch.nn.functional.silu(gu[:, :n]) * gu[:, n:], REC["down"])
    assert close(mlp, bf16(G["mlp"]), frac=0.1, steps=2)  # two products in a row: a one-step difference in the first moves the second


def test_steps_before_the_recurrence_bit_for_bit():
    """on the reference's own in-projection output: path convolution, SiLU, l2 norms, beta, g (GatedDeltaNet.forward, qwen.py:651-668)"""
    b = stream(P)
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    q, k, v, z, g, beta = OGD.prologue(bf16(G["gdn_y"]), plan.conv, REC["conv_w"], REC["A_log"], REC["dt_bias"], CFG.hk, CFG.dk, CFG.hv, CFG.dv)
    real = torch.from_numpy(b.art >= 0)
    for mine, key in ((q, "gdn_q"), (k, "gdn_k"), (v, "gdn_v"), (beta, "gdn_beta")):
        ref = bf16(G[key]).reshape(mine.shape)
        assert torch.equal(mine[real], ref[real]), key
    assert np.array_equal(g[real].numpy(), G["gdn_g"][real.numpy()])


def test_steps_after_the_recurrence():
    """on the recurrence output the reference's layer was given: gated RMS norm (bit for bit up to the out-projection's summation)"""
    b = stream(P)
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    _, _, _, z, _, _ = OGD.prologue(bf16(G["gdn_y"]), plan.conv, REC["conv_w"], REC["A_log"], REC["dt_bias"], CFG.hk, CFG.dk, CFG.hv, CFG.dv)
    o = bf16(G["gdn_o"]).reshape(-1, CFG.hv, CFG.dv)
    out = lin(OGD.epilogue(o, z, REC["gdn_norm"], CFG.eps), REC["out_proj"])
    real = torch.from_numpy(b.art >= 0)
    assert close(out[real], bf16(G["gdn_out"])[real])


def test_recurrence_oracle_reproduces_what_the_layer_was_given():
    """the stand-in recurrence of the generator is this oracle: same inputs, same plan (the product's, bit-equal to the
    reference's), same output, so the recorded layer outputs belong to this recurrence"""
    b = stream(P)
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    q, k = bf16(G["gdn_q"]).reshape(-1, CFG.hk, CFG.dk), bf16(G["gdn_k"]).reshape(-1, CFG.hk, CFG.dk)
    v, beta = bf16(G["gdn_v"]).reshape(-1, CFG.hv, CFG.dv), bf16(G["gdn_beta"]).reshape(-1, CFG.hv)
    o = OGD.gdn_tree(q, k, v, torch.from_numpy(G["gdn_g"]), beta, plan)
    assert torch.equal(o, bf16(G["gdn_o"]).reshape(o.shape))


def test_attention_mixer():
    """projection, head norms with (1 + w), partial rotary embedding, the tree attention, the sigmoid gate, out-projection
    (Attention.forward, qwen.py:683-697; the reference side ran its eager FlexAttention with its BlockMask)"""
    b = stream(P)
    T = b.length
    H, K, D = CFG.heads, CFG.kv_heads, CFG.head_dim
    xa = bf16(G["xa"])
    inv_freq = 1.0 / (CFG.theta ** (torch.arange(0, CFG.rotary, 2, dtype=torch.float32) / CFG.rotary))
    f = torch.from_numpy(b.pos.astype(np.float32))[:, None] * inv_freq[None]
    e = torch.cat([f, f], -1)
    cos, sin = e.cos().to(torch.bfloat16), e.sin().to(torch.bfloat16)
    y = lin(xa, ATT["qkv_proj"])
    nq, nk = H * 2 * D, K * D
    qg = y[:, :nq].reshape(T, H, 2 * D)
    q, gate = qg[..., :D], qg[..., D:].reshape(T, -1)
    q = OQ.rope(OQ.rmsnorm(q, ATT["q_norm"], CFG.eps), cos, sin)
    k = OQ.rope(OQ.rmsnorm(y[:, nq : nq + nk].reshape(T, K, D), ATT["k_norm"], CFG.eps), cos, sin)
    v = y[:, nq + nk :].reshape(T, K, D)
    o = OA.tree_attention(q, k, v, b.art, b.end, b.pos, D**-0.5, None).to(torch.bfloat16)
    out = lin(o.reshape(T, -1) * torch.sigmoid(gate), ATT["o_proj"])
    real = torch.from_numpy(b.art >= 0)
    ref = bf16(G["attn_out"])
    d = (out.float() - ref.float())[real]
    # the two attentions round at different points (the reference's eager FlexAttention forms its products in bf16): single values
    # move by one bf16 step, 3e-3 of the rms overall
    assert float(d.abs().max()) <= 2.0**-7 * float(ref.float()[real].abs().max()) and float(d.pow(2).mean().sqrt()) < 5e-3 * float(ref.float()[real].pow(2).mean().sqrt())


def test_whole_forward_layer_by_layer():
    b = stream(P)
    plan = tree_plan(b.prev, b.art >= 0, "cpu")
    taps = {}
    out = OQ.forward(CFG, W, b.ids, b.art, b.end, b.pos, plan, taps=taps)
    real = torch.from_numpy(b.art >= 0)

    def rel(a, r):
        a, r = a[real].float(), r[real].float()
        return float((a - r).pow(2).mean().sqrt() / r.pow(2).mean().sqrt())

    errs = [rel(taps[i], bf16(G[f"resid{i}"])) for i in range(CFG.layers)] + [rel(out, bf16(G["final"]))]
    print("oracle vs the reference's model, rms err / rms per layer and final:", ["%.2e" % e for e in errs])
    # bf16 steps from summation order and the attention's rounding points only: 2e-4 after the first (recurrent) layer, 5e-3 after
    # four; a wrong formula anywhere shows as > 1e-1
    assert errs[0] < 1e-3 and max(errs) < 1e-2
