"""GPU parity of the fused layer-glue kernels against the oracle's module arithmetic (oracle.gemma: RMSNorm, rotary, GeGLU,
embedding scale as transformers' Gemma 4 layer computes them; row-wise fp8 quantiser as spinf_serve/quant/linears.py:29-33),
operator by operator on identical inputs."""

import numpy as np
import pytest
import torch

from oracle import gemma as OG
from oracle import linears as OL

pytestmark = pytest.mark.gpu


def _bf(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


def _frac_diff(a, b):
    return (a.float() != b.float()).float().mean().item()


@pytest.mark.parametrize("hidden", [512, 3840, 5376])
def test_fused_norm_chain(dev, hidden):
    from spinf_serve_b200 import ops

    n, eps = 77, 1e-6
    y, res = _bf((n, hidden), 1, 2.0), _bf((n, hidden), 2, 30.0)
    w1, w2 = (1 + 0.1 * _bf((hidden,), 3).float()).to(torch.bfloat16), (1 + 0.1 * _bf((hidden,), 4).float()).to(torch.bfloat16)
    h_ref = res + OG.rmsnorm(y, w1, eps)
    x_ref = OG.rmsnorm(h_ref, w2, eps)
    x8_ref, xs_ref = OL.quant_act_row(x_ref)
    r = ops.fused_norm(y.to(dev), w1=w1.to(dev), residual=res.to(dev), w2=w2.to(dev), eps=eps, want_h=True, want_norm=True, want_fp8=True)
    fh, fx = _frac_diff(r["h"].cpu(), h_ref), _frac_diff(r["norm"].cpu(), x_ref)
    print(f"hidden {hidden}: h differs on {fh:.4%}, norm on {fx:.4%}")
    assert fh < 1e-3 and fx < 1e-3  # fp32 reduction order and pow() may flip a last bf16 bit, rarely
    assert (r["h"].cpu().float() - h_ref.float()).abs().max() <= 2.0**-7 * h_ref.float().abs().max()
    # the quantiser applied to the kernel's own bf16 output is bit-exact
    k8, ks = OL.quant_act_row(r["norm"].cpu())
    assert torch.equal(r["xs"].cpu(), ks) and torch.equal(r["x8"].cpu().view(torch.uint8), k8.view(torch.uint8))
    # single norm + quantisation, and the row-selecting final norm
    r1 = ops.fused_norm(y.to(dev), w2=w2.to(dev), eps=eps, want_norm=True)
    assert _frac_diff(r1["norm"].cpu(), OG.rmsnorm(y, w2, eps)) < 1e-3
    rows = torch.tensor([5, 0, 76, 5], dtype=torch.int64)
    r2 = ops.fused_norm(y.to(dev), w2=w2.to(dev), rows=rows.to(dev), eps=eps, want_norm=True)
    assert torch.equal(r2["norm"], r1["norm"][rows.to(dev)])


@pytest.mark.parametrize("H,K,D", [(4, 2, 128), (16, 8, 256), (3, 1, 256)])
def test_qkv_norm_rope(dev, H, K, D):
    from spinf_serve_b200 import ops

    n, eps = 200, 1e-6
    qkv = _bf((n, (H + 2 * K) * D), 5, 3.0)
    wq, wk = (1 + 0.1 * _bf((D,), 6).float()).to(torch.bfloat16), (1 + 0.1 * _bf((D,), 7).float()).to(torch.bfloat16)
    pos = np.random.default_rng(0).integers(0, 3000, n).astype(np.int32)
    for theta in (10_000.0, 1_000_000.0):
        cos, sin = OG.rope_tables(pos, D, theta)
        q = OG.apply_rope(OG.rmsnorm(qkv[:, : H * D].view(n, H, D), wq, eps), cos, sin)
        k = OG.apply_rope(OG.rmsnorm(qkv[:, H * D : (H + K) * D].view(n, K, D), wk, eps), cos, sin)
        v = OG.rmsnorm(qkv[:, (H + K) * D :].view(n, K, D), None, eps)
        ref = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], dim=1)
        inv_freq = (1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))).to(dev)
        c_g, s_g = ops.rope_table(torch.from_numpy(pos).to(dev), inv_freq)
        ft = max(_frac_diff(c_g.cpu(), cos[:, : D // 2]), _frac_diff(s_g.cpu(), sin[:, : D // 2]))
        out = ops.qkv_norm_rope(qkv.to(dev).clone(), H, K, D, wq.to(dev), wk.to(dev), c_g, s_g, eps).cpu()
        f = _frac_diff(out, ref)
        print(f"H{H} K{K} D{D} theta {theta:g}: table differs on {ft:.4%}, output on {f:.4%}")
        assert ft < 2e-3 and f < 5e-3
        assert (out.float() - ref.float()).abs().max() <= 2.0**-6 * ref.float().abs().max()


@pytest.mark.parametrize("F", [1024, 15360])
def test_geglu_quant(dev, F):
    from spinf_serve_b200 import ops

    n = 50
    gu = _bf((n, 2 * F), 8, 2.0)
    ref = torch.nn.functional.gelu(gu[:, :F], approximate="tanh") * gu[:, F:]
    x8, xs, y = ops.glu_quant(gu.to(dev), "gelu_tanh", want_fp8=True, want_y=True)
    f = _frac_diff(y.cpu(), ref)
    print(f"F {F}: GeGLU differs on {f:.4%}")
    assert f < 2e-3 and (y.cpu().float() - ref.float()).abs().max() <= 2.0**-7 * ref.float().abs().max()
    k8, ks = OL.quant_act_row(y.cpu())
    assert torch.equal(xs.cpu(), ks) and torch.equal(x8.cpu().view(torch.uint8), k8.view(torch.uint8))
    ref_s = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    _, _, ys = ops.glu_quant(gu.to(dev), "silu", want_fp8=False, want_y=True)
    assert _frac_diff(ys.cpu(), ref_s) < 2e-3


def test_embed_scale(dev):
    from spinf_serve_b200 import ops

    emb = _bf((1000, 512), 9, 0.02)
    ids = torch.from_numpy(np.random.default_rng(1).integers(0, 1000, 300))
    scale = torch.tensor(512**0.5).to(torch.bfloat16)
    ref = emb[ids] * scale
    out = ops.embed_scale(ids.to(dev), emb.to(dev), float(scale)).cpu()
    assert torch.equal(out, ref)


def test_gelu_tanh_over_every_bf16_gate(dev):
    """the branch-free GELU of the kernels against torch's tanh-form GELU for every finite bf16 gate value (up = 1): the fp32
    expressions differ only in how tanh is evaluated, so after the bf16 rounding all but a handful of inputs agree exactly"""
    from spinf_serve_b200 import ops

    gate = (torch.arange(65536, dtype=torch.int32) << 16).view(torch.float32)
    finite = torch.isfinite(gate)
    gate = torch.where(finite, gate, torch.zeros(())).to(torch.bfloat16).view(64, 1024)
    gu = torch.cat([gate, torch.ones_like(gate)], dim=1).contiguous()
    _, _, y = ops.glu_quant(gu.to(dev), "gelu_tanh", want_fp8=False, want_y=True)
    ref = torch.nn.functional.gelu(gate.float(), approximate="tanh").to(torch.bfloat16)
    bad = y.cpu().float() != ref.float()
    print(f"GELU over all bf16 gates: {int(bad.sum())} of {int(finite.sum())} differ")
    assert int(bad.sum()) <= 64
    err = (y.cpu().float() - ref.float()).abs()
    assert (err <= 2.0**-7 * ref.float().abs() + 1e-6).all()


def test_silu_over_every_bf16_gate(dev):
    """the five-instruction SiLU of the kernels against torch's for every finite bf16 gate value (up = 1): after the bf16 rounding
    all but a handful of inputs agree exactly, the rest by one step"""
    from spinf_serve_b200 import ops

    gate = (torch.arange(65536, dtype=torch.int32) << 16).view(torch.float32)
    finite = torch.isfinite(gate)
    gate = torch.where(finite, gate, torch.zeros(())).to(torch.bfloat16).view(64, 1024)
    gu = torch.cat([gate, torch.ones_like(gate)], dim=1).contiguous()
    _, _, y = ops.glu_quant(gu.to(dev), "silu", want_fp8=False, want_y=True)
    ref = torch.nn.functional.silu(gate.float()).to(torch.bfloat16)
    bad = y.cpu().float() != ref.float()
    print(f"SiLU over all bf16 gates: {int(bad.sum())} of {int(finite.sum())} differ")
    assert int(bad.sum()) <= 64
    err = (y.cpu().float() - ref.float()).abs()
    assert (err <= 2.0**-7 * ref.float().abs() + 1e-30).all()
