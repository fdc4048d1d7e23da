"""GPU parity of the tcgen05 GEMMs (through the C ABI) against the CPU oracle: row-wise fp8 quantiser + GEMM
(spinf_serve/quant/linears.py:29-33,84-96), plain bf16 GEMM, and batch invariance of rows across M."""

import numpy as np
import pytest
import torch

from oracle import linears as O

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,K", [(1, 64), (7, 3840), (128, 4096), (300, 15360), (1000, 5376)])
def test_rowwise_quant_bit_exact(dev, M, K):
    """x8 and xs equal the oracle's bit for bit (true division, clamp, round-to-nearest-even)"""
    from spinf_serve_b200 import ops

    x = _rand((M, K), 1, 3.0)
    x[0, : min(K, 16)] = 0  # a run of zeros
    x[0, min(K, 16) : min(K, 32)] = -0.0  # negative zeros keep their sign through the division
    if M > 2:
        x[2] = 0  # an all-zero row: the scale clamps at 1e-12 / 448
    x8, xs = ops.fp8_rowwise_quant(x.to(dev))
    r8, rs = O.quant_act_row(x)
    assert torch.equal(xs.cpu(), rs)
    assert torch.equal(x8.cpu().view(torch.uint8), r8.view(torch.uint8))


# (M, N, K): ragged M, one tile, the cfg-2 projection shapes at reduced M, K with a tail block
SHAPES = [(128, 256, 128), (1, 256, 256), (130, 512, 384), (257, 2048, 3840), (640, 3840, 4096), (384, 15360, 3840), (200, 3840, 15360), (100, 304, 208)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_fp8_rowwise_gemm_vs_oracle(dev, M, N, K):
    from spinf_serve_b200 import ops

    x = _rand((M, K), 2)
    w = _rand((N, K), 3, 0.02)
    w8, ws = O.quantize_weight_rowwise(w)
    x8, xs = O.quant_act_row(x)
    y = ops.fp8_rowwise_gemm(x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev)).cpu()
    exact = O.scaled_mm_rowwise(x8, xs, w8, ws, exact=True)
    # the exact product rounded to bf16 is at most half an ulp away; the fp32 tensor-core accumulation adds a little
    err = (y.double() - exact).abs()
    tol = exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-14
    assert bool((err <= tol).all()), f"max err {err.max():.3e} at |ref| {exact.abs().max():.3e}"
    ref = O.scaled_mm_rowwise(x8, xs, w8, ws)
    mism = (y != ref).float().mean().item()
    print(f"fp8 gemm {M}x{N}x{K}: max abs err vs exact {err.max():.3e}, rows differing from fp32-oracle bf16: {mism:.4%}")
    assert mism < 0.05  # same value up to the last bf16 bit on almost every element


# the 12B-class down and o projections at a decoding step's rows (the second too short to slice), a ragged last slice and
# ragged column tile, one row
@pytest.mark.parametrize("M,N,K", [(120, 3840, 15360), (120, 3840, 4096), (36, 1072, 15104), (128, 304, 208), (1, 2048, 12288)])
def test_fp8_few_rows_with_k_slices(dev, M, N, K):
    """the few-row entry point: same bound against the exact product as the plain kernel, rows independent of their neighbours,
    run-to-run identical"""
    from spinf_serve_b200 import ops

    x = _rand((M, K), 12)
    w = _rand((N, K), 13, 0.02)
    w8, ws = O.quantize_weight_rowwise(w)
    x8, xs = O.quant_act_row(x)
    d8, ds, dw, dws = x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev)
    y = ops.fp8_rowwise_gemm_small(d8, ds, dw, dws)
    exact = O.scaled_mm_rowwise(x8, xs, w8, ws, exact=True)
    err = (y.cpu().double() - exact).abs()
    tol = exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-14
    assert bool((err <= tol).all()), f"max err {err.max():.3e} at |ref| {exact.abs().max():.3e}"
    plain = ops.fp8_rowwise_gemm(d8, ds, dw, dws)
    mism = (y != plain).float().mean().item()
    print(f"fp8 few rows {M}x{N}x{K}: differs from the unsliced kernel on {mism:.4%} of the elements")
    assert mism < 0.05
    assert torch.equal(ops.fp8_rowwise_gemm_small(d8, ds, dw, dws), y)
    one = ops.fp8_rowwise_gemm_small(d8[:1].contiguous(), ds[:1].contiguous(), dw, dws)
    assert torch.equal(one, y[:1])  # the slicing does not depend on M


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (3, 512, 128), (300, 3840, 4096), (1000, 1024, 5120)])
def test_bf16_gemm_vs_oracle(dev, M, N, K):
    from spinf_serve_b200 import ops

    x = _rand((M, K), 4)
    w = _rand((N, K), 5, 0.05)
    y = ops.bf16_gemm(x.to(dev), w.to(dev)).cpu()
    exact = x.double() @ w.double().t()
    err = (y.double() - exact).abs()
    tol = exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-13
    assert bool((err <= tol).all()), f"max err {err.max():.3e}"


def test_fp8_gemm_rows_do_not_depend_on_M(dev):
    """batch invariance: the first rows of the product are bit-identical for M = 1, 100, 128, 1000, 4096"""
    from spinf_serve_b200 import ops

    K, N = 3840, 2048
    x = _rand((4096, K), 6)
    w8, ws = O.quantize_weight_rowwise(_rand((N, K), 7, 0.02))
    x8, xs = O.quant_act_row(x)
    x8, xs, w8, ws = x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev)
    full = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    for M in (1, 100, 128, 1000):
        part = ops.fp8_rowwise_gemm(x8[:M].contiguous(), xs[:M].contiguous(), w8, ws)
        assert torch.equal(part, full[:M])
    again = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    assert torch.equal(again, full)  # run-to-run determinism


@pytest.mark.parametrize("M,F,K,act", [(300, 1024, 512, "gelu_tanh"), (130, 15360, 3840, "gelu_tanh"), (64, 256, 128, "silu")])
def test_fused_glu_gemm_equals_the_unfused_chain(dev, M, F, K, act):
    """gate|up GEMM with the gated activation in its epilogue == row-wise GEMM followed by the activation kernel, bit for bit
    (same rounding chain), and both quantised forms agree with the oracle's quantiser applied to the kernel's bf16 output"""
    from spinf_serve_b200 import ops

    x = _rand((M, K), 8)
    w8, ws = O.quantize_weight_rowwise(_rand((2 * F, K), 9, 0.02))
    x8, xs = O.quant_act_row(x)
    x8, xs, w8, ws = x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev).reshape(-1)
    gu = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
    u8, us, y_ref = ops.glu_quant(gu, act, want_fp8=True, want_y=True)
    order = ops.glu_tile_order(F).to(dev)
    f8, fs, y = ops.fp8_gemm_glu(x8, xs, w8.view(torch.uint8)[order].view(torch.float8_e4m3fn).contiguous(), ws[order].contiguous(), act)
    assert torch.equal(y, y_ref)
    assert torch.equal(fs, us) and torch.equal(f8.view(torch.uint8), u8.view(torch.uint8))
    k8, ks = O.quant_act_row(y.cpu())
    assert torch.equal(fs.cpu(), ks) and torch.equal(f8.cpu().view(torch.uint8), k8.view(torch.uint8))


@pytest.mark.parametrize("M,H,Hkv,D,K", [(300, 4, 2, 128, 512), (517, 16, 8, 256, 3840), (64, 2, 1, 256, 256), (129, 6, 1, 128, 384)])
def test_fused_qkv_gemm_equals_gemm_then_norm_rope(dev, M, H, Hkv, D, K):
    """q|k|v projection with the head norms and rotary in its epilogue == the row-wise GEMM followed by the norm + rotary kernel.
    The rounding chain is the same; the fp32 sum of squares of a head is added in another order, so a last bf16 bit may flip
    on a few elements. A row's result does not depend on the rows packed beside it."""
    from oracle import gemma as OG
    from spinf_serve_b200 import ops

    N = (H + 2 * Hkv) * D
    x = _rand((M, K), 21)
    w8, ws = O.quantize_weight_rowwise(_rand((N, K), 22, 0.05))
    x8, xs = O.quant_act_row(x)
    x8, xs, w8, ws = x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev).reshape(-1)
    g = torch.Generator().manual_seed(23)
    wq = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(dev)
    wk = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(dev)
    pos = np.random.default_rng(1).integers(0, 4000, M).astype(np.int32)
    cos, sin = OG.rope_tables(pos, D, 10_000.0)
    cos, sin = cos[:, : D // 2].contiguous().to(dev), sin[:, : D // 2].contiguous().to(dev)
    for plus1, norm_v in ((False, True), (True, False)):
        ref = ops.fp8_rowwise_gemm(x8, xs, w8, ws)
        ops.qkv_norm_rope(ref, H, Hkv, D, wq, wk, cos, sin, 1e-6, plus1=plus1, norm_v=norm_v)
        got = ops.fp8_gemm_qkv(x8, xs, w8, ws, H, Hkv, D, wq, wk, cos, sin, 1e-6, plus1=plus1, norm_v=norm_v)
        differs = (got.float() != ref.float()).float().mean().item()
        print(f"M {M} heads {H}+2x{Hkv} D {D}: {differs:.5%} of elements differ")
        assert differs < 2e-3
        # a flipped last bit of a normed value moves a rotated output by one ulp of the larger of the pair it mixes
        assert (got.float() - ref.float()).abs().max() <= 2.0**-6 * ref.float().abs().max()
        if not norm_v:
            assert torch.equal(got[:, (H + Hkv) * D :], ref[:, (H + Hkv) * D :])  # values pass through untouched
        for m in (1, 100):
            m = min(m, M)
            part = ops.fp8_gemm_qkv(x8[:m].contiguous(), xs[:m].contiguous(), w8, ws, H, Hkv, D, wq, wk, cos[:m].contiguous(),
                                    sin[:m].contiguous(), 1e-6, plus1=plus1, norm_v=norm_v)
            assert torch.equal(part, got[:m])
