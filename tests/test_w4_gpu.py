"""GPU parity of the int4 weight-only GEMM (through the C ABI) with the oracle of Int4Linear in bf16 mode
(spinf_serve/models/qwen35/qwen.py:383-391 unpack, :326-330 dq_bf16, :455-458 forward)."""

import pytest
import torch

from oracle import linears as O

pytestmark = pytest.mark.gpu


def _gptq(N, K, G, seed):
    g = torch.Generator().manual_seed(seed)
    nib = torch.randint(0, 16, (K, N), generator=g, dtype=torch.int32)
    qweight = torch.zeros((K // 8, N), dtype=torch.int32)
    for i in range(8):
        qweight |= nib[i::8] << (4 * i)
    scales = (torch.rand((K // G, N), generator=g) * 0.02 + 0.001).to(torch.float16)
    return qweight, scales


def _repack_host(q):
    """the layout spinf_w4_repack documents, restated with numpy: per 8 consecutive k (4 bytes), even k in nibbles 0..3, odd k in 4..7"""
    import numpy as np

    b = q.numpy().reshape(q.shape[0], -1, 4).astype(np.uint32)
    lo, hi = b & 15, b >> 4  # k = 2j, k = 2j + 1 of byte j
    w = sum(lo[..., j] << (4 * j) for j in range(4)) | sum(hi[..., j] << (16 + 4 * j) for j in range(4))
    return torch.from_numpy(w.astype("<u4").view(np.uint8).reshape(q.shape[0], -1).copy())


@pytest.mark.parametrize("M,N,K,G,E", [(256, 128, 64, 32, 0), (1, 256, 128, 128, 0), (300, 384, 512, 128, 64), (700, 5120, 4096, 128, 0), (130, 1024, 5120, 32, 64),
                                       (77, 200, 192, 64, 0), (513, 72, 128, 128, 0)])
def test_w4_linear_vs_oracle(dev, M, N, K, G, E):
    from spinf_serve_b200.linears import Int4Linear

    qweight, scales = _gptq(N, K, G, 1)
    g = torch.Generator().manual_seed(2)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    extra = (torch.randn((E, K), generator=g) * 0.05).to(torch.bfloat16) if E else None
    lin = Int4Linear(qweight.to(dev), scales.to(dev))
    assert lin.group == G and (lin.out_features, lin.in_features) == (N, K)
    q, s = O.gptq_unpack(qweight, scales)
    assert torch.equal(lin.q.cpu(), _repack_host(q)) and torch.equal(lin.s.cpu(), s)  # the oracle's bytes, re-ordered for the kernel
    if E:
        lin.set_extra(extra.to(dev))
    y = lin(x.to(dev)).cpu()
    assert y.shape == (M, N + E)
    exact = O.int4_linear(x, q, s, G, extra, exact=True)
    err = (y.double() - exact).abs()
    tol = exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-13
    print(f"w4 {M}x{N}x{K} g{G}: max abs err {err.max():.3e} at |ref| max {exact.abs().max():.3e}")
    assert bool((err <= tol).all())
    ref = O.int4_linear(x, q, s, G, extra)
    assert (y != ref).float().mean().item() < 0.05


def test_w4_rows_do_not_depend_on_M(dev):
    from spinf_serve_b200 import ops

    qweight, scales = _gptq(512, 1024, 128, 3)
    q, s = O.gptq_unpack(qweight, scales)
    q, s = ops.w4_repack(q.to(dev)), s.to(dev)
    x = torch.randn((1000, 1024), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(dev)
    full = ops.w4_gemm(x, q, s, 128)
    for M in (1, 36, 64, 65, 255, 256, 257):  # up to 64 rows run on the 64-token tile, more on the 256-token one
        assert torch.equal(ops.w4_gemm(x[:M].contiguous(), q, s, 128), full[:M])


@pytest.mark.parametrize("G", [32, 64, 128])
def test_w4_expansion_is_the_reference_dequantisation_bit_for_bit(dev, G):
    """x = identity reads the expanded weight back through the GEMM: every element equals dq_bf16's (nibble - 8) * scale rounded once
    to bf16, for all 16 nibble values under scales that use all 11 significant bits of half precision (and subnormal ones)"""
    from spinf_serve_b200 import ops

    N, K = 512, 256
    g = torch.Generator().manual_seed(7)
    qweight, _ = _gptq(N, K, G, 9)
    scales = torch.randint(1, 0x7BFF, (K // G, N), generator=g, dtype=torch.int16).view(torch.float16)  # every positive finite pattern
    scales[0, :8] = torch.tensor([6e-8, 1e-7, 5.96e-8, 6.1e-5, 1.0, 0.333, 65504.0, 3e-5]).to(torch.float16)
    q, s = O.gptq_unpack(qweight, scales)
    y = ops.w4_gemm(torch.eye(K, dtype=torch.bfloat16, device=dev), ops.w4_repack(q.to(dev)), s.to(dev), G).cpu()
    want = O.dq_bf16(q, s, G).t()
    assert torch.equal(y.view(torch.int16), want.contiguous().view(torch.int16))


@pytest.mark.parametrize("M,F,K,G,act", [(300, 384, 512, 128, "silu"), (77, 104, 192, 64, "silu"), (513, 1024, 1024, 32, "gelu_tanh"), (1, 64, 128, 128, "silu"),
                                             (36, 640, 1024, 128, "silu"), (64, 104, 192, 64, "gelu_tanh")])
def test_w4_glu_epilogue_equals_the_separate_pass(dev, M, F, K, G, act):
    """the fused gate|up projection with the gated activation in its epilogue gives the bits of the plain projection followed by
    the gated-activation pass (ragged M, F not a multiple of the tile, both activations)"""
    from spinf_serve_b200 import ops
    from spinf_serve_b200.linears import Int4Linear

    qweight, scales = _gptq(2 * F, K, G, 11)
    x = torch.randn((M, K), generator=torch.Generator().manual_seed(12)).to(torch.bfloat16).to(dev)
    plain = Int4Linear(qweight.to(dev), scales.to(dev))
    _, _, want = ops.glu_quant(plain(x), act, want_fp8=False, want_y=True)
    fused = Int4Linear(qweight.to(dev), scales.to(dev)).fuse_glu(act)
    got = fused(x)
    assert got.shape == (M, F) and torch.equal(got, want)
    with pytest.raises(RuntimeError):
        fused.fuse_glu(act)


@pytest.mark.parametrize("M,N,K,G,E", [(36, 5120, 4096, 128, 0), (36, 5120, 17408, 128, 0), (120, 1024, 5120, 32, 64), (1, 256, 128, 128, 0),
                                       (200, 6144, 2048, 64, 0), (36, 34816, 5120, 128, 0), (36, 2048, 5120, 128, 96)])
def test_w4_few_rows_with_k_slices(dev, M, N, K, G, E):
    """Int4Linear.few (a decoding step): the kernel with K cut into slices for narrow projections, exact against the float64
    product to bf16 rounding and within one bf16 step of forward on a few elements (wide ones run forward's kernel: equal)"""
    from spinf_serve_b200 import ops
    from spinf_serve_b200.linears import Int4Linear

    qweight, scales = _gptq(N, K, G, 5)
    g = torch.Generator().manual_seed(6)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    extra = (torch.randn((E, K), generator=g) * 0.05).to(torch.bfloat16) if E else None
    lin = Int4Linear(qweight.to(dev), scales.to(dev))
    if E:
        lin.set_extra(extra.to(dev))
    big, few = lin(x.to(dev)), lin.few(x.to(dev))
    q, s = O.gptq_unpack(qweight, scales)
    exact = O.int4_linear(x, q, s, G, extra, exact=True)
    err = (few.cpu().double() - exact).abs()
    assert bool((err <= exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-13).all())
    d = (few.float() - big.float()).abs()
    sliced = int(ops._lib.lib().spinf_w4_gemm_small_workspace_bytes(M, N, K)) > 0
    print(f"w4 few {M}x{N}x{K}: K slices {'yes' if sliced else 'no'}, {(d > 0).float().mean().item():.4%} of elements differ from forward")
    # sums that cancel to near zero move by more than one of their own bf16 steps: the bound is in steps of the row's scale
    assert (d > 0).float().mean().item() < 0.01 and bool((d <= big.float().abs() * 2.0**-7 + big.float().abs().max() * 2.0**-12).all())
    if not sliced:
        assert torch.equal(few, big)
    assert torch.equal(lin.few(x.to(dev)), few)  # run-to-run determinism
