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
    assert torch.equal(lin.q.cpu(), q) and torch.equal(lin.s.cpu(), s)
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
    q, s = q.to(dev), s.to(dev)
    x = torch.randn((1000, 1024), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(dev)
    full = ops.w4_gemm(x, q, s, 128)
    for M in (1, 255, 256, 257):
        assert torch.equal(ops.w4_gemm(x[:M].contiguous(), q, s, 128), full[:M])
