"""GPU parity of the per-tensor fp8 linears (through the C ABI): Fp8Linear (dynamic) and Fp8StaticLinear (calibrated static scale,
with its clipping monitor) of spinf_serve/quant/linears.py:66-131, against the reference's own CPU outputs (golden) and the oracle."""

import os

import numpy as np
import pytest
import torch

from oracle import linears as O

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "fp8_tensor_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,K", [(1, 64), (7, 3840), (300, 15360), (1001, 5376)])
def test_tensor_quant_bit_exact(dev, M, K):
    """dynamic and static quantisation equal the oracle's bit for bit; the static monitor equals max|x| / (448 s)"""
    from spinf_serve_b200 import ops

    x = _rand((M, K), 1, 3.0)
    x[0, :8] = 0
    x[0, 8:16] = -0.0
    x8, s = ops.fp8_tensor_quant(x.to(dev))
    r8, rs = O.quant_act(x)
    assert float(s) == float(rs)
    assert torch.equal(x8.cpu().view(torch.uint8), r8.view(torch.uint8))
    for xs in (2.0**-6, 2.0**-9, 0.013):  # covers everything; clips most of it; not a power of two
        scale = torch.tensor(xs, dtype=torch.float32, device=dev)
        peak = torch.zeros((), dtype=torch.float32, device=dev)
        x8, s2 = ops.fp8_tensor_quant(x.to(dev), scale, peak)
        assert s2 is scale
        assert torch.equal(x8.cpu().view(torch.uint8), O.quant_act_static(x, torch.tensor(xs)).view(torch.uint8))
        assert float(peak) == float(x.float().abs().amax() / (torch.tensor(xs) * 448.0))
        ops.fp8_tensor_quant((x * 0.5).to(dev), scale, peak)  # a smaller input leaves the monitor where it was
        assert float(peak) == float(x.float().abs().amax() / (torch.tensor(xs) * 448.0))
    z8, zs = ops.fp8_tensor_quant(torch.zeros((4, 64), dtype=torch.bfloat16, device=dev))  # an all-zero tensor: the scale clamps
    assert float(zs) == float(torch.tensor(1e-12) / 448.0) and int(z8.view(torch.uint8).max()) == 0


def test_linears_match_the_reference_outputs(dev):
    """the modules, built as the reference builds them, against the reference's own Fp8Linear / Fp8StaticLinear outputs"""
    from spinf_serve_b200 import linears

    ns = linears.quant_linears(None, dev)
    for i in range(3):
        w, x = bf16(G[f"w{i}"]), bf16(G[f"x{i}"])
        xs = float(G[f"xs{i}"][0])
        # the constructors run the reference's load-time torch ops on the device, where dividing by a scalar multiplies by its
        # reciprocal: the scale may differ from the CPU's in its last bit (and a few weights by one fp8 step with it)
        built = ns.Fp8StaticLinear(w.to(dev), xs)
        assert abs(float(built.ws) - float(G[f"ws{i}"][0])) <= float(G[f"ws{i}"][0]) * 2.0**-22 and float(built.xs) == xs
        assert (built.w8t.t().contiguous().view(torch.uint8).cpu() != torch.from_numpy(G[f"w8_{i}"])).float().mean() < 0.01
        # the forward is compared on the reference's own quantized tensors (what an fp8-static checkpoint holds)
        w8g, wsg = torch.from_numpy(G[f"w8_{i}"]).view(torch.float8_e4m3fn), torch.from_numpy(G[f"ws{i}"])
        dyn, sta = ns.prequantized(ns.Fp8Linear, w8g, wsg), ns.prequantized(ns.Fp8StaticLinear, w8g, wsg, torch.from_numpy(G[f"xs{i}"]))
        assert float(dyn.ws) == float(G[f"ws{i}"][0]) and float(sta.xs) == xs and not hasattr(dyn, "xs")
        linears.MONITOR["on"] = True
        try:
            y_sta = sta(x.to(dev)).cpu()
        finally:
            linears.MONITOR["on"] = False
        y_dyn = dyn(x.to(dev)).cpu()
        for mine, ref in ((y_dyn, bf16(G[f"y_dyn{i}"])), (y_sta, bf16(G[f"y_sta{i}"]))):
            d = (mine.float() - ref.float()).abs()
            assert bool((d <= ref.float().abs() * 2.0**-7 + 1e-30).all())  # one bf16 step at most (fp32 summation order)
            assert (mine != ref).float().mean().item() < 0.02
        assert float(sta.peak) == float(G[f"peak{i}"][0])


@pytest.mark.parametrize("M,N,K", [(130, 512, 384), (640, 3840, 4096), (200, 3840, 15360)])
def test_tensor_gemm_vs_oracle(dev, M, N, K):
    from spinf_serve_b200 import ops

    x, w = _rand((M, K), 2), _rand((N, K), 3, 0.02)
    w8, ws = O.quantize_weight(w)
    x8, xs = O.quant_act(x)
    y = ops.fp8_tensor_gemm(x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev)).cpu()
    exact = O.scaled_mm_tensor(x8, xs, w8, ws, exact=True)
    err = (y.double() - exact).abs()
    assert bool((err <= exact.abs() * 2.0**-7 + exact.abs().max() * 2.0**-14).all())
    assert (y != O.scaled_mm_tensor(x8, xs, w8, ws)).float().mean().item() < 0.05


def test_static_rows_do_not_depend_on_the_stream(dev):
    """the point of the static scheme (a job's scores do not depend on its neighbours): a row's output is the same bits whatever
    else is in the call, while the dynamic scheme's rows move with the stream's maximum"""
    from spinf_serve_b200 import linears

    ns = linears.quant_linears(None, dev)
    w = _rand((768, 1024), 5, 0.02).to(dev)
    x = _rand((700, 1024), 6).to(dev)
    x[650, 3] = 60.0  # a neighbour with an outlier
    sta = ns.Fp8StaticLinear(w, linears.static_scale(64.0))
    full = sta(x)
    for M in (1, 129, 300):
        assert torch.equal(sta(x[:M].contiguous()), full[:M])
    dyn = ns.Fp8Linear(w)
    assert not torch.equal(dyn(x[:300].contiguous()), dyn(x)[:300])


@pytest.mark.parametrize("M,K", [(1, 64), (7, 3840), (300, 15360)])
def test_int8_quant_bit_exact(dev, M, K):
    from spinf_serve_b200 import ops

    x = _rand((M, K), 1, 3.0)
    x[0, :8] = 0
    if M > 2:
        x[2] = 0  # an all-zero row: the scale clamps at 1e-12 / 127
    x8, xs = ops.int8_rowwise_quant(x.to(dev))
    r8, rs = O.quant_act_int8(x)
    assert torch.equal(xs.cpu(), rs) and torch.equal(x8.cpu(), r8)


def test_int8_linear_matches_the_reference_outputs(dev):
    """Int8Linear on the int8 tensor cores against the reference's own module outputs (CPU run): the integer product is exact and
    the scaling is the same two fp32 multiplications, so the w8a8 outputs are the same bits"""
    from spinf_serve_b200 import linears, ops

    ns = linears.quant_linears(None, dev)
    for i in range(3):
        w, x = bf16(G[f"w{i}"]), bf16(G[f"x{i}"])
        w8, ws = torch.from_numpy(G[f"i8_w8_{i}"]), torch.from_numpy(G[f"i8_ws{i}"])
        x8, xs = ops.int8_rowwise_quant(x.to(dev))
        y = ops.int8_rowwise_gemm(x8, xs, w8.to(dev), ws.to(dev)).cpu()
        assert torch.equal(y, bf16(G[f"y_i8a{i}"]))
        a8, a16 = ns.Int8Linear(w.to(dev), True), ns.Int8Linear(w.to(dev), False)
        # the module quantises its weight on the device (the scale's last bit may differ from the CPU's, see above)
        ya, ra = a8(x.to(dev)).cpu().float(), bf16(G[f"y_i8a{i}"]).float()
        # (a weight that moves by one int8 step moves an output by about |x| * scale: an absolute term, not a relative one)
        assert (ya != ra).float().mean().item() < 0.05 and bool(((ya - ra).abs() <= ra.abs() * 2.0**-6 + ra.abs().max() * 2.0**-8).all())
        yw, rw = a16(x.to(dev)).cpu().float(), bf16(G[f"y_i8w{i}"]).float()
        assert bool(((yw - rw).abs() <= rw.abs() * 2.0**-6 + rw.abs().max() * 2.0**-12).all())


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (130, 512, 384), (640, 3840, 4096), (200, 3840, 15360)])
def test_int8_gemm_exact(dev, M, N, K):
    """every output equals the oracle's: int32 accumulation has no summation order (|sum| < 2^31 at these K)"""
    from spinf_serve_b200 import ops

    x, w = _rand((M, K), 2), _rand((N, K), 3, 0.02)
    w8, ws = O.quantize_weight_int8(w)
    x8, xs = O.quant_act_int8(x)
    y = ops.int8_rowwise_gemm(x8.to(dev), xs.to(dev), w8.to(dev), ws.to(dev)).cpu()
    acc = (x8.long() @ w8.long().t()).to(torch.int32)
    assert torch.equal(y, (acc.float() * xs * ws).to(torch.bfloat16))
