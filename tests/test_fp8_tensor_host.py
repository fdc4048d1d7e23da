"""The oracle's per-tensor fp8 linears (dynamic and static) against outputs of the reference's own Fp8Linear / Fp8StaticLinear run on
the CPU (tests/golden/fp8_tensor_golden.npz, written by tests/golden/make_fp8_golden.py)."""

import os

import numpy as np
import torch

from oracle import linears as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "fp8_tensor_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def test_weight_quantiser_is_the_reference_s():
    for i in range(3):
        w8, ws = O.quantize_weight(bf16(G[f"w{i}"]))
        assert np.array_equal(w8.view(torch.uint8).numpy(), G[f"w8_{i}"])
        assert float(ws) == float(G[f"ws{i}"][0])


def test_linears_match_the_reference_outputs():
    for i in range(3):
        w, x = bf16(G[f"w{i}"]), bf16(G[f"x{i}"])
        w8, ws = O.quantize_weight(w)
        xs = float(G[f"xs{i}"][0])
        y_dyn = O.fp8_linear(x, w8, ws)
        y_sta, peak = O.fp8_static_linear(x, w8, ws, xs)
        for mine, ref in ((y_dyn, bf16(G[f"y_dyn{i}"])), (y_sta, bf16(G[f"y_sta{i}"]))):
            # the same e4m3 operands and scales; only the fp32 summation order inside the matmul may differ: at most one bf16
            # step on a few elements
            d = (mine.float() - ref.float()).abs()
            tol = ref.float().abs() * 2.0**-7 + 1e-30
            assert bool((d <= tol).all())
            assert (mine != ref).float().mean().item() < 0.02
        assert float(peak) == float(G[f"peak{i}"][0])
    assert float(G["peak2"][0]) > 1.0  # case 2 clips: its inputs pass 448 x scale


def test_static_scale_rule():
    assert O.static_scale(448.0, 2.0) == 2.0
    assert O.static_scale(100.0, 2.0) == 0.5
    assert O.static_scale(0.0, 2.0) == 2.0 ** -27
    for i in range(2):  # the generator applied the same rule with headroom 2 to the tensor's own maximum
        amax = float(bf16(G[f"x{i}"]).float().abs().max())
        assert O.static_scale(amax, 2.0) == float(G[f"xs{i}"][0])


def test_product_side_host_logic():
    """the product's copy of the scale rule, the scheme names, and the classes' refusal of a CPU device (no CPU fallback)"""
    import pytest

    from spinf_serve_b200 import gemma_stack as GS
    from spinf_serve_b200 import linears

    for amax in (0.0, 1e-3, 0.7, 100.0, 448.0, 449.0, 3.0e4):
        assert linears.static_scale(amax, 2.0) == O.static_scale(amax, 2.0)
        assert linears.static_scale(amax, 1.0) == O.static_scale(amax, 1.0)
    assert GS.SCHEMES == ("fp8row", "fp8", "fp8s", "w8a8", "w8a16", "bf16") and GS.LINEARS == ("q", "k", "v", "o", "gate", "up", "down")
    ns = linears.quant_linears(None, "cpu")
    w = torch.zeros((16, 16), dtype=torch.bfloat16)
    for make in (lambda: ns.Fp8Linear(w), lambda: ns.Fp8StaticLinear(w, 0.5), lambda: ns.Fp8RowLinear(w), lambda: ns.Int8Linear(w, True)):
        with pytest.raises(RuntimeError):
            make()
    with pytest.raises(RuntimeError):
        GS.GemmaWeights(GS.GemmaConfig(layers=0), None, None, [], scheme="int8")


def test_int8_linear_matches_the_reference_outputs():
    """the oracle's Int8Linear (both modes) against the reference's own module run on the CPU: integer accumulation is exact, so
    the w8a8 outputs are the same bits; the w8a16 mode is a bf16 matmul (summation order may move a last bit)"""
    for i in range(3):
        w, x = bf16(G[f"w{i}"]), bf16(G[f"x{i}"])
        w8, ws = O.quantize_weight_int8(w)
        assert np.array_equal(w8.numpy(), G[f"i8_w8_{i}"]) and np.array_equal(ws.numpy(), G[f"i8_ws{i}"])
        assert torch.equal(O.int8_linear(x, w8, ws, True), bf16(G[f"y_i8a{i}"]))
        mine, ref = O.int8_linear(x, w8, ws, False), bf16(G[f"y_i8w{i}"])
        assert bool(((mine.float() - ref.float()).abs() <= ref.float().abs() * 2.0**-7 + 1e-30).all())


def test_rowwise_quantisers_are_the_reference_s():
    """the benchmark's scheme: the oracle's weight and activation quantisers against Fp8RowLinear's buffers and the reference's
    quant_act_row run on the CPU (bit for bit: bytes and fp32 scales)"""
    for i in range(3):
        w, x = bf16(G[f"w{i}"]), bf16(G[f"x{i}"])
        w8, ws = O.quantize_weight_rowwise(w)
        assert np.array_equal(w8.view(torch.uint8).numpy(), G[f"row_w8_{i}"]) and np.array_equal(ws.numpy(), G[f"row_ws{i}"])
        x8, xs = O.quant_act_row(x)
        assert np.array_equal(x8.view(torch.uint8).numpy(), G[f"row_x8_{i}"]) and np.array_equal(xs.numpy(), G[f"row_xs{i}"])
