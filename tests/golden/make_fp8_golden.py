"""Writes tests/golden/fp8_tensor_golden.npz: inputs and outputs of the reference's own per-tensor fp8 and int8 linears run on the CPU.

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_fp8_golden.py <path of the reference checkout>

Fp8Linear and Fp8StaticLinear (spinf_serve/quant/linears.py:66-116) are built by the reference's quant_linears and called as the
reference calls them; torch._scaled_mm with per-tensor scales has a CPU kernel, so nothing is restated. TORCHDYNAMO_DISABLE makes
the reference's torch.compile decorators run their functions eagerly (the arithmetic is the same ops). The static scale comes from
the reference's calibration rule restated in one line (quant/calibrate.py:176-177; its main() needs a model and a GPU).
Int8Linear (linears.py:40-64) in both modes: torch._int_mm has a CPU kernel (the reference pads to 17 rows itself).
Row-wise scheme (the benchmark's): Fp8RowLinear's constructor (linears.py:85-91: w8t, ws) and the reference's quant_act_row
(linears.py:29-33, taken from the closure of Fp8RowLinear.forward) run eagerly on the CPU and are recorded; only the row-wise
torch._scaled_mm of its forward has no CPU kernel, so no row-wise output is recorded (it is compared on the GPU instead)."""

import math
import os
import sys

import numpy as np
import torch


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root):
    sys.path.insert(0, ref_root)
    from spinf_serve.quant import linears as RL

    ns = RL.quant_linears(None, "cpu")
    out = {}
    cases = [(24, 64, 32, 0.02, 1.0), (33, 128, 48, 0.05, 3.0), (7, 256, 16, 0.02, 40.0)]  # (M, K, N, weight std, input std)
    for i, (M, K, N, wstd, xstd) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        w = (torch.randn((N, K), generator=g) * wstd).to(torch.bfloat16)
        x = (torch.randn((M, K), generator=g) * xstd).to(torch.bfloat16)
        x[0, 0] = 3.0 * xstd * 4  # one outlier sets the dynamic scale
        amax = float(x.float().abs().max())
        # the static scale: headroom 2 over a "calibration" maximum that case 2 exceeds (its inputs clip)
        xs = 2.0 ** math.ceil(math.log2(max(amax if i != 2 else amax / 8, 1e-6) * 2.0 / 448.0))
        dyn = ns.Fp8Linear(w)
        sta = ns.Fp8StaticLinear(w, xs)
        RL.MONITOR["on"] = True
        y_dyn = dyn(x)
        y_sta = sta(x)
        RL.MONITOR["on"] = False
        out[f"w{i}"], out[f"x{i}"] = bits(w), bits(x)
        out[f"w8_{i}"] = dyn.w8t.t().contiguous().view(torch.uint8).numpy()
        out[f"ws{i}"] = dyn.ws.numpy().reshape(1)
        out[f"xs{i}"] = np.float32(xs).reshape(1)
        out[f"y_dyn{i}"], out[f"y_sta{i}"] = bits(y_dyn), bits(y_sta)
        out[f"peak{i}"] = sta.peak.numpy().reshape(1)
        row = ns.Fp8RowLinear(w)
        fwd = type(row).forward
        quant_act_row = fwd.__closure__[fwd.__code__.co_freevars.index("quant_act_row")].cell_contents
        x8r, xsr = quant_act_row(x)
        out[f"row_w8_{i}"] = row.w8t.t().contiguous().view(torch.uint8).numpy()
        out[f"row_ws{i}"] = row.ws.numpy()
        out[f"row_x8_{i}"] = x8r.contiguous().view(torch.uint8).numpy()
        out[f"row_xs{i}"] = xsr.numpy()
        i8a, i8w = ns.Int8Linear(w, True), ns.Int8Linear(w, False)
        out[f"i8_w8_{i}"] = i8a.w8t.t().contiguous().numpy()
        out[f"i8_ws{i}"] = i8a.ws.numpy()
        out[f"y_i8a{i}"], out[f"y_i8w{i}"] = bits(i8a(x)), bits(i8w(x))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "fp8_tensor_golden.npz"), **out)
    print("cases", len(cases), "peaks", [float(out[f"peak{i}"][0]) for i in range(len(cases))])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
