"""Quantized linear modules with the reference's interface (spinf_serve/quant/linears.py:17-19,133-135): quant_linears(opts, device)
returns a namespace of module classes built from a bf16 [out, in] weight on the device, exposing in_features / out_features and
forward(x[..., K]) -> [..., N] bf16, with the same buffers (`w8t` = the [in, out] column-major view, `ws` [1, out]).

Fp8RowLinear (per-output-channel weight scales, per-token activation scales: the scheme of the BASELINE configurations) runs on
the sm_100a kernels. The other schemes of the reference (dynamic / static per-tensor fp8, int8) are outside this path: their names
resolve, constructing one raises RuntimeError, as the reference does for a scheme the device cannot run (gemma4.py:61-62)."""

from types import SimpleNamespace

import torch
import torch.nn as nn

from spinf_serve_b200 import ops

FP8_MAX = 448.0  # the largest finite e4m3 value (spinf_serve/quant/fp8.py:11)


def quantize_weight_rowwise(w):
    """bf16 [out, in] on the device -> (w8 [out, in] e4m3, ws [1, out] fp32): load-time arithmetic of Fp8RowLinear.__init__
    (spinf_serve/quant/linears.py:85-91), run with the same eager torch ops on the same device as the reference runs them"""
    wf = w.float()
    s = wf.abs().amax(-1, keepdim=True).clamp(min=1e-12) / FP8_MAX
    return (wf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s.t().contiguous()


def quant_linears(opts: dict | None, device) -> SimpleNamespace:
    """opts (the reference's inductor options) is accepted and unused: nothing here is compiled"""

    class Fp8RowLinear(nn.Module):
        def __init__(self, w):  # w: bf16 [out, in] on device
            super().__init__()
            if not w.is_cuda:
                raise RuntimeError("Fp8RowLinear needs a CUDA device with sm_100a kernels; there is no CPU path")
            w8, ws = quantize_weight_rowwise(w)
            self.register_buffer("w8t", w8.t())  # [in, out] column-major view of the [out, in] storage
            self.register_buffer("ws", ws)  # [1, out]
            self.out_features, self.in_features = w.shape

        def forward(self, x):
            x8, xs = ops.fp8_rowwise_quant(x if x.is_contiguous() else x.contiguous())
            y = ops.fp8_rowwise_gemm(x8, xs, self.w8t.t(), self.ws)
            return y.reshape(*x.shape[:-1], self.out_features)

    def _outside(name):
        class Unsupported(nn.Module):
            def __init__(self, *a, **k):
                raise RuntimeError(f"quant scheme {name} is outside the packed scoring path of this build (use fp8row)")

        Unsupported.__name__ = name
        return Unsupported

    def prequantized(cls, w8, ws, xs=None):
        raise RuntimeError("fp8-static checkpoints are outside the packed scoring path of this build (use fp8row)")

    return SimpleNamespace(
        Int8Linear=_outside("Int8Linear"), Fp8Linear=_outside("Fp8Linear"), Fp8RowLinear=Fp8RowLinear,
        Fp8StaticLinear=_outside("Fp8StaticLinear"), prequantized=prequantized,
    )
