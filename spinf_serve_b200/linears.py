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


def gptq_unpack(qweight, scales):
    """GPTQ v1 storage -> the engine layout, at load time with the reference's eager torch ops (Int4Linear.__init__,
    spinf_serve/models/qwen35/qwen.py:383-391): qweight int32 [K/8, N] (8 nibbles per word, shifts 0..28) -> q uint8 [N, K/2] with the
    low nibble = even k; scales fp16 [K/G, N] -> [N, K/G]"""
    sh = torch.arange(0, 32, 4, dtype=torch.int32, device=qweight.device)
    q = ((qweight[:, None, :] >> sh[None, :, None]) & 15).reshape(-1, qweight.shape[1]).t()
    return (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous(), scales.t().contiguous()


class Int4Linear(nn.Module):
    """GPTQ int4 symmetric weights, bf16 activations, dequantised inside the GEMM kernel (the reference's Int4Linear in bf16 mode,
    qwen.py:378-458): same constructor arguments, buffers q / s / extra, set_extra and forward. The group size is inferred from
    the scales' shape (the reference reads it from the checkpoint's quantization_config, qwen.py:301)."""

    def __init__(self, qweight, scales):
        super().__init__()
        if not qweight.is_cuda:
            raise RuntimeError("Int4Linear needs a CUDA device with sm_100a kernels; there is no CPU path")
        q, s = gptq_unpack(qweight, scales)
        self.out_features, self.in_features = q.shape[0], q.shape[1] * 2
        self.group = self.in_features // s.shape[1]
        self.register_buffer("q", q)
        self.register_buffer("s", s.to(torch.float16))
        self.extra = None
        self.name = ""

    def set_extra(self, w):
        """bf16 rows [E, in] appended to the output (the Gated DeltaNet's b / a projections)"""
        del self.extra
        self.register_buffer("extra", w.to(torch.bfloat16).contiguous())

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        y = ops.w4_gemm(x2 if x2.is_contiguous() else x2.contiguous(), self.q, self.s, self.group, self.extra)
        return y.reshape(*x.shape[:-1], y.shape[-1])
