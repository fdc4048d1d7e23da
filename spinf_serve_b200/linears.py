"""Quantized linear modules with the reference's interface (spinf_serve/quant/linears.py:17-19,133-135): quant_linears(opts, device)
returns a namespace of module classes built from a bf16 [out, in] weight on the device, exposing in_features / out_features and
forward(x[..., K]) -> [..., N] bf16, with the same buffers (`w8t` = the [in, out] column-major view, `ws`, and for the static
scheme `xs` and `peak`).

On the sm_100a kernels: Fp8RowLinear (per-output-channel weight scales, per-token activation scales: the scheme of the benchmark
configurations), Fp8Linear (per-tensor scales, the activation scale from the forward's own maximum) and Fp8StaticLinear
(per-tensor scales, a calibrated fixed activation scale: the reference's "fp8s"), `prequantized` for the tensors of an
fp8-static checkpoint, and Int8Linear (int8 weights; int8 per-token activations on the int8 tensor cores, or bf16 activations).
Constructing any of them on a device without the kernels raises RuntimeError, as the reference does for a scheme the device
cannot run (gemma4.py:61-62): there is no CPU path."""

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


def quantize_weight(w):
    """bf16 [out, in] on the device -> (w8 [out, in] e4m3, fp32 scale []), one scale for the tensor: load-time arithmetic of
    Fp8Linear / Fp8StaticLinear (spinf_serve/quant/linears.py:69-71, quant/fp8.py:14-21), same eager torch ops"""
    wf = w.float()
    s = wf.abs().amax().clamp(min=1e-12) / FP8_MAX
    return (wf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s.reshape(())


def static_scale(amax: float, headroom: float = 2.0) -> float:
    """the calibrated activation scale of a linear whose largest input seen was `amax`: a power of two (exact in the kernel) at
    least `headroom` times amax / 448 (spinf_serve/quant/calibrate.py:176-177)"""
    import math

    return 2.0 ** math.ceil(math.log2(max(amax, 1e-6) * headroom / FP8_MAX))


# fp8s: a caller turns this on for sampled forwards; the peak check costs one block reduction per linear (linears.py:13-14)
MONITOR = {"on": False}


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

    class Fp8Linear(nn.Module):
        """per-tensor scales both sides, the activation scale from this forward's maximum (linears.py:66-78): rows depend on
        their neighbours in the stream through that maximum, as in the reference"""

        def __init__(self, w):  # w: bf16 [out, in] on device
            super().__init__()
            if not w.is_cuda:
                raise RuntimeError("Fp8Linear needs a CUDA device with sm_100a kernels; there is no CPU path")
            w8, ws = quantize_weight(w)
            self.register_buffer("w8t", w8.t())
            self.register_buffer("ws", ws)
            self.out_features, self.in_features = w.shape

        def forward(self, x):
            x8, xs = ops.fp8_tensor_quant(x if x.is_contiguous() else x.contiguous())
            y = ops.fp8_tensor_gemm(x8, xs, self.w8t.t(), self.ws)
            return y.reshape(*x.shape[:-1], self.out_features)

    class Fp8StaticLinear(nn.Module):
        """fp8 with a fixed activation scale (linears.py:98-116). `peak` keeps the largest |input| / (448 * scale) seen while
        MONITOR["on"]: above 1 the input was clipped"""

        def __init__(self, w, xs: float):  # w: bf16 [out, in] on device
            super().__init__()
            if not w.is_cuda:
                raise RuntimeError("Fp8StaticLinear needs a CUDA device with sm_100a kernels; there is no CPU path")
            w8, ws = quantize_weight(w)
            self.register_buffer("w8t", w8.t())
            self.register_buffer("ws", ws)
            self.register_buffer("xs", torch.tensor(xs, dtype=torch.float32, device=w.device))
            self.register_buffer("peak", torch.zeros((), dtype=torch.float32, device=w.device))
            self.out_features, self.in_features = w.shape

        def forward(self, x):
            x8, _ = ops.fp8_tensor_quant(x if x.is_contiguous() else x.contiguous(), self.xs, self.peak if MONITOR["on"] else None)
            y = ops.fp8_tensor_gemm(x8, self.xs, self.w8t.t(), self.ws)
            return y.reshape(*x.shape[:-1], self.out_features)

    class Int8Linear(nn.Module):
        """int8 weights with per-output-channel scales; act8: int8 per-token activations on the int8 tensor cores (w8a8), else
        bf16 activations against the weight dequantised to bf16 (w8a16) (linears.py:40-64). Load-time arithmetic with the
        reference's eager torch ops."""

        def __init__(self, w, act8):
            super().__init__()
            if not w.is_cuda:
                raise RuntimeError("Int8Linear needs a CUDA device with sm_100a kernels; there is no CPU path")
            wf = w.float()
            s = wf.abs().amax(-1).clamp(min=1e-12) / 127.0
            w8 = (wf / s[:, None]).round_().clamp_(-127, 127).to(torch.int8)
            if act8:
                self.register_buffer("w8t", w8.t())  # [in, out] column-major view of the [out, in] storage
                self.register_buffer("ws", s)  # [out] fp32
            else:
                self.register_buffer("w8", w8)  # [out, in]
                self.register_buffer("ws", s.to(torch.bfloat16)[:, None])  # [out, 1]
            self.act8 = act8
            self.out_features, self.in_features = w.shape

        def forward(self, x):
            x2 = x.reshape(-1, x.shape[-1])
            x2 = x2 if x2.is_contiguous() else x2.contiguous()
            if self.act8:
                x8, xs = ops.int8_rowwise_quant(x2)
                y = ops.int8_rowwise_gemm(x8, xs, self.w8t.t(), self.ws)
            else:  # the scale folded into the weight, one bf16 rounding per element, as the reference folds it on every call
                y = ops.bf16_gemm(x2, self.w8.to(torch.bfloat16) * self.ws)
            return y.reshape(*x.shape[:-1], self.out_features)

    def prequantized(cls, w8, ws, xs=None):
        """Fp8StaticLinear / Fp8Linear from an fp8-static checkpoint's tensors: w8 e4m3 [out, in], ws fp32 [1], xs fp32 [1]
        (linears.py:121-131)"""
        if cls not in (Fp8Linear, Fp8StaticLinear):
            raise RuntimeError(f"prequantized: {cls.__name__} is not a per-tensor fp8 linear")
        lin = cls.__new__(cls)
        nn.Module.__init__(lin)
        lin.register_buffer("w8t", w8.to(device, non_blocking=True).contiguous().t())
        lin.register_buffer("ws", ws.to(device, torch.float32).reshape(()))
        if xs is not None:
            lin.register_buffer("xs", xs.to(device, torch.float32).reshape(()))
            lin.register_buffer("peak", torch.zeros((), dtype=torch.float32, device=device))
        lin.out_features, lin.in_features = w8.shape
        return lin

    return SimpleNamespace(
        Int8Linear=Int8Linear, Fp8Linear=Fp8Linear, Fp8RowLinear=Fp8RowLinear, Fp8StaticLinear=Fp8StaticLinear,
        prequantized=prequantized,
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
        self.register_buffer("q", ops.w4_repack(q))  # the reference's bytes, nibbles re-ordered inside each 8-k word for the kernel
        self.register_buffer("s", s.to(torch.float16))
        self.extra = None
        self.glu = None
        self.name = ""

    def fuse_glu(self, act: str):
        """for a fused gate|up projection (gate channels first, then up): from now on forward returns act(gate) * up [.., out/2],
        computed in the GEMM's epilogue. The rows are interleaved once, here (gate c, up c, gate c + 1, ...), which is the order the
        kernel's lane pairs read them in; the values are those of forward followed by the gated-activation pass."""
        if self.extra is not None or self.glu is not None or self.out_features % 16:
            raise RuntimeError("fuse_glu: a plain fused gate|up projection with an output width that is a multiple of 16")
        F = self.out_features // 2
        order = torch.stack((torch.arange(F), torch.arange(F) + F), dim=1).reshape(-1).to(self.q.device)
        self.q, self.s = self.q[order].contiguous(), self.s[order].contiguous()
        self.glu = act
        return self

    def set_extra(self, w):
        """bf16 rows [E, in] appended to the output (the Gated DeltaNet's b / a projections)"""
        del self.extra
        self.register_buffer("extra", w.to(torch.bfloat16).contiguous())

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        if self.glu is not None:
            y = ops.w4_gemm_glu(x2 if x2.is_contiguous() else x2.contiguous(), self.q, self.s, self.group, self.glu)
            return y.reshape(*x.shape[:-1], y.shape[-1])
        y = ops.w4_gemm(x2 if x2.is_contiguous() else x2.contiguous(), self.q, self.s, self.group, self.extra)
        return y.reshape(*x.shape[:-1], y.shape[-1])

    def few(self, x):
        """forward for a decoding step's few rows (at most 256): narrow projections run the kernel with its K dimension cut into
        slices so that every SM streams weights (the last bf16 bit may differ from forward's); gated projections as forward"""
        if self.glu is not None:
            return self.forward(x)
        x2 = x.reshape(-1, x.shape[-1])
        y = ops.w4_gemm_small(x2 if x2.is_contiguous() else x2.contiguous(), self.q, self.s, self.group, self.extra)
        return y.reshape(*x.shape[:-1], y.shape[-1])
