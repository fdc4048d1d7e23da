"""Oracle of the quantized linears (CPU torch; test infrastructure only, never imported by the product).

Row-wise fp8 follows spinf_serve/quant/linears.py:29-33 (quant_act_row) and :84-96 (Fp8RowLinear); torch._scaled_mm with row-wise
scales has no CPU kernel, so the product is restated as the fp32 matmul of the e4m3 values times both scales, rounded once to bf16.
The quantiser formula is pinned bit-for-bit by the reference's own test (tests/test_fp8_checkpoint.py:11-23, per-tensor variant).
int4 follows spinf_serve/models/qwen35/qwen.py:383-391 (GPTQ unpack), :326-330 (dq_bf16) and :455-458 (bf16 mode)."""

import torch

FP8_MAX = 448.0  # spinf_serve/quant/fp8.py:11


def quantize_weight_rowwise(w):
    """bf16 [out, in] -> (w8 [out, in] e4m3, ws [1, out] fp32): Fp8RowLinear.__init__, linears.py:85-91"""
    wf = w.float()
    s = wf.abs().amax(-1, keepdim=True).clamp(min=1e-12) / FP8_MAX
    return (wf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s.t().contiguous()


def quant_act_row(x):
    """[..., K] -> (x8 [M, K] e4m3, xs [M, 1] fp32): linears.py:29-33"""
    xf = x.reshape(-1, x.shape[-1]).float()
    s = xf.abs().amax(-1, keepdim=True).clamp_(min=1e-12) / FP8_MAX
    return (xf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s


def scaled_mm_rowwise(x8, xs, w8, ws, exact=False):
    """bf16((x8 @ w8^T) * xs * ws): the row-wise torch._scaled_mm of linears.py:95. exact=True accumulates in float64 (the exact
    product of the quantized operands, used to bound a kernel's error independently of summation order)"""
    if exact:
        acc = x8.double() @ w8.double().t()
        return acc * xs.double().reshape(-1, 1) * ws.double().reshape(1, -1)
    acc = x8.float() @ w8.float().t()
    return (acc * xs.reshape(-1, 1) * ws.reshape(1, -1)).to(torch.bfloat16)


def fp8_row_linear(x, w8, ws):
    """Fp8RowLinear.forward, linears.py:93-96"""
    x8, xs = quant_act_row(x)
    return scaled_mm_rowwise(x8, xs, w8, ws).reshape(*x.shape[:-1], w8.shape[0])


# ------------------------------------------------------------------------------------------------ int4 (GPTQ v1, symmetric)
def gptq_unpack(qweight, scales):
    """qweight int32 [K/8, N] (8 nibbles per word, shifts 0..28), scales fp16 [K/G, N] -> (q uint8 [N, K/2] low nibble = even k,
    s fp16 [N, K/G]): Int4Linear.__init__, qwen.py:383-391"""
    K8, N = qweight.shape
    shifts = torch.arange(0, 32, 4, dtype=torch.int32)
    nib = ((qweight[:, None, :] >> shifts[None, :, None]) & 15).reshape(K8 * 8, N).to(torch.uint8)  # [K, N]
    nt = nib.t().contiguous()  # [N, K]
    q = nt[:, 0::2] | (nt[:, 1::2] << 4)
    return q.contiguous(), scales.t().contiguous()


def dq_bf16(q, s, group):
    """(nibble - 8) * scale in fp32, rounded once to bf16 -> [N, K]: qwen.py:326-330"""
    lo = (q & 15).to(torch.int16) - 8
    hi = (q >> 4).to(torch.int16) - 8
    w = torch.stack((lo, hi), dim=-1).reshape(q.shape[0], -1).float()
    return (w * s.float().repeat_interleave(group, dim=1)).to(torch.bfloat16)


def int4_linear(x, q, s, group, extra=None, exact=False):
    """Int4Linear.forward in bf16 mode, qwen.py:455-458: x @ dq(w)^T with fp32 accumulation, bf16 out; `extra` un-quantised bf16
    rows are appended to the output channels (qwen.py:421-426)"""
    w = dq_bf16(q, s, group)
    if extra is not None:
        w = torch.cat([w, extra.to(torch.bfloat16)], 0)
    if exact:
        return x.double() @ w.double().t()
    return (x.float() @ w.float().t()).to(torch.bfloat16)


def w4_small_splits(N, K, bn=64, bk=256, programs=512):
    """the split-K count of the few-row W4A16 linear (spinf_serve/quant/w4gemm.py:51-56)"""
    n_blocks = -(-N // bn)
    splits = max(1, min(K // bk, programs // n_blocks))
    while (K // bk) % splits:
        splits -= 1
    return splits


def w4_small_linear(x, q, s, group=32, extra=None, exact=False):
    """the W4A16 linear of the decoding steps, spinf_serve/quant/w4gemm.py:17-66: x [M, K] bf16 rounded to fp16; q uint8 [N, K/2]
    (low nibble = even k, value nibble - 8), s fp16 [N, K/group]; the weight (nibble - 8) * scale formed in fp16; fp16 products
    summed in fp32 per K slice, the slices' partial sums added in order, bf16 out. The order of the fp32 additions inside a slice
    is the tensor core's: here they are summed exactly (float64) and rounded to fp32 once, which a kernel meets to the last bit or
    two of the fp32 partial sum. `extra` [E, K] bf16 rows are appended as a plain product (w4gemm.py:63-64)."""
    M, K = x.shape
    N = q.shape[0]
    lo = (q & 15).to(torch.float16) - 8.0
    hi = (q >> 4).to(torch.float16) - 8.0
    w = torch.stack([lo, hi], -1).reshape(N, K)
    w = (w.reshape(N, K // group, group) * s.to(torch.float16)[:, :, None]).reshape(N, K)  # fp16 product, rounded to fp16
    xh = x.to(torch.float16)
    if exact:
        y = xh.double() @ w.double().t()
    else:
        splits = w4_small_splits(N, K)
        k_per = K // splits
        y = torch.zeros((M, N), dtype=torch.float32)
        for sp in range(splits):
            sl = slice(sp * k_per, (sp + 1) * k_per)
            y = y + (xh[:, sl].double() @ w[:, sl].double().t()).float()
        y = y.to(torch.bfloat16)
    if extra is not None:
        e = x.double() @ extra.double().t() if exact else (x.to(extra.dtype) @ extra.t()).to(torch.bfloat16)
        y = torch.cat([y, e], -1)
    return y


# ------------------------------------------------------------------------------------------------ per-tensor fp8 (dynamic and static)
def quantize_weight(w):
    """bf16 [out, in] -> (w8 [out, in] e4m3, fp32 scale []): Fp8Linear / Fp8StaticLinear.__init__, linears.py:69-71,104-106
    (quant/fp8.py:14-21)"""
    wf = w.float()
    s = wf.abs().amax().clamp(min=1e-12) / FP8_MAX
    return (wf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s.reshape(())


def quant_act(x):
    """[..., K] -> (x8 [M, K] e4m3, fp32 scale []), one scale from the tensor's maximum: linears.py:22-26"""
    xf = x.reshape(-1, x.shape[-1]).float()
    s = xf.abs().amax().clamp_(min=1e-12) / FP8_MAX
    return (xf / s).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s


def quant_act_static(x, xs):
    """[..., K] -> x8 [M, K] e4m3 with the fixed scale xs: Fp8StaticLinear.forward, linears.py:110,113"""
    return (x.reshape(-1, x.shape[-1]).float() / xs).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def scaled_mm_tensor(x8, xs, w8, ws, exact=False):
    """bf16((x8 @ w8^T) * xs * ws) with scalar scales: the per-tensor torch._scaled_mm of linears.py:77,114, restated as the fp32
    matmul of the e4m3 values (exact=True: float64, unrounded)"""
    if exact:
        return (x8.double() @ w8.double().t()) * float(xs) * float(ws)
    return ((x8.float() @ w8.float().t()) * xs * ws).to(torch.bfloat16)


def fp8_linear(x, w8, ws):
    """Fp8Linear.forward, linears.py:75-78"""
    x8, xs = quant_act(x)
    return scaled_mm_tensor(x8, xs, w8, ws).reshape(*x.shape[:-1], w8.shape[0])


def fp8_static_linear(x, w8, ws, xs):
    """Fp8StaticLinear.forward, linears.py:108-115 (without the monitor) -> (y, peak contribution max|x| / (xs * 448))"""
    y = scaled_mm_tensor(quant_act_static(x, xs), xs, w8, ws).reshape(*x.shape[:-1], w8.shape[0])
    return y, x.float().abs().amax() / (xs * FP8_MAX)


def static_scale(amax, headroom=2.0):
    """2^ceil(log2(headroom * amax / 448)): quant/calibrate.py:176-177"""
    import math

    return 2.0 ** math.ceil(math.log2(max(amax, 1e-6) * headroom / FP8_MAX))


# ------------------------------------------------------------------------------------------------ int8 (w8a8 and w8a16)
def quantize_weight_int8(w):
    """bf16 [out, in] -> (w8 [out, in] int8, s [out] fp32): Int8Linear.__init__, linears.py:43-46"""
    wf = w.float()
    s = wf.abs().amax(-1).clamp(min=1e-12) / 127.0
    return (wf / s[:, None]).round_().clamp_(-127, 127).to(torch.int8), s


def quant_act_int8(x):
    """[..., K] -> (x8 [M, K] int8, xs [M, 1] fp32): linears.py:34-38"""
    xf = x.reshape(-1, x.shape[-1]).float()
    s = xf.abs().amax(-1, keepdim=True).clamp_(min=1e-12) / 127.0
    return (xf / s).round_().clamp_(-127, 127).to(torch.int8), s


def int8_linear(x, w8, ws, act8=True):
    """Int8Linear.forward, linears.py:55-64. act8: the int32 product (exact; restated as an int64 matmul, torch._int_mm needs CUDA
    or M > 16) converted to fp32 and scaled; else the weight dequantised to bf16 against bf16 activations"""
    x2 = x.reshape(-1, x.shape[-1])
    if act8:
        x8, xs = quant_act_int8(x2)
        acc = (x8.long() @ w8.long().t()).to(torch.int32)
        y = (acc.float() * xs * ws).to(torch.bfloat16)
    else:
        y = torch.nn.functional.linear(x2, w8.to(torch.bfloat16) * ws.to(torch.bfloat16)[:, None])
    return y.reshape(*x.shape[:-1], w8.shape[0])
