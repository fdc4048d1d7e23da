"""Tensor-level wrappers over the C ABI: each function checks dtype / layout / device, allocates the outputs with torch (device
memory and streams are torch's), and enqueues one entry point of libspinf_b200.so on the current stream. Nothing here computes on
the CPU or through another library: a tensor that is not on a CUDA device is an error."""

import ctypes

import torch

from spinf_serve_b200 import _lib
from spinf_serve_b200._lib import SpinfError, check, ptr, stream_ptr

FP8 = torch.float8_e4m3fn

# Measurement hooks (bench.py): COUNTS["launches"] counts the kernels this module enqueued; when PROFILE is a list, every row-wise
# fp8 or int4 GEMM, every attention launch and every recurrent layer pass is bracketed by CUDA events on its stream and
# (start, end, work, kind) is appended: kind "fp8_gemm" / "w4_gemm" with 2 M N K, "attn:<window>" with 0 (the caller knows the
# stream's unmasked pairs), "gdn" with the pass's algorithmic bytes.
COUNTS = {"launches": 0}
PROFILE = None


def _need(t, dtype, name, dims=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise SpinfError(f"{name}: expected a CUDA tensor (this library has no CPU path)")
    if t.dtype != dtype:
        raise SpinfError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise SpinfError(f"{name}: expected {dims} dimensions, got {t.dim()}")
    if not t.is_contiguous():
        raise SpinfError(f"{name}: expected a contiguous tensor")
    _lib.init(t.device)


def fp8_rowwise_quant(x):
    """x [..., K] bf16 -> (x8 [M, K] e4m3, xs [M, 1] fp32), per-row dynamic scales (quant_act_row, spinf_serve/quant/linears.py:29-33)"""
    x2 = x.reshape(-1, x.shape[-1])
    _need(x2, torch.bfloat16, "x", 2)
    M, K = x2.shape
    x8 = torch.empty((M, K), dtype=FP8, device=x.device)
    xs = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    check(_lib.lib().spinf_fp8_rowwise_quant(ptr(x2), M, K, ptr(x8), ptr(xs), stream_ptr()), "spinf_fp8_rowwise_quant")
    COUNTS["launches"] += 1
    return x8, xs


def fp8_rowwise_gemm(x8, xs, w8, ws, out=None):
    """y [M, N] bf16 = (x8 [M, K] @ w8 [N, K]^T) * xs [M] * ws [N] (spinf_serve/quant/linears.py:93-96)"""
    _need(x8, FP8, "x8", 2)
    _need(w8, FP8, "w8", 2)
    xs1, ws1 = xs.reshape(-1), ws.reshape(-1)
    _need(xs1, torch.float32, "xs", 1)
    _need(ws1, torch.float32, "ws", 1)
    M, K = x8.shape
    N = w8.shape[0]
    if w8.shape[1] != K or xs1.numel() != M or ws1.numel() != N:
        raise SpinfError(f"fp8_rowwise_gemm: shapes do not agree: x8 {tuple(x8.shape)}, w8 {tuple(w8.shape)}, xs {xs1.numel()}, ws {ws1.numel()}")
    y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    if out is not None:
        _need(out, torch.bfloat16, "out", 2)
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(
        _lib.lib().spinf_fp8_rowwise_gemm(ptr(x8), ptr(xs1), ptr(w8), ptr(ws1), ptr(y), M, N, K, stream_ptr()),
        "spinf_fp8_rowwise_gemm",
    )
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N * K, "fp8_gemm"))
    COUNTS["launches"] += 1
    return y


def fp8_rowwise_gemm_small(x8, xs, w8, ws, workspace=None):
    """fp8_rowwise_gemm for a decoding step's few rows (M <= 128): the K dimension is cut into slices where the column tiles alone
    do not occupy the GPU, the slices' fp32 sums added in order before the scales and the rounding (may differ from
    fp8_rowwise_gemm in the last bf16 bit). workspace: optional uint8 tensor reused between calls."""
    _need(x8, FP8, "x8", 2)
    _need(w8, FP8, "w8", 2)
    xs1, ws1 = xs.reshape(-1), ws.reshape(-1)
    _need(xs1, torch.float32, "xs", 1)
    _need(ws1, torch.float32, "ws", 1)
    M, K = x8.shape
    N = w8.shape[0]
    if w8.shape[1] != K or xs1.numel() != M or ws1.numel() != N:
        raise SpinfError("fp8_rowwise_gemm_small: shapes do not agree")
    need = int(_lib.lib().spinf_fp8_rowwise_gemm_small_workspace_bytes(M, N, K))
    if not need:
        return fp8_rowwise_gemm(x8, xs, w8, ws)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x8.device)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    check(
        _lib.lib().spinf_fp8_rowwise_gemm_small(ptr(x8), ptr(xs1), ptr(w8), ptr(ws1), ptr(y), M, N, K, ptr(workspace), workspace.numel(),
                                                stream_ptr()),
        "spinf_fp8_rowwise_gemm_small",
    )
    COUNTS["launches"] += 2
    return y


def fp8_tensor_quant(x, scale=None, peak=None, want_amax=False):
    """per-tensor fp8 quantisation of x [..., K] bf16 -> (x8 [M, K] e4m3, s fp32 scalar on the device).
    scale = None: dynamic, s = max(max|x|, 1e-12) / 448 (quant_act, spinf_serve/quant/linears.py:22-26; two kernels, no host
    sync); scale = fp32 device scalar: static, s = scale (Fp8StaticLinear.forward, linears.py:113). peak: optional fp32 device
    scalar updated to max(peak, max|x| / (448 s)) (the static scheme's clipping monitor, linears.py:111-112). want_amax (dynamic
    only): also return the device scalar max|x|."""
    x2 = x.reshape(-1, x.shape[-1])
    _need(x2, torch.bfloat16, "x", 2)
    M, K = x2.shape
    if (M * K) % 8:
        raise SpinfError("fp8_tensor_quant: the element count must be a multiple of 8")
    x8 = torch.empty((M, K), dtype=FP8, device=x.device)
    L = _lib.lib()
    if scale is None and M * K == 0:  # no maximum to take: the scale at its floor, max(0, 1e-12) / 448
        s = torch.full((), float(torch.tensor(1e-12) / 448.0), dtype=torch.float32, device=x.device)
        return (x8, s, torch.zeros((), dtype=torch.float32, device=x.device)) if want_amax else (x8, s)
    if scale is None:
        both = torch.empty(2, dtype=torch.float32, device=x.device)  # [max|x|, s]: other CTAs still read the maximum when s is written
        amax, s = both[0], both[1]
        check(L.spinf_abs_max(ptr(x2), M * K, ptr(amax), stream_ptr()), "spinf_abs_max")
        check(L.spinf_fp8_tensor_quant(ptr(x2), M * K, ptr(amax), 1, ptr(x8), ptr(s), ptr(peak), stream_ptr()), "spinf_fp8_tensor_quant")
        COUNTS["launches"] += 2
        if want_amax:
            return x8, s, amax
    else:
        s = scale
        _need(s.reshape(1), torch.float32, "scale", 1)
        check(L.spinf_fp8_tensor_quant(ptr(x2), M * K, ptr(s), 0, ptr(x8), None, ptr(peak), stream_ptr()), "spinf_fp8_tensor_quant")
        COUNTS["launches"] += 1
    return x8, s


def fp8_tensor_gemm(x8, xs, w8, ws, out=None):
    """y [M, N] bf16 = (x8 [M, K] @ w8 [N, K]^T) * xs * ws with one fp32 device scalar per operand (the per-tensor
    torch._scaled_mm of Fp8Linear / Fp8StaticLinear, spinf_serve/quant/linears.py:77,114)"""
    _need(x8, FP8, "x8", 2)
    _need(w8, FP8, "w8", 2)
    _need(xs.reshape(1), torch.float32, "xs", 1)
    _need(ws.reshape(1), torch.float32, "ws", 1)
    M, K = x8.shape
    N = w8.shape[0]
    if w8.shape[1] != K:
        raise SpinfError(f"fp8_tensor_gemm: shapes do not agree: x8 {tuple(x8.shape)}, w8 {tuple(w8.shape)}")
    y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    if out is not None:
        _need(out, torch.bfloat16, "out", 2)
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(_lib.lib().spinf_fp8_tensor_gemm(ptr(x8), ptr(xs), ptr(w8), ptr(ws), ptr(y), M, N, K, stream_ptr()), "spinf_fp8_tensor_gemm")
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N * K, "fp8_gemm"))
    COUNTS["launches"] += 1
    return y


def int8_rowwise_quant(x):
    """x [..., K] bf16 -> (x8 [M, K] int8, xs [M, 1] fp32), per-row dynamic scales amax / 127, round half to even
    (quant_act_int8, spinf_serve/quant/linears.py:34-38)"""
    x2 = x.reshape(-1, x.shape[-1])
    _need(x2, torch.bfloat16, "x", 2)
    M, K = x2.shape
    x8 = torch.empty((M, K), dtype=torch.int8, device=x.device)
    xs = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    check(_lib.lib().spinf_int8_rowwise_quant(ptr(x2), M, K, ptr(x8), ptr(xs), stream_ptr()), "spinf_int8_rowwise_quant")
    COUNTS["launches"] += 1
    return x8, xs


def int8_rowwise_gemm(x8, xs, w8, ws):
    """y [M, N] bf16 = float(x8 [M, K] @ w8 [N, K]^T as int32) * xs [M] * ws [N] (torch._int_mm and the scaling after it,
    spinf_serve/quant/linears.py:61)"""
    _need(x8, torch.int8, "x8", 2)
    _need(w8, torch.int8, "w8", 2)
    xs1, ws1 = xs.reshape(-1), ws.reshape(-1)
    _need(xs1, torch.float32, "xs", 1)
    _need(ws1, torch.float32, "ws", 1)
    M, K = x8.shape
    N = w8.shape[0]
    if w8.shape[1] != K or xs1.numel() != M or ws1.numel() != N:
        raise SpinfError(f"int8_rowwise_gemm: shapes do not agree: x8 {tuple(x8.shape)}, w8 {tuple(w8.shape)}, xs {xs1.numel()}, ws {ws1.numel()}")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    check(_lib.lib().spinf_int8_rowwise_gemm(ptr(x8), ptr(xs1), ptr(w8), ptr(ws1), ptr(y), M, N, K, stream_ptr()), "spinf_int8_rowwise_gemm")
    COUNTS["launches"] += 1
    return y


def w4_repack(q):
    """q uint8 [N, K/2] in the reference's engine layout (low nibble = even k) -> the same bytes re-ordered for w4_gemm (per 8
    consecutive k: even k in the low half of the 32-bit word, odd k in the high half). Load time, once per weight."""
    _need(q, torch.uint8, "q", 2)
    N, K2 = q.shape
    if (2 * K2) % 8:
        raise SpinfError("w4_repack: K must be a multiple of 8")
    out = torch.empty_like(q)
    check(_lib.lib().spinf_w4_repack(ptr(q), ptr(out), N, 2 * K2, stream_ptr()), "spinf_w4_repack")
    COUNTS["launches"] += 1
    return out


def w4_gemm_glu(x, qw, scales, group, act="silu"):
    """y [M, F] bf16 = act(gate) * up of the fused gate|up int4 projection, the activation inside the GEMM epilogue: qw [2F, K/2]
    and scales [2F, K/group] hold the rows interleaved (2c = gate channel c, 2c + 1 = up channel c), each row as w4_repack leaves it"""
    _need(x, torch.bfloat16, "x", 2)
    _need(qw, torch.uint8, "qw", 2)
    _need(scales, torch.float16, "scales", 2)
    M, K = x.shape
    N2 = qw.shape[0]
    if qw.shape[1] * 2 != K or scales.shape[0] != N2 or N2 % 16:
        raise SpinfError(f"w4_gemm_glu: shapes do not agree: x {tuple(x.shape)}, qw {tuple(qw.shape)}, scales {tuple(scales.shape)}")
    y = torch.empty((M, N2 // 2), dtype=torch.bfloat16, device=x.device)
    code = {"gelu_tanh": 0, "silu": 1}[act]
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(_lib.lib().spinf_w4_gemm_glu(ptr(x), ptr(qw), ptr(scales), group, code, ptr(y), M, N2, K, N2 // 2, stream_ptr()), "spinf_w4_gemm_glu")
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N2 * K, "w4_gemm"))
    COUNTS["launches"] += 1
    return y


def w4_gemm(x, qw, scales, group, extra=None):
    """y [M, N (+ E)] bf16 = x [M, K] bf16 @ dq(qw, scales)^T (qw as w4_repack leaves it), with E un-quantised bf16 output channels `extra` [E, K] appended
    (Int4Linear.forward in bf16 mode, spinf_serve/models/qwen35/qwen.py:455-458); qw uint8 [N, K/2], scales fp16 [N, K/group]"""
    _need(x, torch.bfloat16, "x", 2)
    _need(qw, torch.uint8, "qw", 2)
    _need(scales, torch.float16, "scales", 2)
    M, K = x.shape
    N = qw.shape[0]
    if qw.shape[1] * 2 != K or scales.shape != (N, K // group):
        raise SpinfError("w4_gemm: shapes do not agree")
    E = 0 if extra is None else extra.shape[0]
    if extra is not None:
        _need(extra, torch.bfloat16, "extra", 2)
    y = torch.empty((M, N + E), dtype=torch.bfloat16, device=x.device)
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(_lib.lib().spinf_w4_gemm(ptr(x), ptr(qw), ptr(scales), group, ptr(y), M, N, K, N + E, stream_ptr()), "spinf_w4_gemm")
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N * K, "w4_gemm"))
    COUNTS["launches"] += 1
    if E:
        tail = ctypes.c_void_p(y.data_ptr() + 2 * N)
        check(_lib.lib().spinf_bf16_gemm_ld(ptr(x), ptr(extra), tail, M, E, K, N + E, stream_ptr()), "spinf_bf16_gemm_ld")
        COUNTS["launches"] += 1
    return y


def w4_small(x, q, scales, group, extra=None, workspace=None):
    """the W4A16 linear of a decoding step (w4gemm.linear, spinf_serve/quant/w4gemm.py:44-66): x [M <= 128, K] bf16, q uint8
    [N, K/2] in the ENGINE layout (not w4_repack'ed), scales fp16 [N, K/group] -> [M, N (+ E)] bf16, `extra` [E, K] bf16 rows
    appended as a plain product"""
    _need(x, torch.bfloat16, "x", 2)
    _need(q, torch.uint8, "q", 2)
    _need(scales, torch.float16, "scales", 2)
    M, K = x.shape
    N = q.shape[0]
    if q.shape[1] * 2 != K or scales.shape != (N, K // group) or M > 128:
        raise SpinfError(f"w4_small: shapes do not agree: x {tuple(x.shape)}, q {tuple(q.shape)}, scales {tuple(scales.shape)}")
    E = 0 if extra is None else extra.shape[0]
    if extra is not None:
        _need(extra, torch.bfloat16, "extra", 2)
    y = torch.empty((M, N + E), dtype=torch.bfloat16, device=x.device)
    need = int(_lib.lib().spinf_w4_small_workspace_bytes(M, N, K))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(_lib.lib().spinf_w4_small(ptr(x), ptr(q), ptr(scales), group, ptr(y), M, N, K, N + E, ptr(workspace), workspace.numel(), stream_ptr()), "spinf_w4_small")
    COUNTS["launches"] += 3
    if E:
        tail = ctypes.c_void_p(y.data_ptr() + 2 * N)
        check(_lib.lib().spinf_bf16_gemm_ld(ptr(x), ptr(extra), tail, M, E, K, N + E, stream_ptr()), "spinf_bf16_gemm_ld")
        COUNTS["launches"] += 1
    return y


def x_attention(q, kp, vp, pos_p, kt, vt, pos_t, own_t, gk, gv, qpos, step, beam, scaling, window=None, softcap=None, out=None, workspace=None,
                k_new=None, v_new=None):
    """the decoding step's attention (`_x_attention`, spinf_serve/decode.py:71-104) on token-major tensors: q [G, Q, H, D] (a view
    with unit stride over (H, D) and any row pitch); prefix kp / vp [G, Lp, h, D] + pos_p [G, Lp] int32 (-1: padding); templates
    kt / vt [G, Tt, h, D] + pos_t, own_t [G, Tt] int32; generated gk / gv [G, Q, S, h, D]; qpos [G, Q] int32; step: int32 device
    scalar (tokens 0..step of the generated range are live) -> [G, Q, H, D] bf16. k_new, v_new [G * Q, h, D] (views with contiguous
    heads and one row pitch, e.g. of the fused q|k|v projection): written into gk / gv at token `step` inside the same launch"""
    G, Q, H, D = q.shape
    if q.dtype != torch.bfloat16 or not q.is_cuda or q.stride(3) != 1 or q.stride(2) != D or q.stride(0) != Q * q.stride(1):
        raise SpinfError("x_attention: q must be a CUDA bf16 [G, Q, H, D] view with contiguous heads and evenly pitched rows")
    for name, t, dt in (("kp", kp, torch.bfloat16), ("vp", vp, torch.bfloat16), ("kt", kt, torch.bfloat16), ("vt", vt, torch.bfloat16),
                        ("gk", gk, torch.bfloat16), ("gv", gv, torch.bfloat16), ("pos_p", pos_p, torch.int32), ("pos_t", pos_t, torch.int32),
                        ("own_t", own_t, torch.int32), ("qpos", qpos, torch.int32), ("step", step, torch.int32)):
        _need(t, dt, name)
    Lp, h = kp.shape[1], kp.shape[2]
    Tt, S = kt.shape[1], gk.shape[2]
    if kp.shape != (G, Lp, h, D) or vp.shape != kp.shape or kt.shape != (G, Tt, h, D) or vt.shape != kt.shape or gk.shape != (G, Q, S, h, D) or gv.shape != gk.shape:
        raise SpinfError("x_attention: key / value shapes do not agree")
    if pos_p.shape != (G, Lp) or pos_t.shape != (G, Tt) or own_t.shape != (G, Tt) or qpos.shape != (G, Q) or step.numel() != 1:
        raise SpinfError("x_attention: position / owner shapes do not agree")
    kv_pitch = 0
    if (k_new is None) != (v_new is None):
        raise SpinfError("x_attention: k_new and v_new come together")
    if k_new is not None:
        for t in (k_new, v_new):
            if t.dtype != torch.bfloat16 or not t.is_cuda or t.shape != (G * Q, h, D) or t.stride(2) != 1 or t.stride(1) != D or t.stride(0) != k_new.stride(0):
                raise SpinfError("x_attention: k_new / v_new must be CUDA bf16 [G * Q, h, D] views with contiguous heads and one row pitch")
        kv_pitch = k_new.stride(0)
    if out is None:
        out = torch.empty((G, Q, H, D), dtype=torch.bfloat16, device=q.device)
    need = int(_lib.lib().spinf_x_attention_workspace_bytes(G, Q, H, D, Lp, Tt, S))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    check(
        _lib.lib().spinf_x_attention(
            ptr(q), q.stride(1), ptr(kp), ptr(vp), ptr(pos_p), Lp, ptr(kt), ptr(vt), ptr(pos_t), ptr(own_t), Tt, ptr(gk), ptr(gv), S,
            ptr(k_new), ptr(v_new), kv_pitch, ptr(qpos), ptr(step), G, Q, H, h, D, beam, int(window or 0), float(scaling), float(softcap or 0.0), ptr(out), out.stride(1),
            ptr(workspace), workspace.numel(), stream_ptr(),
        ),
        "spinf_x_attention",
    )
    COUNTS["launches"] += 4
    return out


def w4_gemm_small(x, qw, scales, group, extra=None, workspace=None):
    """w4_gemm for a decoding step's few rows (M <= 256): the K dimension is cut into slices where the column tiles alone do not
    occupy the GPU, the slices' fp32 sums added in order before the rounding (may differ from w4_gemm in the last bf16 bit)"""
    _need(x, torch.bfloat16, "x", 2)
    _need(qw, torch.uint8, "qw", 2)
    _need(scales, torch.float16, "scales", 2)
    M, K = x.shape
    N = qw.shape[0]
    if qw.shape[1] * 2 != K or scales.shape != (N, K // group) or M > 256:
        raise SpinfError("w4_gemm_small: shapes do not agree")
    E = 0 if extra is None else extra.shape[0]
    if extra is not None:
        _need(extra, torch.bfloat16, "extra", 2)
    y = torch.empty((M, N + E), dtype=torch.bfloat16, device=x.device)
    need = int(_lib.lib().spinf_w4_gemm_small_workspace_bytes(M, N, K))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(_lib.lib().spinf_w4_gemm_small(ptr(x), ptr(qw), ptr(scales), group, ptr(y), M, N, K, N + E, ptr(workspace) if need else None,
                                         workspace.numel() if need else 0, stream_ptr()), "spinf_w4_gemm_small")
    COUNTS["launches"] += 2 if need else 1
    if E:
        tail = ctypes.c_void_p(y.data_ptr() + 2 * N)
        need_e = int(_lib.lib().spinf_bf16_gemm_small_workspace_bytes(M, E, K))  # the extra rows' product in K slices too
        ws_e = torch.empty(max(need_e, 16), dtype=torch.uint8, device=x.device)
        check(_lib.lib().spinf_bf16_gemm_small(ptr(x), ptr(extra), tail, M, E, K, N + E, ptr(ws_e), ws_e.numel(), stream_ptr()),
              "spinf_bf16_gemm_small")
        COUNTS["launches"] += 2 if need_e else 1
    return y


def glu_tile_order(F: int):
    """row permutation that puts a fused gate|up weight [2F, K] (gate rows first) into the tiled order of fp8_gemm_glu: per 128
    features, four blocks of 32 gate rows followed by the 32 up rows of the same features"""
    if F % 128:
        raise SpinfError("the fused gate|up GEMM needs an intermediate size that is a multiple of 128")
    f = torch.arange(F).view(F // 32, 1, 32)
    return torch.cat([f, f + F], dim=1).reshape(-1)


def fp8_gemm_glu(x8, xs, w8_tiled, ws_tiled, act="gelu_tanh"):
    """gate|up projection + gated activation + row-wise fp8 quantisation: x8 [M, K], weights in glu_tile_order ->
    (y8 [M, F] e4m3, ys [M, 1] fp32); equals fp8_rowwise_gemm followed by glu_quant"""
    _need(x8, FP8, "x8", 2)
    _need(w8_tiled, FP8, "w8_tiled", 2)
    xs1, ws1 = xs.reshape(-1), ws_tiled.reshape(-1)
    _need(xs1, torch.float32, "xs", 1)
    _need(ws1, torch.float32, "ws_tiled", 1)
    M, K = x8.shape
    F = w8_tiled.shape[0] // 2
    if w8_tiled.shape[1] != K or xs1.numel() != M or ws1.numel() != 2 * F:
        raise SpinfError("fp8_gemm_glu: shapes do not agree")
    dev = x8.device
    y = torch.empty((M, F), dtype=torch.bfloat16, device=dev)
    amax = torch.empty((M,), dtype=torch.float32, device=dev)
    code = {"gelu_tanh": 0, "silu": 1}[act]
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(
        _lib.lib().spinf_fp8_rowwise_gemm_glu(ptr(x8), ptr(xs1), ptr(w8_tiled), ptr(ws1), ptr(y), ptr(amax), M, F, K, code, stream_ptr()),
        "spinf_fp8_rowwise_gemm_glu",
    )
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * 2 * F * K, "fp8_gemm"))
    y8 = torch.empty((M, F), dtype=FP8, device=dev)
    ys = torch.empty((M, 1), dtype=torch.float32, device=dev)
    check(_lib.lib().spinf_fp8_quant_from_amax(ptr(y), ptr(amax), M, F, ptr(y8), ptr(ys), stream_ptr()), "spinf_fp8_quant_from_amax")
    COUNTS["launches"] += 2
    return y8, ys, y


def fp8_gemm_qkv(x8, xs, w8, ws, H, Hkv, D, wq, wk, cos, sin, eps=1e-6, plus1=False, norm_v=True):
    """fused q|k|v projection with the head norms and the (full-width) rotary embedding in the GEMM epilogue: equals
    fp8_rowwise_gemm followed by qkv_norm_rope; -> [M, (H + 2 Hkv) D] bf16"""
    _need(x8, FP8, "x8", 2)
    _need(w8, FP8, "w8", 2)
    xs1, ws1 = xs.reshape(-1), ws.reshape(-1)
    _need(xs1, torch.float32, "xs", 1)
    _need(ws1, torch.float32, "ws", 1)
    for t, name in ((wq, "wq"), (wk, "wk")):
        _need(t, torch.bfloat16, name, 1)
    _need(cos, torch.bfloat16, "cos", 2)
    _need(sin, torch.bfloat16, "sin", 2)
    M, K = x8.shape
    N = (H + 2 * Hkv) * D
    if w8.shape != (N, K) or xs1.numel() != M or ws1.numel() != N or cos.shape != (M, D // 2) or sin.shape != (M, D // 2):
        raise SpinfError("fp8_gemm_qkv: shapes do not agree (the rotary table must span the whole head)")
    if wq.numel() != D or wk.numel() != D:
        raise SpinfError("fp8_gemm_qkv: head-norm weights must have D entries")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    prof = PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(
        _lib.lib().spinf_fp8_rowwise_gemm_qkv(
            ptr(x8), ptr(xs1), ptr(w8), ptr(ws1), ptr(y), M, H, Hkv, D, K, ptr(wq), ptr(wk), ptr(cos), ptr(sin), ctypes.c_float(eps),
            int(plus1), int(norm_v), stream_ptr(),
        ),
        "spinf_fp8_rowwise_gemm_qkv",
    )
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N * K, "fp8_gemm"))
    COUNTS["launches"] += 1
    return y


def fp8_quant_from_amax(y, row_amax):
    """row-wise fp8 quantisation of y [M, K] bf16 with the row maxima already known (fp32 [M]): one pass -> (x8 [M, K], xs [M, 1])"""
    _need(y, torch.bfloat16, "y", 2)
    _need(row_amax, torch.float32, "row_amax", 1)
    M, K = y.shape
    if row_amax.numel() != M:
        raise SpinfError("fp8_quant_from_amax: one maximum per row")
    x8 = torch.empty((M, K), dtype=FP8, device=y.device)
    xs = torch.empty((M, 1), dtype=torch.float32, device=y.device)
    check(_lib.lib().spinf_fp8_quant_from_amax(ptr(y), ptr(row_amax), M, K, ptr(x8), ptr(xs), stream_ptr()), "spinf_fp8_quant_from_amax")
    COUNTS["launches"] += 1
    return x8, xs


def bf16_gemm(x, w):
    """y [M, N] bf16 = x [M, K] @ w [N, K]^T, fp32 accumulation"""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.bfloat16, "w", 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise SpinfError("bf16_gemm: inner dimensions differ")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    check(_lib.lib().spinf_bf16_gemm(ptr(x), ptr(w), ptr(y), M, N, K, stream_ptr()), "spinf_bf16_gemm")
    COUNTS["launches"] += 1
    return y


def option_logprobs(h, W, cols, softcap=None, workspace=None):
    """log-probs of the option tokens `cols` (sorted distinct int32 ids, on the device) at read rows h [R, hidden] bf16 under the
    lm head W [vocab, hidden] bf16 -> [R, len(cols)] fp32 (Scorer._logprobs + the column gather, spinf_serve/scorer.py:340-355,254)"""
    _need(h, torch.bfloat16, "h", 2)
    _need(W, torch.bfloat16, "W", 2)
    _need(cols, torch.int32, "cols", 1)
    R, hidden = h.shape
    vocab = W.shape[0]
    if W.shape[1] != hidden:
        raise SpinfError("option_logprobs: hidden sizes differ")
    n_cols = cols.numel()
    out = torch.empty((R, n_cols), dtype=torch.float32, device=h.device)
    need = _lib.lib().spinf_option_logprobs_workspace_bytes(R, vocab, n_cols)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=h.device)
    check(
        _lib.lib().spinf_option_logprobs(
            ptr(h), ptr(W), R, hidden, vocab, ptr(cols), n_cols, ctypes.c_float(softcap or 0.0), ptr(out), ptr(workspace),
            workspace.numel(), stream_ptr(),
        ),
        "spinf_option_logprobs",
    )
    COUNTS["launches"] += 3
    return out


def fused_norm(y, w1=None, residual=None, w2=None, rows=None, eps=1e-6, plus1=False, want_h=False, want_norm=False, want_fp8=False):
    """[RMSNorm w1] -> [+ residual] -> [RMSNorm w2] over the rows of y [*, hidden] bf16 (rows: int64 indices of the input rows to
    read) -> dict with "h" (after the residual add), "norm" (bf16 of the second norm), "x8"/"xs" (its row-wise fp8 form)"""
    _need(y, torch.bfloat16, "y", 2)
    hidden = y.shape[1]
    n_out = rows.numel() if rows is not None else y.shape[0]
    dev = y.device
    if rows is not None:
        _need(rows, torch.int64, "rows", 1)
    for name, w in (("w1", w1), ("w2", w2)):
        if w is not None:
            _need(w, torch.bfloat16, name, 1)
    if residual is not None:
        _need(residual, torch.bfloat16, "residual", 2)
    out = {}
    if want_h:
        out["h"] = torch.empty((n_out, hidden), dtype=torch.bfloat16, device=dev)
    if want_norm:
        out["norm"] = torch.empty((n_out, hidden), dtype=torch.bfloat16, device=dev)
    if want_fp8:
        out["x8"] = torch.empty((n_out, hidden), dtype=FP8, device=dev)
        out["xs"] = torch.empty((n_out, 1), dtype=torch.float32, device=dev)
    check(
        _lib.lib().spinf_fused_norm(
            ptr(y), ptr(rows), ptr(w1), ptr(residual), ptr(w2), n_out, hidden, ctypes.c_float(eps), int(plus1), ptr(out.get("h")),
            ptr(out.get("norm")), ptr(out.get("x8")), ptr(out.get("xs")), stream_ptr(),
        ),
        "spinf_fused_norm",
    )
    COUNTS["launches"] += 1
    return out


def rope_table(pos, inv_freq):
    """pos int32 [n], inv_freq fp32 [R/2] -> (cos, sin) bf16 [n, R/2]"""
    _need(pos, torch.int32, "pos", 1)
    _need(inv_freq, torch.float32, "inv_freq", 1)
    n, half = pos.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.bfloat16, device=pos.device)
    sin = torch.empty_like(cos)
    check(_lib.lib().spinf_rope_table(ptr(pos), n, 2 * half, ptr(inv_freq), ptr(cos), ptr(sin), stream_ptr()), "spinf_rope_table")
    COUNTS["launches"] += 1
    return cos, sin


def qkv_norm_rope(qkv, H, Hkv, D, wq, wk, cos, sin, eps=1e-6, plus1=False, norm_v=True):
    """in place on the fused projection output qkv [n, (H + 2 Hkv) D]: head norms, then rotary on q and k"""
    _need(qkv, torch.bfloat16, "qkv", 2)
    _need(wq, torch.bfloat16, "wq", 1)
    _need(wk, torch.bfloat16, "wk", 1)
    _need(cos, torch.bfloat16, "cos", 2)
    _need(sin, torch.bfloat16, "sin", 2)
    n = qkv.shape[0]
    check(
        _lib.lib().spinf_qkv_norm_rope(
            ptr(qkv), qkv.stride(0), n, H, Hkv, D, ptr(wq), ptr(wk), ptr(cos), ptr(sin), 2 * cos.shape[1], ctypes.c_float(eps),
            int(plus1), int(norm_v), stream_ptr(),
        ),
        "spinf_qkv_norm_rope",
    )
    COUNTS["launches"] += 1
    return qkv


def qkv_norm_rope_gated(y, H, Hkv, D, wq, wk, cos, sin, eps=1e-6, plus1=True):
    """the Qwen attention layout [H x (q | gate)] | k | v: -> dense q [n, H, D] (normed, rotated); k normed and rotated in place"""
    _need(y, torch.bfloat16, "y", 2)
    n = y.shape[0]
    q = torch.empty((n, H, D), dtype=torch.bfloat16, device=y.device)
    check(
        _lib.lib().spinf_qkv_norm_rope_gated(
            ptr(y), y.stride(0), n, H, Hkv, D, ptr(wq), ptr(wk), ptr(cos), ptr(sin), 2 * cos.shape[1], ctypes.c_float(eps), int(plus1),
            ptr(q), stream_ptr(),
        ),
        "spinf_qkv_norm_rope_gated",
    )
    COUNTS["launches"] += 1
    return q


def attn_gate(o, y, H, D):
    """in place o [n, H, D] *= sigmoid(gate), the gates read from the interleaved projection rows y"""
    check(_lib.lib().spinf_attn_gate(ptr(o), ptr(y), y.stride(0), o.shape[0], H, D, stream_ptr()), "spinf_attn_gate")
    COUNTS["launches"] += 1
    return o


def glu_quant(gu, act="gelu_tanh", want_fp8=True, want_y=False):
    """gu [n, 2F] bf16 (gate | up) -> act(gate) * up as (x8 [n, F], xs [n, 1]) and/or bf16 y [n, F]"""
    _need(gu, torch.bfloat16, "gu", 2)
    n, F = gu.shape[0], gu.shape[1] // 2
    x8 = torch.empty((n, F), dtype=FP8, device=gu.device) if want_fp8 else None
    xs = torch.empty((n, 1), dtype=torch.float32, device=gu.device) if want_fp8 else None
    y = torch.empty((n, F), dtype=torch.bfloat16, device=gu.device) if want_y else None
    code = {"gelu_tanh": 0, "silu": 1}[act]
    check(_lib.lib().spinf_glu_quant(ptr(gu), n, F, code, ptr(x8), ptr(xs), ptr(y), stream_ptr()), "spinf_glu_quant")
    COUNTS["launches"] += 1
    return x8, xs, y


def embed_scale(ids, emb, scale):
    """ids int64 [n], emb [vocab, hidden] bf16 -> bf16(emb[ids] * scale) [n, hidden]"""
    _need(ids, torch.int64, "ids", 1)
    _need(emb, torch.bfloat16, "emb", 2)
    out = torch.empty((ids.numel(), emb.shape[1]), dtype=torch.bfloat16, device=emb.device)
    check(
        _lib.lib().spinf_embed_scale(ptr(ids), ptr(emb), ids.numel(), emb.shape[1], emb.shape[0], ctypes.c_float(scale), ptr(out), stream_ptr()),
        "spinf_embed_scale",
    )
    COUNTS["launches"] += 1
    return out
