"""Gated DeltaNet on the library's kernels, with the reference's call signatures: recurrent / chunked (spinf_serve/models/qwen35/
gdn.py:197-235, :109-133) and gdn_tree / gdn_indexed (spinf_serve/models/qwen35/qwen.py:515-590), plus the fused steps around the
recurrence (GatedDeltaNet.forward, qwen.py:640-673). Tensors keep the reference's leading batch dimension of 1 where it has one."""

import ctypes

import torch

from spinf_serve_b200 import _lib, ops
from spinf_serve_b200._lib import SpinfError, check, ptr, stream_ptr


def _rows(t, heads, dim, name):
    """[1, rows, heads, dim] or [rows, heads, dim] bf16 with a dense (heads, dim) block per row -> (tensor, row pitch)"""
    if t.dim() == 4:
        t = t[0]
    if not t.is_cuda or t.dim() != 3 or t.shape[1] != heads or t.shape[2] != dim or t.stride(2) != 1 or t.stride(1) != dim:
        raise SpinfError(f"{name}: expected a CUDA [rows, {heads}, {dim}] tensor with dense rows")
    return t, t.stride(0)


def recurrent(q, k, v, g, beta, scale, cu, n, h0=None, h0_idx=None, ht=None, ht_idx=None, idx=None, o=None):
    """the reference's gdn.recurrent contract: segments cu [n + 1] of the rows idx (None: rows 0.. in call order) of q / k
    [1, rows, Hk, 128], v [1, rows, Hv, 128], g (fp32) / beta (bf16) [1, rows, Hv]; states read at h0[h0_idx], written at
    ht[ht_idx]; outputs go to the same rows of o [1, rows, Hv, 128] bf16 (allocated, zero-filled, when None), which is returned"""
    Hk, K = q.shape[-2], q.shape[-1]
    Hv, V = v.shape[-2], v.shape[-1]
    q3, qp = _rows(q, Hk, K, "q")
    k3, kp = _rows(k, Hk, K, "k")
    v3, vp = _rows(v, Hv, V, "v")
    g2 = g[0] if g.dim() == 3 else g
    b2 = beta[0] if beta.dim() == 3 else beta
    if qp != kp or g2.stride(0) != b2.stride(0) or g2.stride(1) != 1 or b2.stride(1) != 1:
        raise SpinfError("gdn.recurrent: q / k and g / beta must share their row pitches")
    if g2.dtype != torch.float32 or b2.dtype != torch.bfloat16 or q3.dtype != torch.bfloat16 or v3.dtype != torch.bfloat16:
        raise SpinfError("gdn.recurrent: expected bf16 q / k / v / beta and fp32 g")
    _lib.init(q3.device)
    rows = v3.shape[0]
    if o is None:
        o = torch.zeros((1, rows, Hv, V), dtype=torch.bfloat16, device=v3.device)
    o3 = o[0] if o.dim() == 4 else o
    if not o3.is_contiguous() or o3.dtype != torch.bfloat16:
        raise SpinfError("gdn.recurrent: o must be a contiguous bf16 tensor")
    for name, t in (("cu", cu), ("idx", idx), ("h0_idx", h0_idx), ("ht_idx", ht_idx)):
        if t is not None and (t.dtype != torch.int64 or not t.is_cuda or not t.is_contiguous()):
            raise SpinfError(f"gdn.recurrent: {name} must be a contiguous int64 CUDA tensor")
    for name, t in (("h0", h0), ("ht", ht)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape[1:]) != (Hv, K, V)):
            raise SpinfError(f"gdn.recurrent: {name} must be a contiguous fp32 [*, Hv, K, V] tensor")
    check(
        _lib.lib().spinf_gdn_recurrent(
            ptr(q3), ptr(k3), ptr(v3), ptr(g2), ptr(b2), ptr(o3), rows, qp, vp, g2.stride(0), Hk, Hv, K, V, ctypes.c_float(scale),
            ptr(cu), int(n), ptr(idx), ptr(h0 if h0_idx is not None else None), ptr(h0_idx if h0 is not None else None),
            ptr(ht if ht_idx is not None else None), ptr(ht_idx if ht is not None else None), stream_ptr(),
        ),
        "spinf_gdn_recurrent",
    )
    ops.COUNTS["launches"] += 1
    return o


CHUNK = 64


def chunk_table(cu_cpu, device):
    """(chunk_seg, chunk_t0) int32 device tensors: the 64-token chunks of a call's segments, in order (what the reference gets
    from fla's prepare_chunk_indices)"""
    segs, t0s = [], []
    for n in range(len(cu_cpu) - 1):
        length = int(cu_cpu[n + 1]) - int(cu_cpu[n])
        for t0 in range(0, length, CHUNK):
            segs.append(n)
            t0s.append(t0)
    mk = lambda x: torch.tensor(x, dtype=torch.int32).pin_memory().to(device, non_blocking=True)
    return mk(segs), mk(t0s)


def chunked(q, k, v, g, beta, scale, cu, cu_cpu, h0=None, h0_idx=None, ht=None, ht_idx=None, chunk_size=64, idx=None, o=None, table=None):
    """the reference's gdn.chunked contract (gdn.py:109-133): the recurrence in its chunked form, 64 tokens at a time. As in the
    reference the tensors may be gathered (rows 0.. in call order, idx None); with idx the kernels read and write the stream rows
    themselves. table: the call's chunk_table when the caller keeps it (built here otherwise)."""
    if chunk_size != CHUNK:
        raise SpinfError("gdn.chunked: the kernels are written for 64-token chunks")
    Hk, K = q.shape[-2], q.shape[-1]
    Hv, V = v.shape[-2], v.shape[-1]
    q3, qp = _rows(q, Hk, K, "q")
    k3, kp = _rows(k, Hk, K, "k")
    v3, vp = _rows(v, Hv, V, "v")
    g2 = g[0] if g.dim() == 3 else g
    b2 = beta[0] if beta.dim() == 3 else beta
    if qp != kp or g2.stride(0) != b2.stride(0) or g2.stride(1) != 1 or b2.stride(1) != 1:
        raise SpinfError("gdn.chunked: q / k and g / beta must share their row pitches")
    if g2.dtype != torch.float32 or b2.dtype != torch.bfloat16 or q3.dtype != torch.bfloat16 or v3.dtype != torch.bfloat16:
        raise SpinfError("gdn.chunked: expected bf16 q / k / v / beta and fp32 g")
    _lib.init(q3.device)
    rows = v3.shape[0]
    if o is None:
        o = torch.zeros((1, rows, Hv, V), dtype=torch.bfloat16, device=v3.device)
    o3 = o[0] if o.dim() == 4 else o
    if not o3.is_contiguous() or o3.dtype != torch.bfloat16:
        raise SpinfError("gdn.chunked: o must be a contiguous bf16 tensor")
    for name, t in (("cu", cu), ("idx", idx), ("h0_idx", h0_idx), ("ht_idx", ht_idx)):
        if t is not None and (t.dtype != torch.int64 or not t.is_cuda or not t.is_contiguous()):
            raise SpinfError(f"gdn.chunked: {name} must be a contiguous int64 CUDA tensor")
    for name, t in (("h0", h0), ("ht", ht)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape[1:]) != (Hv, K, V)):
            raise SpinfError(f"gdn.chunked: {name} must be a contiguous fp32 [*, Hv, K, V] tensor")
    n = len(cu_cpu) - 1
    tokens = int(cu_cpu[-1]) if n > 0 else 0
    seg, t0 = table if table is not None else chunk_table(cu_cpu, q3.device)
    need = _lib.lib().spinf_gdn_chunked_workspace_bytes(tokens, Hv)
    ws = torch.empty(max(int(need), 16), dtype=torch.uint8, device=q3.device)
    check(
        _lib.lib().spinf_gdn_chunked(
            ptr(q3), ptr(k3), ptr(v3), ptr(g2), ptr(b2), ptr(o3), rows, qp, vp, g2.stride(0), Hk, Hv, K, V, ctypes.c_float(scale),
            ptr(cu), n, ptr(idx), ptr(h0 if h0_idx is not None else None), ptr(h0_idx if h0 is not None else None),
            ptr(ht if ht_idx is not None else None), ptr(ht_idx if ht is not None else None), ptr(seg), ptr(t0), seg.numel(), tokens,
            ptr(ws), ws.numel(), stream_ptr(),
        ),
        "spinf_gdn_chunked",
    )
    ops.COUNTS["launches"] += 2
    return o


FUSED = True  # gdn_tree runs the one-launch-per-level kernels when the plan carries their schedule (False: the per-call kernels)
SCAN = "tc"  # the level scan: "tc" = tcgen05 / tensor memory (spinf_gdn_tree_scan_tc), "mma" = warp-level MMAs (spinf_gdn_tree_scan)


def gdn_tree_fused(q, k, v, g, beta, plan):
    """gdn_tree on the fused kernels: one preparation launch for the layer (every chunk of every segment), then one scan launch per
    level of the trie, a parent's state read once per group of siblings. The workspace is kept on the plan: every recurrent layer
    of the forward reuses it."""
    f = plan.fused
    Hk, K = q.shape[-2], q.shape[-1]
    Hv, V = v.shape[-2], v.shape[-1]
    q3, qp = _rows(q, Hk, K, "q")
    k3, kp = _rows(k, Hk, K, "k")
    v3, vp = _rows(v, Hv, V, "v")
    if qp != kp or g.stride(0) != beta.stride(0) or g.stride(1) != 1 or beta.stride(1) != 1:
        raise SpinfError("gdn_tree: q / k and g / beta must share their row pitches")
    if g.dtype != torch.float32 or beta.dtype != torch.bfloat16 or q3.dtype != torch.bfloat16 or v3.dtype != torch.bfloat16:
        raise SpinfError("gdn_tree: expected bf16 q / k / v / beta and fp32 g")
    _lib.init(q3.device)
    rows = v3.shape[0]
    o = torch.zeros((rows, Hv, V), dtype=torch.bfloat16, device=v3.device)
    if f.plan_tokens == 0:
        return o
    L = _lib.lib()
    need = int(L.spinf_gdn_tree_workspace_bytes(f.plan_tokens, Hv))
    if f.workspace is None or f.workspace.numel() < need or f.workspace.device != q3.device:
        f.workspace = torch.empty(need, dtype=torch.uint8, device=q3.device)
    ws = f.workspace
    prof = ops.PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(
        L.spinf_gdn_tree_prep(ptr(q3), ptr(k3), ptr(v3), ptr(g), ptr(beta), rows, qp, vp, g.stride(0), Hk, Hv, K, V, ptr(f.row_of), f.plan_tokens,
                              ptr(f.chunk_p0), ptr(f.chunk_len), f.chunk_p0.numel(), ptr(ws), ws.numel(), stream_ptr()),
        "spinf_gdn_tree_prep",
    )
    ops.COUNTS["launches"] += 1
    scale = K**-0.5
    prev_states = None
    for (grp_parent, grp_ubeg, units, unit_rows), nk in zip(f.levels, f.n_keep):
        states = torch.empty((nk, Hv, K, V), dtype=torch.float32, device=q3.device) if nk else None
        if SCAN == "tc":
            check(
                L.spinf_gdn_tree_scan_tc(ptr(q3), ptr(k3), ptr(o), rows, qp, Hk, Hv, K, V, ctypes.c_float(scale), f.plan_tokens, ptr(grp_parent),
                                         ptr(grp_ubeg), ptr(units), ptr(unit_rows), grp_parent.numel(), ptr(prev_states), ptr(states), ptr(ws),
                                         ws.numel(), stream_ptr()),
                "spinf_gdn_tree_scan_tc",
            )
        else:
            check(
                L.spinf_gdn_tree_scan(ptr(q3), ptr(k3), ptr(o), rows, qp, Hk, Hv, K, V, ctypes.c_float(scale), ptr(f.row_of), f.plan_tokens,
                                      ptr(grp_parent), ptr(grp_ubeg), ptr(units), grp_parent.numel(), ptr(prev_states), ptr(states), ptr(ws),
                                      ws.numel(), stream_ptr()),
                "spinf_gdn_tree_scan",
            )
        ops.COUNTS["launches"] += 1
        prev_states = states
    if prof is not None:
        e1.record()
        # q, k in; v in and o out (bf16); g fp32 and beta bf16: the bytes a pass must move per real token
        prof.append((e0, e1, float(f.plan_tokens) * (2 * Hk * K * 2 + 2 * Hv * V * 2 + Hv * 6), "gdn"))
    return o


def gdn_tree(q, k, v, g, beta, plan, mod=None):
    """q, k [T, Hk, Dk], v [T, Hv, Dv], g, beta [T, Hv] -> [T, Hv, Dv]: every segment of the plan from its parent's final state,
    level by level (gdn_indexed, qwen.py:550-590); the kernel reads and writes the stream rows itself through each call's idx"""
    if FUSED and getattr(plan, "fused", None) is not None and q.shape[-1] == 128 and v.shape[-1] == 128 and q.is_cuda:
        return gdn_tree_fused(q, k, v, g, beta, plan)
    scale = q.shape[-1] ** -0.5
    o = torch.zeros_like(v)
    prev_states = None
    for calls, nk in zip(plan.levels, plan.n_keep):
        states = torch.empty((nk, v.shape[1], q.shape[-1], v.shape[-1]), dtype=torch.float32, device=q.device) if nk else None
        for c in calls:
            h0 = prev_states if c.h0_idx is not None else None
            ht = states if c.ht_idx is not None else None
            if c.kind == "chunked":  # segments longer than the plan's `short` (64), as the reference dispatches them
                if getattr(c, "table", None) is None:
                    c.table = chunk_table(c.cu_cpu, q.device)  # kept on the call: every recurrent layer of the forward reuses it
                chunked(q, k, v, g, beta, scale, c.cu, c.cu_cpu, h0=h0, h0_idx=c.h0_idx, ht=ht, ht_idx=c.ht_idx, idx=c.idx, o=o, table=c.table)
            else:
                recurrent(q, k, v, g, beta, scale, c.cu, len(c.cu_cpu) - 1, h0=h0, h0_idx=c.h0_idx, ht=ht, ht_idx=c.ht_idx, idx=c.idx, o=o)
        prev_states = states
    return o


def prologue(y, conv, conv_w, A_log, dt_bias, Hk, Dk, Hv, Dv, n_tokens=None):
    """in-projection rows y [rows, 2 Hk Dk + 2 Hv Dv + 2 Hv] bf16 -> q, k [T, Hk, Dk], v [T, Hv, Dv] bf16, z (a view of y)
    [T, Hv, Dv], g [T, Hv] fp32, beta [T, Hv] bf16 (qwen.py:651-668)"""
    if not y.is_cuda or y.dtype != torch.bfloat16 or y.dim() != 2 or y.stride(1) != 1:
        raise SpinfError("gdn.prologue: y must be a CUDA bf16 [rows, features] tensor")
    _lib.init(y.device)
    T = y.shape[0] if n_tokens is None else n_tokens
    dev = y.device
    q = torch.empty((T, Hk, Dk), dtype=torch.bfloat16, device=dev)
    k = torch.empty_like(q)
    v = torch.empty((T, Hv, Dv), dtype=torch.bfloat16, device=dev)
    g = torch.empty((T, Hv), dtype=torch.float32, device=dev)
    beta = torch.empty((T, Hv), dtype=torch.bfloat16, device=dev)
    check(
        _lib.lib().spinf_gdn_prologue(
            ptr(y), y.stride(0), y.shape[0], T, ptr(conv), ptr(conv_w), ptr(A_log), ptr(dt_bias), Hk, Hv, Dk, Dv, ptr(q), ptr(k), ptr(v),
            ptr(g), ptr(beta), stream_ptr(),
        ),
        "spinf_gdn_prologue",
    )
    ops.COUNTS["launches"] += 1
    conv_dim = 2 * Hk * Dk + Hv * Dv
    return q, k, v, y[:T, conv_dim : conv_dim + Hv * Dv], g, beta


def epilogue(o, z, norm_w, eps):
    """o [T, Hv, Dv] bf16, z [T, Hv Dv] (a row-pitched view) -> gated RMS norm [T, Hv Dv] bf16 (qwen.py:670-673)"""
    T, Hv, Dv = o.shape
    out = torch.empty((T, Hv * Dv), dtype=torch.bfloat16, device=o.device)
    check(
        _lib.lib().spinf_gdn_epilogue(ptr(o), ptr(z), z.stride(0), ptr(norm_w), ctypes.c_float(eps), T, Hv, Dv, ptr(out), stream_ptr()),
        "spinf_gdn_epilogue",
    )
    ops.COUNTS["launches"] += 1
    return out
