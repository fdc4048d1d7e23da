"""Tree-mask attention seam: the "tree_flex" attention interface of the Gemma stack (spinf_serve/models/gemma4.py:99-121) and the
Qwen stack's tree_attention (spinf_serve/models/qwen35/qwen.py:605-623), backed by the sm_100a kernel spinf_tree_attn_fwd.

Where the reference hands FlexAttention a BlockMask (block tables + a mask_mod closure over device copies of art / end / pos,
spinf_serve/scorer.py:163-238), this build hands the kernel a TileMask: the same per-token arrays on the device plus the packed
tile lists of packer.tile_desc."""

from dataclasses import dataclass

import numpy as np
import torch

from spinf_serve_b200 import _lib, ops, packer
from spinf_serve_b200._lib import SpinfError, check, ptr, stream_ptr


@dataclass
class TileMask:
    """what one layer type's attention needs on the device (the counterpart of the reference's BlockMask)"""

    art: torch.Tensor      # int32 [n]
    end: torch.Tensor      # int32 [n]
    pos: torch.Tensor      # int32 [n]
    offsets: torch.Tensor  # int32 [nb + 1]
    blocks: torch.Tensor   # int32 [visited]
    flags: torch.Tensor    # uint8 [visited]
    bits: torch.Tensor     # int64 [visited, 2, 128]: per entry, key half and query row, which of the half's 64 keys the row sees
    window: int            # 0 = full attention
    n: int
    visited: int
    skipped_fraction: float


def stream_masks(art, end, pos, window, device, always_window=True):
    """{"full_attention": TileMask, "sliding_attention": TileMask} for one packed stream, as Scorer._block_masks builds them
    (spinf_serve/scorer.py:207-238): the sliding table is used when a position reaches the window or always_window is set (aligned
    jobs), else sliding layers share the full table. Host arrays go up through pinned memory on the current stream."""
    art = np.ascontiguousarray(art, np.int32)
    end = np.ascontiguousarray(end, np.int32)
    pos = np.ascontiguousarray(pos, np.int32)
    n = len(art)
    if n % packer.BLOCK:
        raise SpinfError(f"stream length {n} is not a multiple of {packer.BLOCK}")

    def up(a):
        return torch.from_numpy(a).pin_memory().to(device, non_blocking=True)

    d_art, d_end, d_pos = up(art), up(end), up(pos)

    def one(w):
        td = packer.tile_desc(art, end, pos, w)
        blocks = td.blocks if len(td.blocks) else np.zeros(1, np.int32)
        flags = td.flags if len(td.flags) else np.zeros(1, np.uint8)
        d_off, d_blocks = up(td.offsets), up(blocks)
        # the mask rule, evaluated once for the stream: every layer of this type and every head reads these words
        bits = torch.empty((len(blocks), 2, packer.BLOCK), dtype=torch.int64, device=device)
        if n:
            check(
                _lib.lib().spinf_tile_mask_bits(ptr(d_art), ptr(d_end), ptr(d_pos), n, int(w or 0), ptr(d_off), ptr(d_blocks), ptr(bits), stream_ptr()),
                "spinf_tile_mask_bits",
            )
            ops.COUNTS["launches"] += 1
        return TileMask(d_art, d_end, d_pos, d_off, d_blocks, up(flags), bits, int(w or 0), n, td.visited, td.skipped_fraction)

    full = one(None)
    binding = window is not None and (always_window or (n > 0 and int(pos.max()) >= window))
    return {"full_attention": full, "sliding_attention": one(window) if binding else full}


def tree_attention(q, k, v, mask: TileMask, scale: float, out=None, row_amax=None):
    """q [n, H, D], k / v [n, Hkv, D] bf16 (the last two dimensions dense, any row pitch) -> out [n, H, D] bf16. row_amax: optional
    zeroed fp32 [n] that receives max |out| per token (for ops.fp8_quant_from_amax)"""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise SpinfError(f"{name}: expected a CUDA bf16 [n, heads, head_dim] tensor with dense heads")
    n, H, D = q.shape
    Hkv = k.shape[1]
    if k.shape != v.shape or k.shape[0] != n or k.shape[2] != D or n != mask.n or k.stride(0) != v.stride(0):
        raise SpinfError("tree_attention: q / k / v / mask shapes do not agree")
    _lib.init(q.device)
    if out is None:
        out = torch.empty((n, H, D), dtype=torch.bfloat16, device=q.device)
    check(
        _lib.lib().spinf_tree_attn_fwd(
            ptr(q), ptr(k), ptr(v), ptr(out), n, H, Hkv, D, q.stride(0), k.stride(0), out.stride(0), ptr(mask.art), ptr(mask.end),
            ptr(mask.pos), mask.window, float(scale), ptr(mask.offsets), ptr(mask.blocks), ptr(mask.flags), ptr(mask.bits), ptr(row_amax),
            stream_ptr(),
        ),
        "spinf_tree_attn_fwd",
    )
    ops.COUNTS["launches"] += 1
    return out


def tree_flex_forward(module, query, key, value, attention_mask, scaling=None, sliding_window=None, **kw):
    """the attention-interface callable: query [1, H, N, D], key / value [1, Hkv, N, D] -> (out [1, N, H, D] contiguous, None).
    attention_mask is the TileMask of the layer's type (the stack passes {"full_attention": ..., "sliding_attention": ...}[type])"""
    if query.shape[0] != 1:
        raise SpinfError("the packed path runs one stream per forward (batch dimension 1)")

    def rows(t):  # [1, h, N, D] -> [N, h, D] without a copy when it is the transpose of a token-major tensor
        t = t[0].transpose(0, 1)
        return t if t.stride(2) == 1 and t.stride(1) == t.shape[2] else t.contiguous()

    scale = float(scaling) if scaling is not None else query.shape[-1] ** -0.5
    out = tree_attention(rows(query), rows(key), rows(value), attention_mask, scale)
    return out[None], None


def register() -> None:
    """registers "tree_flex" with transformers' attention interfaces; registering before the reference's register_flex makes
    that call a no-op (spinf_serve/models/gemma4.py:82-83), so a reference-built model runs this kernel unchanged"""
    from transformers import AttentionInterface

    if "tree_flex" not in AttentionInterface._global_mapping:
        AttentionInterface.register("tree_flex", tree_flex_forward)
