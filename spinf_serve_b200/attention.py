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


@dataclass
class HostTiles:
    """the host half of a stream's masks: the per-token arrays and the tile lists of both layer types, built ahead of the GPU (the
    scorer's producer thread); `sliding` is None when sliding layers share the full table"""

    art: np.ndarray
    end: np.ndarray
    pos: np.ndarray
    window: int
    full: "packer.TileDesc"
    sliding: "packer.TileDesc | None"
    grp: "np.ndarray | None" = None  # streams with images: the image of every placeholder token, -1 elsewhere
    bidir_all: bool = True           # images' bidirectional blocks on every layer, past the window; False: sliding layers only, within it

    @property
    def n(self) -> int:
        return len(self.art)

    def arrays(self) -> dict:
        """name -> array, everything the device half needs (one staging copy carries them all)"""
        out = {"art": self.art, "end": self.end, "pos32": self.pos}
        if self.grp is not None:
            out["grp"] = self.grp
        for name, td in (("full", self.full), ("sliding", self.sliding)):
            if td is not None:
                out[name + ".offsets"] = td.offsets
                out[name + ".blocks"] = td.blocks if len(td.blocks) else np.zeros(1, np.int32)
                out[name + ".flags"] = td.flags if len(td.flags) else np.zeros(1, np.uint8)
        return out


def host_tiles(art, end, pos, window, always_window=True, grp=None, bidir_all=True) -> HostTiles:
    """the tile lists of one packed stream as Scorer._block_masks takes them from block_tables (spinf_serve/scorer.py:207-238,
    packer.py:426-491): the sliding table is used when a position reaches the window or always_window is set (aligned jobs),
    else sliding layers share the full table. grp: Batch.grp of a stream with images (None: text only); bidir_all: which layers
    give an image's placeholders their two-way block (the reference's model._vision_bidir_all, scorer.py:178-198). Host work only
    (the library's C++ descriptor builder)."""
    art = np.ascontiguousarray(art, np.int32)
    end = np.ascontiguousarray(end, np.int32)
    pos = np.ascontiguousarray(pos, np.int32)
    grp = None if grp is None else np.ascontiguousarray(grp, np.int32)
    n = len(art)
    if n % packer.BLOCK:
        raise SpinfError(f"stream length {n} is not a multiple of {packer.BLOCK}")
    if grp is not None and len(grp) != n:
        raise SpinfError("grp does not cover the stream")
    binding = window is not None and (always_window or (n > 0 and int(pos.max()) >= window))
    return HostTiles(art, end, pos, int(window or 0), packer.tile_desc(art, end, pos, None, grp),
                     packer.tile_desc(art, end, pos, window, grp) if binding else None, grp, bool(bidir_all))


def device_masks(ht: HostTiles, st: dict, device) -> dict:
    """the device half: st maps the names of HostTiles.arrays() to device tensors (already copied, or in flight on the current
    stream). Evaluates the mask rule once per layer type (spinf_tile_mask_bits): every layer of the type and every head reads
    those words. -> {"full_attention": TileMask, "sliding_attention": TileMask}"""
    n = ht.n
    grp = st["grp"] if ht.grp is not None else None

    def one(name, td, w, g, in_window):
        d_off, d_blocks, d_flags = st[name + ".offsets"], st[name + ".blocks"], st[name + ".flags"]
        bits = torch.empty((d_blocks.numel(), 2, packer.BLOCK), dtype=torch.int64, device=device)
        if n:
            check(
                _lib.lib().spinf_tile_mask_bits_img(ptr(st["art"]), ptr(st["end"]), ptr(st["pos32"]), ptr(g), n, int(w), int(in_window),
                                                    ptr(d_off), ptr(d_blocks), ptr(bits), stream_ptr()),
                "spinf_tile_mask_bits_img",
            )
            ops.COUNTS["launches"] += 1
        return TileMask(st["art"], st["end"], st["pos32"], d_off, d_blocks, d_flags, bits, int(w), n, td.visited, td.skipped_fraction)

    # images: every layer, past the window (bidir_all), or the sliding layers only and within the window (scorer.py:186-198)
    full = one("full", ht.full, 0, grp if ht.bidir_all else None, 0)
    if ht.sliding is not None:
        sliding = one("sliding", ht.sliding, ht.window, grp, 0 if ht.bidir_all else 1)
    elif grp is not None and not ht.bidir_all:  # no position reaches the window: the full table with the sliding layers' rule
        sliding = one("full", ht.full, ht.window, grp, 1)
    else:
        sliding = full
    return {"full_attention": full, "sliding_attention": sliding}


def stream_masks(art, end, pos, window, device, always_window=True, grp=None, bidir_all=True):
    """host_tiles + device_masks in one call, each array going up through pinned memory on the current stream (one-off streams:
    tests, calibration; the scorer stages a forward's arrays in one copy instead)"""
    ht = host_tiles(art, end, pos, window, always_window, grp, bidir_all)
    st = {k: torch.from_numpy(a).pin_memory().to(device, non_blocking=True) for k, a in ht.arrays().items()}
    return device_masks(ht, st, device)


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
    prof = ops.PROFILE
    if prof is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(
        _lib.lib().spinf_tree_attn_fwd(
            ptr(q), ptr(k), ptr(v), ptr(out), n, H, Hkv, D, q.stride(0), k.stride(0), out.stride(0), ptr(mask.art), ptr(mask.end),
            ptr(mask.pos), mask.window, float(scale), ptr(mask.offsets), ptr(mask.blocks), ptr(mask.flags), ptr(mask.bits), ptr(row_amax),
            stream_ptr(),
        ),
        "spinf_tree_attn_fwd",
    )
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 0.0, f"attn:{mask.window}"))
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
