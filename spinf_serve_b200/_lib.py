"""ctypes binding of libspinf_b200.so, the C-ABI library of sm_100a kernels (include/spinf_b200.h).

There is no fallback: if the library is missing or a call is rejected, the caller gets an exception. `lib()` loads the shared
object built in place by spinf_serve_b200.csrc.build; tensors cross the boundary as raw device pointers plus sizes, the CUDA
stream as an integer handle."""

import ctypes
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libspinf_b200.so")

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_f32 = ctypes.c_float

# name -> (restype, argtypes); mirrors include/spinf_b200.h declaration by declaration
SIGNATURES = {
    "spinf_version": (ctypes.c_int, []),
    "spinf_init": (ctypes.c_int, []),
    "spinf_last_status": (ctypes.c_int, [_p]),
    "spinf_selftest_bounded_wait": (ctypes.c_int, [_i64, _p]),
    "spinf_fp8_rowwise_quant": (ctypes.c_int, [_p, _i64, _i64, _p, _p, _p]),
    "spinf_fp8_rowwise_gemm": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "spinf_fp8_rowwise_gemm_small_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "spinf_fp8_rowwise_gemm_small": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "spinf_abs_max": (ctypes.c_int, [_p, _i64, _p, _p]),
    "spinf_fp8_tensor_quant": (ctypes.c_int, [_p, _i64, _p, _i32, _p, _p, _p, _p]),
    "spinf_fp8_tensor_gemm": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "spinf_int8_rowwise_quant": (ctypes.c_int, [_p, _i64, _i64, _p, _p, _p]),
    "spinf_int8_rowwise_gemm": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "spinf_fp8_rowwise_gemm_glu": (ctypes.c_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _p]),
    "spinf_fp8_rowwise_gemm_qkv": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i64, _p, _p, _p, _p, _f32, _i32, _i32, _p]),
    "spinf_fp8_quant_from_amax": (ctypes.c_int, [_p, _p, _i64, _i64, _p, _p, _p]),
    "spinf_bf16_gemm_ld": (ctypes.c_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _p]),
    "spinf_bf16_gemm_small_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "spinf_bf16_gemm_small": (ctypes.c_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _p, _i64, _p]),
    "spinf_w4_repack": (ctypes.c_int, [_p, _p, _i64, _i64, _p]),
    "spinf_w4_gemm_glu": (ctypes.c_int, [_p, _p, _p, _i32, _i32, _p, _i64, _i64, _i64, _i64, _p]),
    "spinf_w4_gemm": (ctypes.c_int, [_p, _p, _p, _i32, _p, _i64, _i64, _i64, _i64, _p]),
    "spinf_bf16_gemm": (ctypes.c_int, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "spinf_option_logprobs_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "spinf_option_logprobs": (ctypes.c_int, [_p, _p, _i64, _i64, _i64, _p, _i64, _f32, _p, _p, _i64, _p]),
    "spinf_option_logprobs_static": (ctypes.c_int, [_p, _p, _i64, _i64, _i64, _p, _i64, _f32, _p, _p, _p]),
    "spinf_tile_desc_build_host": (_i64, [_p, _p, _p, _i64, _i32, _p, _p, _p]),
    "spinf_tile_desc_build_host_img": (_i64, [_p, _p, _p, _p, _i64, _i32, _p, _p, _p]),
    "spinf_fused_norm": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _f32, _i32, _p, _p, _p, _p, _p]),
    "spinf_qkv_norm_rope": (ctypes.c_int, [_p, _i64, _i64, _i32, _i32, _i32, _p, _p, _p, _p, _i32, _f32, _i32, _i32, _p]),
    "spinf_qkv_norm_rope_gated": (ctypes.c_int, [_p, _i64, _i64, _i32, _i32, _i32, _p, _p, _p, _p, _i32, _f32, _i32, _p, _p]),
    "spinf_attn_gate": (ctypes.c_int, [_p, _p, _i64, _i64, _i32, _i32, _p]),
    "spinf_rope_table": (ctypes.c_int, [_p, _i64, _i32, _p, _p, _p, _p]),
    "spinf_glu_quant": (ctypes.c_int, [_p, _i64, _i64, _i32, _p, _p, _p, _p]),
    "spinf_embed_scale": (ctypes.c_int, [_p, _p, _i64, _i64, _i64, _f32, _p, _p]),
    "spinf_gdn_recurrent": (
        ctypes.c_int,
        [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _p, _i64, _p, _p, _p, _p, _p, _p],
    ),
    "spinf_gdn_chunked_workspace_bytes": (_i64, [_i64, _i32]),
    "spinf_gdn_chunked": (
        ctypes.c_int,
        [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _i64, _p],
    ),
    "spinf_gdn_tree_workspace_bytes": (_i64, [_i64, _i32]),
    "spinf_gdn_tree_prep": (ctypes.c_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _p, _i64, _p, _p, _i64, _p, _i64, _p]),
    "spinf_gdn_tree_scan": (ctypes.c_int, [_p, _p, _p, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _p, _i64, _p, _p, _p, _i64, _p, _p, _p, _i64, _p]),
    "spinf_gdn_tree_scan_tc": (ctypes.c_int, [_p, _p, _p, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _i64, _p, _p, _p, _p, _i64, _p, _p, _p, _i64, _p]),
    "spinf_w4_gemm_small_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "spinf_w4_gemm_small": (ctypes.c_int, [_p, _p, _p, _i32, _p, _i64, _i64, _i64, _i64, _p, _i64, _p]),
    "spinf_w4_small_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "spinf_w4_small": (ctypes.c_int, [_p, _p, _p, _i32, _p, _i64, _i64, _i64, _i64, _p, _i64, _p]),
    "spinf_x_attention_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i64, _i64, _i64]),
    "spinf_x_attention": (
        ctypes.c_int,
        [_p, _i64, _p, _p, _p, _i64, _p, _p, _p, _p, _i64, _p, _p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _f32, _f32, _p, _i64, _p, _i64, _p],
    ),
    "spinf_gdn_prologue": (ctypes.c_int, [_p, _i64, _i64, _i64, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _p, _p, _p, _p, _p, _p]),
    "spinf_gdn_epilogue": (ctypes.c_int, [_p, _p, _i64, _p, _f32, _i64, _i32, _i32, _p, _p]),
    "spinf_tree_attn_fwd": (
        ctypes.c_int,
        [_p, _p, _p, _p, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _p, _p, _p, _i32, _f32, _p, _p, _p, _p, _p, _p],
    ),
    "spinf_tile_mask_bits": (ctypes.c_int, [_p, _p, _p, _i64, _i32, _p, _p, _p, _p]),
    "spinf_tile_mask_bits_img": (ctypes.c_int, [_p, _p, _p, _p, _i64, _i32, _i32, _p, _p, _p, _p]),
}

ERRORS = {
    -1: "bad argument (null pointer, unsupported size or alignment)",
    -2: "CUDA runtime error (no sm_100 device, or a launch failed)",
    -3: "TMA descriptor could not be encoded (unaligned base or pitch)",
    -4: "size exceeds a documented maximum",
}
STATUS = {
    1: "a consumer waited for a TMA stage that never filled",
    2: "a producer waited for a pipeline stage that was never released",
    3: "a wait on a tensor-memory accumulator gave up",
    4: "a bounded wait gave up",
    5: "an index read from a descriptor was out of range",
}

_lock = threading.Lock()
_lib = None
_inited = set()


class SpinfError(RuntimeError):
    pass


def lib():
    """the loaded library; raises SpinfError when it has not been built (python -m spinf_serve_b200.csrc.build)"""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise SpinfError(f"{LIB_PATH} is missing: build it with `python -m spinf_serve_b200.csrc.build`; there is no fallback")
                handle = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)  # AttributeError if the header and the library disagree
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code < 0:
        raise SpinfError(f"{what}: {ERRORS.get(code, code)}")


def init(device) -> None:
    """prepares `device` (a torch.device or index) once: status word, driver entry points"""
    import torch

    idx = torch.device(device).index if not isinstance(device, int) else device
    idx = torch.cuda.current_device() if idx is None else idx
    if idx in _inited:
        return
    with torch.cuda.device(idx):
        check(lib().spinf_init(), "spinf_init")
    _inited.add(idx)


def stream_ptr():
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def last_status(raise_on_error: bool = True) -> int:
    """synchronises the current stream and returns the device status word (0 = clean), clearing it"""
    st = lib().spinf_last_status(stream_ptr())
    if st < 0:
        check(st, "spinf_last_status")
    if st and raise_on_error:
        raise SpinfError(f"device status {st}: {STATUS.get(st, 'unknown')}")
    return st


def ptr(t):
    """device (or host) address of a tensor / numpy array, None -> NULL"""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return ctypes.c_void_p(t.data_ptr())
    return ctypes.c_void_p(t.ctypes.data)
