"""The C-ABI library without a GPU: it loads, exports every symbol include/spinf_b200.h declares, and rejects malformed calls on the
host (negative SPINF_ERR_* codes) before touching CUDA. No compute entry point is called with valid arguments here."""

import ctypes
import os
import re

import numpy as np
import pytest

from spinf_serve_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NULL = None


def _declared():
    with open(os.path.join(ROOT, "include", "spinf_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(spinf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol_and_binding_covers_them():
    lib = _lib.lib()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names
    assert lib.spinf_version() >= 100


def test_argument_errors_are_reported_on_the_host():
    lib = _lib.lib()
    p = ctypes.c_void_p(16)  # a non-null, never dereferenced pointer: every call below is rejected before any CUDA work
    assert lib.spinf_fp8_rowwise_quant(NULL, 4, 64, p, p, NULL) == -1           # null input
    assert lib.spinf_fp8_rowwise_quant(p, 4, 60, p, p, NULL) == -1              # K not a multiple of 8
    assert lib.spinf_fp8_rowwise_gemm(p, p, p, p, p, 4, 100, 64, NULL) == -1    # N not a multiple of 16
    assert lib.spinf_fp8_rowwise_gemm(p, p, p, p, p, -1, 128, 64, NULL) == -1   # negative M
    assert lib.spinf_fp8_tensor_gemm(p, p, p, p, p, 4, 128, 60, NULL) == -1     # K not a multiple of 16
    assert lib.spinf_fp8_tensor_quant(p, 100, p, 0, p, NULL, NULL, NULL) == -1  # element count not a multiple of 8
    assert lib.spinf_fp8_tensor_quant(p, 64, p, 2, p, NULL, NULL, NULL) == -1   # from_amax is 0 or 1
    assert lib.spinf_abs_max(p, 12, p, NULL) == -1                              # element count not a multiple of 8
    assert lib.spinf_bf16_gemm_ld(p, p, p, 4, 128, 64, 64, NULL) == -1          # pitch smaller than N
    assert lib.spinf_w4_gemm(p, p, p, 128, p, 4, 128, 100, 128, NULL) == -1     # K not a multiple of 64
    assert lib.spinf_w4_gemm(p, p, p, 12, p, 4, 128, 128, 128, NULL) == -1      # group not a multiple of 8
    assert lib.spinf_w4_gemm_glu(p, p, p, 128, 2, p, 4, 128, 128, 64, NULL) == -1  # activation code
    assert lib.spinf_w4_gemm_glu(p, p, p, 128, 1, p, 4, 136, 128, 72, NULL) == -1  # 2F not a multiple of 16
    assert lib.spinf_w4_repack(p, p, 4, 100, NULL) == -1                        # K not a multiple of 8
    assert lib.spinf_w4_repack(ctypes.c_void_p(18), p, 4, 128, NULL) == -1      # not 4-byte aligned
    assert lib.spinf_fp8_rowwise_gemm_glu(p, p, p, p, p, p, 4, 100, 64, 0, NULL) == -1  # F not a multiple of 128
    # zero rows are nothing to do, whatever the row pointers are (an empty tensor has a null data pointer)
    assert lib.spinf_fp8_rowwise_quant(NULL, 0, 64, NULL, NULL, NULL) == 0
    assert lib.spinf_fp8_rowwise_gemm(NULL, NULL, p, p, NULL, 0, 128, 64, NULL) == 0
    assert lib.spinf_w4_gemm(NULL, p, p, 128, NULL, 0, 128, 128, 128, NULL) == 0
    assert lib.spinf_option_logprobs_workspace_bytes(-1, 10, 1) == -1
    assert lib.spinf_option_logprobs(p, p, 4, 64, 1000, p, 2, ctypes.c_float(0.0), p, p, 8, NULL) == -1  # workspace too small
    assert lib.spinf_option_logprobs_static(p, p, 4096, 64, 262144, p, 2, ctypes.c_float(0.0), p, NULL, NULL) == -4  # beyond the static scratch
    assert lib.spinf_tree_attn_fwd(p, p, p, p, 130, 4, 2, 128, 512, 256, 512, p, p, p, 0, ctypes.c_float(1.0), p, p, p, p, NULL, NULL) == -1  # n % 128
    assert lib.spinf_tree_attn_fwd(p, p, p, p, 128, 4, 3, 128, 512, 384, 512, p, p, p, 0, ctypes.c_float(1.0), p, p, p, p, NULL, NULL) == -1  # H % Hkv
    assert lib.spinf_tree_attn_fwd(p, p, p, p, 128, 4, 2, 64, 256, 128, 256, p, p, p, 0, ctypes.c_float(1.0), p, p, p, p, NULL, NULL) == -1   # head dim
    assert lib.spinf_tree_attn_fwd(p, p, p, p, 128, 4, 2, 128, 512, 256, 512, p, p, p, 0, ctypes.c_float(1.0), p, p, p, NULL, NULL, NULL) == -1  # no visibility words
    assert lib.spinf_tile_mask_bits(p, p, p, 100, 0, p, p, p, NULL) == -1  # n % 128
    assert lib.spinf_fused_norm(p, NULL, NULL, NULL, NULL, 4, 16384, ctypes.c_float(1e-6), 0, NULL, NULL, NULL, NULL, NULL) == -1    # hidden > 8192
    assert lib.spinf_gdn_recurrent(p, p, p, p, p, p, 8, 256, 512, 4, 2, 4, 64, 128, ctypes.c_float(1.0), p, 1, NULL, NULL, NULL, NULL, NULL, NULL) == -1  # K != 128
    assert lib.spinf_gdn_recurrent(p, p, p, p, p, p, 8, 256, 512, 4, 2, 4, 128, 128, ctypes.c_float(1.0), p, 1, NULL, p, NULL, NULL, NULL, NULL) == -1  # h0 without h0_idx
    assert lib.spinf_gdn_chunked_workspace_bytes(-1, 4) == -1
    assert lib.spinf_gdn_chunked(p, p, p, p, p, p, 8, 256, 512, 4, 2, 4, 64, 128, ctypes.c_float(1.0), p, 1, NULL, NULL, NULL, NULL, NULL, p, p, 1, 8, p, 1 << 20, NULL) == -1  # K != 128
    assert lib.spinf_gdn_chunked(p, p, p, p, p, p, 8, 256, 512, 4, 2, 4, 128, 128, ctypes.c_float(1.0), p, 1, NULL, NULL, NULL, NULL, NULL, p, p, 1, 8, p, 16, NULL) == -1  # workspace too small


def test_tile_descriptor_host_function_edge_cases():
    lib = _lib.lib()
    z = np.zeros(0, np.int32)
    out_c, out_b, out_f = np.zeros(1, np.int32), np.zeros(1, np.int32), np.zeros(1, np.uint8)
    assert lib.spinf_tile_desc_build_host(_lib.ptr(z), _lib.ptr(z), _lib.ptr(z), 0, 0, _lib.ptr(out_c), _lib.ptr(out_b), _lib.ptr(out_f)) == 0  # empty stream
    a = np.zeros(100, np.int32)
    assert lib.spinf_tile_desc_build_host(_lib.ptr(a), _lib.ptr(a), _lib.ptr(a), 100, 0, _lib.ptr(out_c), _lib.ptr(out_b), _lib.ptr(out_f)) == -1  # ragged
    # an all-pad stream: every block visits itself only
    from spinf_serve_b200 import packer as P

    pad = np.full(384, -1, np.int32)
    td = P.tile_desc(pad, pad, np.zeros(384, np.int32), 64)
    assert td.offsets.tolist() == [0, 1, 2, 3] and td.blocks.tolist() == [0, 1, 2] and not td.flags.any()


def test_wrappers_refuse_cpu_tensors_and_a_missing_library(monkeypatch):
    import torch

    from spinf_serve_b200 import ops

    with pytest.raises(_lib.SpinfError):
        ops.fp8_rowwise_quant(torch.zeros((4, 64), dtype=torch.bfloat16))  # no CPU path
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libspinf_b200.so")
    with pytest.raises(_lib.SpinfError):
        _lib.lib()
