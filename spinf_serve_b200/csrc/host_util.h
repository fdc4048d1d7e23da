// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry point (the library does not link
// libcuda, so it loads on machines without a driver and fails only when a kernel is actually launched), argument checks, and the
// per-device status word every kernel reports bounded-wait timeouts into.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/spinf_b200.h"

namespace spinf {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn();

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements with a row pitch of `pitch_bytes`; box = box_cols x box_rows,
// 128-byte swizzle (box_cols * elem_bytes must be 128). Returns 0 or SPINF_ERR_TENSORMAP.
int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows);
// 2-D row-major byte tensor [rows, cols] without swizzle: box = box_cols x box_rows bytes (box_cols a multiple of 16).
int make_tmap_2d_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                       uint32_t box_rows);
// 3-D tensor [d2, d1, d0] (d0 innermost) with byte strides s1 (between d1 steps) and s2; box = b0 x b1 x 1, 128-byte swizzle.
int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1);

// One int of device memory per device holding the first error a kernel recorded (0 = none). Allocated on first use.
int* status_word(int device);
// Copies the status word back (synchronises the stream), clears it, and returns it as a positive error code.
int read_and_clear_status(cudaStream_t stream);

int sm_count();

#define SPINF_CHECK_ARG(cond)                  \
  do {                                         \
    if (!(cond)) return SPINF_ERR_BAD_ARGUMENT; \
  } while (0)

#define SPINF_CUDA_OK(expr)                         \
  do {                                              \
    cudaError_t _e = (expr);                        \
    if (_e != cudaSuccess) return SPINF_ERR_CUDA;   \
  } while (0)

}  // namespace spinf
