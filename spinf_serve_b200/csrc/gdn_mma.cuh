// Warp-level bf16 MMA helpers (mma.sync m16n8k16 + ldmatrix) shared by the Gated DeltaNet chunk kernels: fragment loaders for
// row-major bf16 tiles in shared memory and the tile loader that brings 64 rows of 128 values in with cp.async.
#pragma once
#include "common.cuh"

namespace spinf {

static constexpr int CK = 128;   // key / value head dimension (state is CK x CK)
static constexpr int CT = 64;    // chunk length
static constexpr int LD = CK + 8;  // shared-memory row stride in bf16: 272 bytes, rows shift by one 16-byte bank group
static constexpr float RCP_LN2 = 1.4426950408889634f;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
// D (16 x 8, fp32) += A (16 x 16, bf16, row) * B (16 x 8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Fragment addresses inside a row-major bf16 tile with row stride LD (lane = lane of the warp):
//   A operand, 16 x 16 block at (r0, c0) of a matrix stored [m][k]
__device__ __forceinline__ const __nv_bfloat16* frag_a(const __nv_bfloat16* m, int ld, int r0, int c0, int lane) {
  return m + (r0 + (lane & 15)) * ld + c0 + (lane >> 4) * 8;
}
//   A operand from a matrix stored transposed, [k][m] (ldmatrix.trans): block rows k0.., columns m0..
__device__ __forceinline__ const __nv_bfloat16* frag_a_t(const __nv_bfloat16* m, int ld, int k0, int m0, int lane) {
  return m + (k0 + (lane & 7) + (lane >> 4) * 8) * ld + m0 + ((lane >> 3) & 1) * 8;
}
//   B operand for two n-tiles (n0.. n0+15) from a matrix stored [n][k] (the K^T pattern): r[0..1] = tile n0, r[2..3] = tile n0 + 8
__device__ __forceinline__ const __nv_bfloat16* frag_b(const __nv_bfloat16* m, int ld, int n0, int k0, int lane) {
  return m + (n0 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8;
}
//   B operand for two n-tiles from a matrix stored [k][n] (ldmatrix.trans): r[0..1] = tile n0, r[2..3] = tile n0 + 8
__device__ __forceinline__ const __nv_bfloat16* frag_b_t(const __nv_bfloat16* m, int ld, int k0, int n0, int lane) {
  return m + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n0 + (lane >> 4) * 8;
}

// rows of a [CT x CK] bf16 tile from global rows src(t) (nullptr: zero row): every copy of the tile is in flight at once
template <class RowPtr>
__device__ __forceinline__ void load_tile(__nv_bfloat16* dst, RowPtr src, const __nv_bfloat16* any_valid, int tid, int nthreads) {
  for (int i = tid; i < CT * (CK / 8); i += nthreads) {
    const int t = i / (CK / 8), c = i % (CK / 8);
    const __nv_bfloat16* p = src(t);
    cp_async16(dst + t * LD + c * 8, p ? p + c * 8 : any_valid, p ? 16 : 0);
  }
}

}  // namespace spinf
