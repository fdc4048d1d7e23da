// Launchers of the tcgen05 GEMMs: the row-wise fp8 linear, the plain bf16 linear and the fused option-log-prob read.
#include <atomic>
#include <mutex>

#include "gemm_tc.cuh"
#include "host_util.h"

namespace spinf {

// ------------------------------------------------------------------------------------------------ option log-prob epilogue
// Per accumulator tile (128 read rows x 256 vocabulary columns) every thread keeps the running maximum and sum of exponentials
// of its row, writes them to part_max/part_sum[tile_n][row], and copies the (soft-capped) logits of the option columns that fall
// inside the tile to `out`. lse_finalize_kernel then merges the per-tile partials in ascending tile order.
template <int BN>
struct EpiLse {
  static constexpr bool kReadsTmemInEnd = true;
  float softcap;
  float* part_max;  // [tiles_n, Mpad]
  float* part_sum;  // [tiles_n, Mpad]
  int Mpad;
  const int* cols;            // sorted distinct option token ids
  const int* col_tile_start;  // [tiles_n + 1]: cols[col_tile_start[t] .. col_tile_start[t+1]) lie in vocabulary tile t
  float* out;                 // [M, n_cols]
  int n_cols;
  struct State {
    float m, s;
  };

  __device__ __forceinline__ float cap(float v) const { return softcap > 0.f ? softcap * tanhf(v / softcap) : v; }

  __device__ __forceinline__ void begin_tile(State& st, const GemmShape&, int, int, int, float*) const {
    st.m = -INFINITY;
    st.s = 0.f;
  }
  __device__ __forceinline__ void chunk(State& st, const GemmShape& s, int tm, int tn, int row, int et, int c,
                                        const uint32_t (&v0)[32], const uint32_t (&v1)[32], const float*, uint8_t*, uint32_t) const {
    const int n0 = tn * BN + c * 64;
    float x[64];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      x[i] = n0 + i < s.N ? cap(__uint_as_float(v0[i])) : -INFINITY;
      x[32 + i] = n0 + 32 + i < s.N ? cap(__uint_as_float(v1[i])) : -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < 64; ++i) mx = fmaxf(mx, x[i]);
    const float m_new = fmaxf(st.m, mx);
    if (m_new == -INFINITY) return;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) acc += __expf(x[i] - m_new);
    st.s = st.s * __expf(st.m - m_new) + acc;
    st.m = m_new;
  }
  __device__ __forceinline__ void end_tile(State& st, const GemmShape& s, int tm, int tn, int row, int et, uint32_t t_row,
                                           const float*) const {
    const int m = tm * 128 + row;
    part_max[static_cast<size_t>(tn) * Mpad + m] = st.m;
    part_sum[static_cast<size_t>(tn) * Mpad + m] = st.s;
    const int c0 = col_tile_start[tn], c1 = col_tile_start[tn + 1];
    for (int ci = c0; ci < c1; ++ci) {  // uniform across the CTA
      const int col = cols[ci] - tn * BN;
      if (col < 0 || col >= BN) continue;  // malformed column table: skip, never index outside the accumulator
      uint32_t r;
      tmem_ld_x1(t_row + col, r);
      tmem_wait_ld();
      if (m < s.M) out[static_cast<size_t>(m) * n_cols + ci] = cap(__uint_as_float(r));
    }
  }
  __device__ __forceinline__ void finish(State&, int) const {}
};

// ------------------------------------------------------------------------------------------------ gated-activation epilogue
// The gate|up projection with the activation fused: the weight rows are laid out (at load time) so that every 64-column chunk
// of an accumulator tile holds 32 gate channels followed by the 32 up channels of the same features; tile tn covers features
// [128 tn, 128 tn + 128). Per element: gate = bf16((acc rs) cs), up likewise (the linear's own bf16 outputs), then
// y = bf16(bf16(act(gate)) up), written as bf16 [M, F]; the row maximum of |y| is merged into row_amax with an integer atomic
// max (non-negative floats order like their bit patterns, so the result does not depend on tile order).
template <int BN, int ACT>
struct EpiGlu {
  static constexpr bool kReadsTmemInEnd = false;
  CUtensorMap tmC;  // y [M, F] bf16, box 64 x 128, 128-byte swizzle
  const float* rowscale;
  const float* colscale_g;  // [2F] in the tiled channel order
  float* row_amax;          // [M], zeroed before the launch
  struct State {
    uint32_t nstores;
    uint32_t amax2;  // running maxima of |y| as a packed bf16 pair (even / odd columns)
  };
  __device__ __forceinline__ static float act(float x) {
    if (ACT == 0) return gelu_tanh_f32(x);
    return silu_f32(x);
  }
  __device__ __forceinline__ void begin_tile(State& st, const GemmShape& s, int tm, int tn, int et, float* colscale) const {
    named_bar_sync(2, 128);
    for (int i = et; i < BN; i += 128) {
      const int n = tn * BN + i;
      colscale[i] = n < s.N ? colscale_g[n] : 0.f;
    }
    named_bar_sync(2, 128);
    st.amax2 = 0u;
  }
  __device__ __forceinline__ void chunk(State& st, const GemmShape& s, int tm, int tn, int row, int et, int c,
                                        const uint32_t (&v0)[32], const uint32_t (&v1)[32], const float* colscale,
                                        uint8_t* epi_stage, uint32_t) const {
    const int m = tm * 128 + row;
    const float rs = m < s.M ? rowscale[m] : 0.f;
    // packed pairs throughout: the linear's bf16 outputs come out of the pack conversion, the gated product is one bf16x2 multiply
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 cg = *reinterpret_cast<const float2*>(colscale + c * 64 + 2 * i);
      const float2 cu = *reinterpret_cast<const float2*>(colscale + c * 64 + 32 + 2 * i);
      const uint32_t g = pack_bf16x2((__uint_as_float(v0[2 * i]) * rs) * cg.x, (__uint_as_float(v0[2 * i + 1]) * rs) * cg.y);
      const uint32_t u = pack_bf16x2((__uint_as_float(v1[2 * i]) * rs) * cu.x, (__uint_as_float(v1[2 * i + 1]) * rs) * cu.y);
      const uint32_t a = pack_bf16x2(act(bf2_lo(g)), act(bf2_hi(g)));
      packed[i] = bf2_mul(a, u);
      st.amax2 = bf2_max(st.amax2, packed[i] & 0x7fff7fffu);
    }
    uint8_t* buf = epi_stage + (st.nstores & 1u) * (128 * 128);
    if ((c & 1) == 0) {
      if (et == 0) tma_store_wait_read<1>();
      named_bar_sync(1, 128);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(buf + sw128_offset(row, (c & 1) * 4 + j)) =
          make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    if (c & 1) {
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (et == 0) {
        tma_store_2d(&tmC, buf, tn * (BN / 2) + (c >> 1) * 64, tm * 128);
        tma_store_commit();
      }
      ++st.nstores;
    }
  }
  __device__ __forceinline__ void end_tile(State& st, const GemmShape& s, int tm, int, int row, int, uint32_t, const float*) const {
    const int m = tm * 128 + row;
    if (m < s.M) atomicMax(reinterpret_cast<unsigned int*>(row_amax + m), __float_as_uint(fmaxf(bf2_lo(st.amax2), bf2_hi(st.amax2))));
  }
  __device__ __forceinline__ void finish(State&, int et) const {
    if (et == 0) tma_store_wait_all<0>();
  }
};

// ------------------------------------------------------------------------------------------------ q|k|v projection epilogue
// The fused q|k|v projection with the per-head RMS norms and the rotary embedding applied before the tile leaves the SM. A
// 128 x 256 accumulator tile holds whole heads (one of 256 dims, or two of 128), and an epilogue thread owns a full row of it, so
// the head's sum of squares is thread-local. Pass 1 (chunk) rounds the linear's outputs y = bf16((acc * xs) * ws) as packed pairs,
// accumulates their squares and parks the pairs in the accumulator's own TMEM columns (pair word q of the row in column q: always
// behind the columns still to be read). Pass 2 (end_tile) reads the pairs back 16 words at a time, the group D/2 columns further
// along with them, and applies
//     x = bf16(y * rsqrt(mean y^2 + eps) * w)        (q with wq, k with wk, v without weight)
//     out = bf16(bf16(x cos) + bf16(rotate_half(x) sin))      (q and k only; packed bf16 multiplies and adds)
// before writing bf16 rows straight to global memory. Same rounding chain as the row-wise GEMM followed by the norm + rotary kernel.
template <int BN, int D>
struct EpiQkvNormRope {
  static constexpr bool kReadsTmemInEnd = true;
  static constexpr int HEADS = BN / D;
  __nv_bfloat16* y;
  int64_t y_pitch;
  const float* rowscale;
  const float* colscale_g;
  const __nv_bfloat16 *wq, *wk, *cos_t, *sin_t;  // cos / sin [M, D/2]
  int H, Hkv;
  float eps;
  int plus1, norm_v;
  struct State {
    float ss[HEADS];
  };
  __device__ __forceinline__ static float inv_sqrt(float v) {
    const float r = rsqrtf(v);
    return r * fmaf(-0.5f * v * r, r, 1.5f);
  }
  __device__ __forceinline__ void begin_tile(State& st, const GemmShape& s, int tm, int tn, int et, float* colscale) const {
    named_bar_sync(2, 128);
    for (int i = et; i < BN; i += 128) {
      const int n = tn * BN + i;
      colscale[i] = n < s.N ? colscale_g[n] : 0.f;
    }
    named_bar_sync(2, 128);
#pragma unroll
    for (int h = 0; h < HEADS; ++h) st.ss[h] = 0.f;
  }
  __device__ __forceinline__ void chunk(State& st, const GemmShape& s, int tm, int tn, int row, int et, int c,
                                        const uint32_t (&v0)[32], const uint32_t (&v1)[32], const float* colscale, uint8_t*,
                                        uint32_t t_row) const {
    const int m = tm * 128 + row;
    const float rs = m < s.M ? rowscale[m] : 0.f;
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t pk[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 c0 = *reinterpret_cast<const float2*>(colscale + c * 64 + 2 * j);
      const float2 c1 = *reinterpret_cast<const float2*>(colscale + c * 64 + 32 + 2 * j);
      pk[j] = pack_bf16x2((__uint_as_float(v0[2 * j]) * rs) * c0.x, (__uint_as_float(v0[2 * j + 1]) * rs) * c0.y);
      pk[16 + j] = pack_bf16x2((__uint_as_float(v1[2 * j]) * rs) * c1.x, (__uint_as_float(v1[2 * j + 1]) * rs) * c1.y);
      acc0 = fmaf(bf2_lo(pk[j]), bf2_lo(pk[j]), acc0);
      acc1 = fmaf(bf2_hi(pk[j]), bf2_hi(pk[j]), acc1);
      acc0 = fmaf(bf2_lo(pk[16 + j]), bf2_lo(pk[16 + j]), acc0);
      acc1 = fmaf(bf2_hi(pk[16 + j]), bf2_hi(pk[16 + j]), acc1);
    }
    __syncwarp();
    tmem_st_x32(t_row + c * 32, pk);
#pragma unroll
    for (int h = 0; h < HEADS; ++h)
      if ((c * 64) / D == h) st.ss[h] += acc0 + acc1;
  }
  // 32 columns [col_lo, col_lo + 32) of this thread's row with the 32 columns D/2 further along. MODE is a compile-time constant so
  // that the block is straight-line code: 0 = q / k (norm weight + rotary), 1 = v with the weightless norm, 2 = v untouched.
  template <int MODE>
  __device__ __forceinline__ void granule_pair(uint32_t t_row, int col_lo, float inv, float p1, const __nv_bfloat16* w_lo,
                                               const __nv_bfloat16* cs_row, const __nv_bfloat16* sn_row, __nv_bfloat16* dst,
                                               bool live) const {
    const int col_hi = col_lo + D / 2;
    uint32_t a0[16], a1[16];
    __syncwarp();
    tmem_ld_x16(t_row + col_lo / 2, a0);
    tmem_ld_x16(t_row + col_hi / 2, a1);
    // 32 consecutive table / weight entries as two 32-byte loads each, issued while the TMEM load is in flight
    uint32_t cv[2][8], sv[2][8], wl[2][8], wh[2][8];
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        ldg_nc_v8(cs_row + i * 16, cv[i]);
        ldg_nc_v8(sn_row + i * 16, sv[i]);
        ldg_nc_v8(w_lo + i * 16, wl[i]);
        ldg_nc_v8(w_lo + D / 2 + i * 16, wh[i]);
      }
    }
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t out_lo[8], out_hi[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        uint32_t xl = a0[i * 8 + p], xh = a1[i * 8 + p];
        if (MODE == 0) {
          xl = pack_bf16x2(bf2_lo(xl) * inv * (bf2_lo(wl[i][p]) + p1), bf2_hi(xl) * inv * (bf2_hi(wl[i][p]) + p1));
          xh = pack_bf16x2(bf2_lo(xh) * inv * (bf2_lo(wh[i][p]) + p1), bf2_hi(xh) * inv * (bf2_hi(wh[i][p]) + p1));
          out_lo[p] = bf2_sub(bf2_mul(xl, cv[i][p]), bf2_mul(xh, sv[i][p]));
          out_hi[p] = bf2_add(bf2_mul(xh, cv[i][p]), bf2_mul(xl, sv[i][p]));
        } else if (MODE == 1) {
          out_lo[p] = pack_bf16x2(bf2_lo(xl) * inv, bf2_hi(xl) * inv);
          out_hi[p] = pack_bf16x2(bf2_lo(xh) * inv, bf2_hi(xh) * inv);
        } else {
          out_lo[p] = xl, out_hi[p] = xh;
        }
      }
      if (live) {
        stg_v8(dst + col_lo + i * 16, out_lo);
        stg_v8(dst + col_hi + i * 16, out_hi);
      }
    }
  }
  __device__ __forceinline__ void end_tile(State& st, const GemmShape& s, int tm, int tn, int row, int et, uint32_t t_row,
                                           const float* colscale) const {
    constexpr int HALF = D / 64;  // 32-column granules per half head
    const int m = tm * 128 + row;
    const bool live = m < s.M;
    const int64_t mrow = live ? m : 0;
    __nv_bfloat16* dst = y + mrow * y_pitch + static_cast<int64_t>(tn) * BN;
    const float p1 = plus1 ? 1.f : 0.f;  // w + 0 == w for every bf16 weight that is not -0
    tmem_wait_st();                      // the pairs parked by pass 1 are in place
#pragma unroll 1
    for (int hl = 0; hl < HEADS; ++hl) {
      const int hg = tn * HEADS + hl;  // head index in the fused projection: q heads, then k heads, then v heads
      const int mode = hg < H + Hkv ? 0 : (norm_v ? 1 : 2);
      const float inv = mode == 2 ? 1.f : inv_sqrt(st.ss[hl] / D + eps);
      const __nv_bfloat16* w = hg < H ? wq : wk;
#pragma unroll 1
      for (int gi = 0; gi < HALF; ++gi) {
        const int col_lo = hl * D + gi * 32;
        const __nv_bfloat16* cs_row = cos_t + mrow * (D / 2) + gi * 32;
        const __nv_bfloat16* sn_row = sin_t + mrow * (D / 2) + gi * 32;
        if (mode == 0)
          granule_pair<0>(t_row, col_lo, inv, p1, w + gi * 32, cs_row, sn_row, dst, live);
        else if (mode == 1)
          granule_pair<1>(t_row, col_lo, inv, p1, w, cs_row, sn_row, dst, live);
        else
          granule_pair<2>(t_row, col_lo, inv, p1, w, cs_row, sn_row, dst, live);
      }
    }
  }
  __device__ __forceinline__ void finish(State&, int) const {}
};

// x8 = e4m3(clamp(y / s)), s = max(amax, 1e-12) / 448 with the row maxima already known: one pass over y
__global__ void __launch_bounds__(256) fp8_quant_from_amax_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ row_amax,
                                                                  int K, uint8_t* __restrict__ x8, float* __restrict__ xs) {
  const size_t row = blockIdx.x;
  const float s = __fdiv_rn(fmaxf(row_amax[row], 1e-12f), 448.f);
  if (threadIdx.x == 0) xs[row] = s;
  const DivBy div = make_div_by(s);
  const uint4* src = reinterpret_cast<const uint4*>(y + row * K);
  uint2* dst = reinterpret_cast<uint2*>(x8 + row * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float2 a = __bfloat1622float2(p[2 * j]), b = __bfloat1622float2(p[2 * j + 1]);
      // no explicit clamp: |x / s| can exceed 448 only by rounding, and the conversion saturates
      const float q0 = div_by(div, a.x), q1 = div_by(div, a.y), q2 = div_by(div, b.x), q3 = div_by(div, b.y);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
      o[j] = lo | (hi << 16);
    }
    dst[i] = make_uint2(o[0], o[1]);
  }
}

// start[t] = index of the first option column >= t * BN (cols ascending), t = 0..tiles_n
__global__ void col_tile_start_kernel(const int* __restrict__ cols, int n_cols, int tiles_n, int BN, int* __restrict__ start) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > tiles_n) return;
  const long long key = static_cast<long long>(t) * BN;
  int lo = 0, hi = n_cols;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (cols[mid] < key) lo = mid + 1; else hi = mid;
  }
  start[t] = lo;
}

// One CTA per read row: thread i merges the partials of vocabulary tiles i, i + 128, ... in ascending order, the 128 running
// (max, sum) pairs are merged by a fixed tree (shuffles, then the four warps' results in order), and the whole CTA subtracts the
// row's log-sum-exp from its option logits. The order depends on the number of tiles only, never on the number of rows.
__device__ __forceinline__ void lse_merge(float& m, float& s, float pm, float ps) {
  const float mn = fmaxf(m, pm);
  if (mn == -INFINITY) return;
  s = s * __expf(m - mn) + ps * __expf(pm - mn);
  m = mn;
}
__global__ void __launch_bounds__(128) lse_finalize_kernel(const float* __restrict__ part_max, const float* __restrict__ part_sum,
                                                           int tiles_n, int Mpad, int M, float* __restrict__ out, int n_cols) {
  __shared__ float red_m[4], red_s[4];
  const int r = blockIdx.x;
  float m = -INFINITY, s = 0.f;
  for (int t = threadIdx.x; t < tiles_n; t += 128)
    lse_merge(m, s, part_max[static_cast<size_t>(t) * Mpad + r], part_sum[static_cast<size_t>(t) * Mpad + r]);
  for (int o = 1; o < 32; o <<= 1) {
    const float pm = __shfl_xor_sync(0xffffffffu, m, o), ps = __shfl_xor_sync(0xffffffffu, s, o);
    // both partners must arrive at the same pair: the lower lane's value goes first
    float a_m = (threadIdx.x & o) ? pm : m, a_s = (threadIdx.x & o) ? ps : s;
    const float b_m = (threadIdx.x & o) ? m : pm, b_s = (threadIdx.x & o) ? s : ps;
    lse_merge(a_m, a_s, b_m, b_s);
    m = a_m, s = a_s;
  }
  if ((threadIdx.x & 31) == 0) red_m[threadIdx.x >> 5] = m, red_s[threadIdx.x >> 5] = s;
  __syncthreads();
  m = red_m[0], s = red_s[0];
  for (int w = 1; w < 4; ++w) lse_merge(m, s, red_m[w], red_s[w]);
  const float lse = m + logf(s);
  for (int c = threadIdx.x; c < n_cols; c += 128) out[static_cast<size_t>(r) * n_cols + c] -= lse;
}

// ------------------------------------------------------------------------------------------------ per-row fp8 quantiser
// One CTA per row: amax over the row in fp32, then x / s (a true division, as the reference computes it), clamped and cast to e4m3
// with round-to-nearest-even.
// INT8: the int8 scheme's quantiser instead (quant_act_int8): s = amax / 127, round(x / s) to the nearest integer (ties to even),
// clamped to +-127.
template <bool INT8>
__global__ void __launch_bounds__(256) fp8_rowwise_quant_kernel(const __nv_bfloat16* __restrict__ x, int K, uint8_t* __restrict__ x8,
                                                                float* __restrict__ xs) {
  const size_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * K);
  const int nvec = K / 8;
  __shared__ float red[8];
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(p[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float s = __fdiv_rn(fmaxf(amax, 1e-12f), INT8 ? 127.f : 448.f);
  if (threadIdx.x == 0) xs[row] = s;
  const DivBy div = make_div_by(s);
  uint2* dst = reinterpret_cast<uint2*>(x8 + row * K);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float2 a = __bfloat1622float2(p[2 * j]), b = __bfloat1622float2(p[2 * j + 1]);
      // no explicit clamp: |x / s| can exceed 448 only by rounding, and the conversion saturates
      const float q0 = div_by(div, a.x), q1 = div_by(div, a.y), q2 = div_by(div, b.x), q3 = div_by(div, b.y);
      if (INT8) {
        auto r8 = [](float q) { return static_cast<uint32_t>(max(-127, min(127, __float2int_rn(q)))) & 0xffu; };
        o[j] = r8(q0) | (r8(q1) << 8) | (r8(q2) << 16) | (r8(q3) << 24);
      } else {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
        o[j] = lo | (hi << 16);
      }
    }
    dst[i] = make_uint2(o[0], o[1]);
  }
}

// ------------------------------------------------------------------------------------------------ per-tensor fp8 quantiser
// max |x| over a whole tensor (bf16, n a multiple of 8): the reduction of the dynamic per-tensor scheme. Non-negative floats order
// like their bit patterns, so the grid's maxima meet in one integer atomic; *out is zeroed by the caller.
__global__ void __launch_bounds__(256) abs_max_kernel(const __nv_bfloat16* __restrict__ x, int64_t nvec, float* __restrict__ out) {
  const uint4* src = reinterpret_cast<const uint4*>(x);
  __shared__ float red[8];
  float amax = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(amax));
  }
}

// x8 = e4m3(clamp(x / s)) with one scale for the tensor, read from device memory: s = *scale (the static scheme), or
// s = max(*scale, 1e-12) / 448 with *scale the tensor's max |x| (the dynamic scheme). scale_out (optional) receives s.
// peak (optional): *peak = max(*peak, max|x| / (s * 448)), the clipping monitor of the static scheme.
__global__ void __launch_bounds__(256) fp8_tensor_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t nvec,
                                                               const float* __restrict__ scale, int from_amax,
                                                               uint8_t* __restrict__ x8, float* __restrict__ scale_out,
                                                               float* __restrict__ peak) {
  const float s = from_amax ? __fdiv_rn(fmaxf(*scale, 1e-12f), 448.f) : *scale;
  if (scale_out && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = s;
  const DivBy div = make_div_by(s);
  const uint4* src = reinterpret_cast<const uint4*>(x);
  uint2* dst = reinterpret_cast<uint2*>(x8);
  float amax = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float2 a = __bfloat1622float2(p[2 * j]), b = __bfloat1622float2(p[2 * j + 1]);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
      // a true division, as the reference computes it; the conversion saturates at +-448 (the reference's clamp)
      const float q0 = div_by(div, a.x), q1 = div_by(div, a.y), q2 = div_by(div, b.x), q3 = div_by(div, b.y);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
      o[j] = lo | (hi << 16);
    }
    dst[i] = make_uint2(o[0], o[1]);
  }
  if (peak) {
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
      for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
      atomicMax(reinterpret_cast<unsigned int*>(peak), __float_as_uint(__fdiv_rn(amax, s * 448.f)));
    }
  }
}

// ------------------------------------------------------------------------------------------------ launch helpers
template <int KIND, int BN, class Epi>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmShape& shape, const Epi& epi, cudaStream_t stream) {
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  auto kern = gemm_tc_kernel<KIND, BN, Epi>;
  static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice from two threads is harmless
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int tiles = shape.tiles_m * shape.tiles_n * (EpiSplitK<Epi>::value ? shape.splits : 1);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 192, GemmSmem<BN>::TOTAL, stream>>>(tmA, tmB, shape, epi, status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

static GemmShape make_shape(int64_t M, int64_t N, int64_t K, int BN, int elem_bytes = 1) {
  GemmShape s;
  s.M = static_cast<int>(M);
  s.N = static_cast<int>(N);
  s.K = static_cast<int>(K);
  s.tiles_m = static_cast<int>((M + 127) / 128);
  s.tiles_n = static_cast<int>((N + BN - 1) / BN);
  // Row tiles are walked in groups, all column tiles of a group before the next group: the group's activation rows stay in L2
  // while the weight matrix streams past once per group. The group is made as tall as about 32 MB of activations allow (8..64
  // row tiles): with 8, the 118 MB gate|up weight of the 12B shapes crossed HBM 27 times per GEMM; the traffic costs power, and
  // under the power cap power is time (2.52 -> 2.36 ms on that GEMM at 27 648 rows). The order changes no tile's arithmetic.
  const int64_t per_tile = 128 * K * elem_bytes;
  const int64_t g = (32ll << 20) / (per_tile > 0 ? per_tile : 1);
  s.group_m = static_cast<int>(g < 8 ? 8 : (g > 64 ? 64 : g));
  s.splits = 1;
  s.kb_per = 0;
  return s;
}

// K slices of the few-row fp8 linear: as many as put one (128-column tile, slice) unit on every SM, each at least 24 K blocks
// (3 072 elements) long: below that the second launch costs what the slices save (measured inside a CUDA graph at 120 rows:
// 3 840 x 15 360 38.7 -> 20.4 us in four slices, 3 840 x 4 096 13.8 -> 14.2 us). A function of N and K only.
static int fp8_small_splits(int64_t N, int64_t K, int* kb_per_out) {
  const int tiles_n = static_cast<int>((N + 127) / 128), num_kb = static_cast<int>((K + 127) / 128);
  int s = sm_count() / tiles_n;
  s = s > num_kb / 24 ? num_kb / 24 : s;
  s = s > 16 ? 16 : s;
  if (s < 2) {
    *kb_per_out = num_kb;
    return 1;
  }
  const int kb_per = (num_kb + s - 1) / s;
  *kb_per_out = kb_per;
  return (num_kb + kb_per - 1) / kb_per;
}

// y[m, n] = bf16((sum over slices, in slice order, of part[s][m][n]) * xs[m] * ws[n]), four columns per thread
__global__ void __launch_bounds__(256) fp8_small_sum_kernel(const float* __restrict__ part, int splits, int M, int N,
                                                            const float* __restrict__ xs, const float* __restrict__ ws,
                                                            __nv_bfloat16* __restrict__ y) {
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const int64_t MN = static_cast<int64_t>(M) * N;
  if (i >= MN) return;
  float4 acc = *reinterpret_cast<const float4*>(part + i);
  for (int k = 1; k < splits; ++k) {
    const float4 p = *reinterpret_cast<const float4*>(part + k * MN + i);
    acc.x += p.x, acc.y += p.y, acc.z += p.z, acc.w += p.w;
  }
  const int m = static_cast<int>(i / N), n = static_cast<int>(i % N);
  const float rs = xs[m];
  const float4 cs = *reinterpret_cast<const float4*>(ws + n);
  uint2 out;
  out.x = pack_bf16x2((acc.x * rs) * cs.x, (acc.y * rs) * cs.y);
  out.y = pack_bf16x2((acc.z * rs) * cs.z, (acc.w * rs) * cs.w);
  *reinterpret_cast<uint2*>(y + i) = out;
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_fp8_rowwise_quant(const void* x_bf16, int64_t M, int64_t K, void* x8, float* xs, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x_bf16 && x8 && xs && M >= 0 && K > 0 && K % 8 == 0 && K <= 32768 && M < (1ll << 31));
  fp8_rowwise_quant_kernel<false><<<static_cast<unsigned>(M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), static_cast<int>(K), static_cast<uint8_t*>(x8), xs);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_int8_rowwise_quant(const void* x_bf16, int64_t M, int64_t K, void* x8, float* xs, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x_bf16 && x8 && xs && M >= 0 && K > 0 && K % 8 == 0 && K <= 32768 && M < (1ll << 31));
  fp8_rowwise_quant_kernel<true><<<static_cast<unsigned>(M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), static_cast<int>(K), static_cast<uint8_t*>(x8), xs);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_int8_rowwise_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M,
                                       int64_t N, int64_t K, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x8 && xs && w8 && ws && y_bf16 && M >= 0 && N > 0 && K > 0 && K % 16 == 0 && N % 16 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  EpiStoreBf16<BN, true, true> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, N, K, K, 128, BN))) return r;
  if ((r = make_tmap_2d(&epi.tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_bf16, M, N, N * 2, 64, 128))) return r;
  epi.rowscale = xs;
  epi.colscale_g = ws;
  return launch_gemm<KIND_S8, BN>(tmA, tmB, make_shape(M, N, K, BN), epi, static_cast<cudaStream_t>(stream));
}

template <int BN>
static int fp8_rowwise_gemm_bn(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M, int64_t N, int64_t K,
                               void* stream) {
  CUtensorMap tmA, tmB;
  EpiStoreBf16<BN, true> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, N, K, K, 128, BN))) return r;
  if ((r = make_tmap_2d(&epi.tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_bf16, M, N, N * 2, 64, 128))) return r;
  epi.rowscale = xs;
  epi.colscale_g = ws;
  return launch_gemm<KIND_F8, BN>(tmA, tmB, make_shape(M, N, K, BN), epi, static_cast<cudaStream_t>(stream));
}

extern "C" int spinf_fp8_rowwise_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M,
                                      int64_t N, int64_t K, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x8 && xs && w8 && ws && y_bf16 && M >= 0 && N > 0 && K > 0 && K % 16 == 0 && N % 16 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  // a decoding step's few rows: one row tile, so the column tiles are all the parallelism there is; narrower tiles put the weight
  // stream on twice as many SMs (the same sums in the same order: a tile's width changes no element)
  if (M <= 128 && N / 256 < sm_count()) return fp8_rowwise_gemm_bn<128>(x8, xs, w8, ws, y_bf16, M, N, K, stream);
  return fp8_rowwise_gemm_bn<256>(x8, xs, w8, ws, y_bf16, M, N, K, stream);
}

// bytes of workspace spinf_fp8_rowwise_gemm_small needs (0: the shape runs unsplit)
extern "C" int64_t spinf_fp8_rowwise_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || M > 128 || N <= 0 || K <= 0) return 0;
  int kb_per;
  const int s = spinf::fp8_small_splits(N, K, &kb_per);
  return s > 1 ? static_cast<int64_t>(s) * M * N * 4 : 0;
}

// spinf_fp8_rowwise_gemm for a decoding step's few rows (M <= 128): the K dimension is cut into slices so that every SM streams
// weights; fp32 partial sums go to `workspace`, a second kernel adds them in slice order and applies the scales. Differs from
// spinf_fp8_rowwise_gemm in the order of the fp32 sum only. More rows, or a shape that needs no split, run the plain kernel.
extern "C" int spinf_fp8_rowwise_gemm_small(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M,
                                            int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace spinf;
  if (M == 0) return 0;
  const int64_t need = spinf_fp8_rowwise_gemm_small_workspace_bytes(M, N, K);
  if (need == 0) return spinf_fp8_rowwise_gemm(x8, xs, w8, ws, y_bf16, M, N, K, stream);
  SPINF_CHECK_ARG(x8 && xs && w8 && ws && y_bf16 && K % 16 == 0 && N % 16 == 0 && N < (1ll << 31) && K < (1ll << 31));
  SPINF_CHECK_ARG(workspace && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 16 == 0);
  SPINF_CHECK_ARG(reinterpret_cast<uintptr_t>(ws) % 16 == 0);
  constexpr int BN = 128;
  CUtensorMap tmA, tmB;
  EpiPartial<BN> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, N, K, K, 128, BN))) return r;
  epi.part = static_cast<float*>(workspace);
  GemmShape shape = make_shape(M, N, K, BN);
  shape.splits = fp8_small_splits(N, K, &shape.kb_per);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((r = launch_gemm<KIND_F8, BN>(tmA, tmB, shape, epi, st))) return r;
  const int64_t quads = M * N / 4;
  fp8_small_sum_kernel<<<static_cast<unsigned>((quads + 255) / 256), 256, 0, st>>>(epi.part, shape.splits, static_cast<int>(M),
                                                                                   static_cast<int>(N), xs, ws,
                                                                                   static_cast<__nv_bfloat16*>(y_bf16));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_abs_max(const void* x_bf16, int64_t n, float* out, void* stream) {
  if (n == 0) {  // the maximum over nothing is 0: the output is still written (the input pointer may be null)
    SPINF_CHECK_ARG(out);
    SPINF_CUDA_OK(cudaMemsetAsync(out, 0, sizeof(float), static_cast<cudaStream_t>(stream)));
    return 0;
  }
  SPINF_CHECK_ARG(x_bf16 && out && n >= 0 && n % 8 == 0);
  SPINF_CUDA_OK(cudaMemsetAsync(out, 0, sizeof(float), static_cast<cudaStream_t>(stream)));
  const int64_t nvec = n / 8, blocks = (nvec + 255) / 256;
  const int64_t cap = 8ll * sm_count();
  abs_max_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), nvec, out);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_fp8_tensor_quant(const void* x_bf16, int64_t n, const float* scale, int32_t from_amax, void* x8, float* scale_out,
                                      float* peak, void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x_bf16 && scale && x8 && n >= 0 && n % 8 == 0 && (from_amax == 0 || from_amax == 1));
  const int64_t nvec = n / 8, blocks = (nvec + 255) / 256;
  const int64_t cap = 8ll * sm_count();
  fp8_tensor_quant_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), nvec, scale, from_amax, static_cast<uint8_t*>(x8), scale_out, peak);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_fp8_tensor_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M,
                                     int64_t N, int64_t K, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x8 && xs && w8 && ws && y_bf16 && M >= 0 && N > 0 && K > 0 && K % 16 == 0 && N % 16 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  EpiStoreBf16<BN, true> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, N, K, K, 128, BN))) return r;
  if ((r = make_tmap_2d(&epi.tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_bf16, M, N, N * 2, 64, 128))) return r;
  epi.rowscale = xs;
  epi.colscale_g = ws;
  epi.rowscale_stride = 0;
  epi.colscale_stride = 0;
  return launch_gemm<KIND_F8, BN>(tmA, tmB, make_shape(M, N, K, BN), epi, static_cast<cudaStream_t>(stream));
}

extern "C" int spinf_bf16_gemm_ld(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t y_pitch, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x && w && y && M >= 0 && N > 0 && K > 0 && K % 8 == 0 && N % 8 == 0 && y_pitch >= N && y_pitch % 8 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  EpiStoreBf16<BN, false> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, K * 2, 64, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, N, K, K * 2, 64, BN))) return r;
  if ((r = make_tmap_2d(&epi.tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, M, N, y_pitch * 2, 64, 128))) return r;
  epi.rowscale = nullptr;
  epi.colscale_g = nullptr;
  return launch_gemm<KIND_BF16, BN>(tmA, tmB, make_shape(M, N, K, BN, 2), epi, static_cast<cudaStream_t>(stream));
}

namespace spinf {
// K slices of the few-row bf16 product (a handful of un-quantised output channels beside a quantised linear: one or two column
// tiles whose serial K loop, not their bytes, is the cost): slices of at least 8 K blocks (512 elements), at most 16
static int bf16_small_splits(int64_t N, int64_t K, int* kb_per_out) {
  const int tiles_n = static_cast<int>((N + 127) / 128), num_kb = static_cast<int>((K + 63) / 64);
  int s = sm_count() / tiles_n;
  s = s > num_kb / 8 ? num_kb / 8 : s;
  s = s > 16 ? 16 : s;
  if (s < 2) {
    *kb_per_out = num_kb;
    return 1;
  }
  const int kb_per = (num_kb + s - 1) / s;
  *kb_per_out = kb_per;
  return (num_kb + kb_per - 1) / kb_per;
}

// y[m, n] = bf16(sum over slices, in slice order, of part[s][m][n]); y rows y_pitch elements apart
__global__ void __launch_bounds__(256) bf16_small_sum_kernel(const float* __restrict__ part, int splits, int M, int N,
                                                             __nv_bfloat16* __restrict__ y, int64_t y_pitch) {
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const int64_t MN = static_cast<int64_t>(M) * N;
  if (i >= MN) return;
  float4 acc = *reinterpret_cast<const float4*>(part + i);
  for (int k = 1; k < splits; ++k) {
    const float4 p = *reinterpret_cast<const float4*>(part + k * MN + i);
    acc.x += p.x, acc.y += p.y, acc.z += p.z, acc.w += p.w;
  }
  uint2 out;
  out.x = pack_bf16x2(acc.x, acc.y);
  out.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(y + (i / N) * y_pitch + i % N) = out;
}
}  // namespace spinf

extern "C" int64_t spinf_bf16_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || M > 128 || N <= 0 || K <= 0 || N % 4) return 0;
  int kb_per;
  const int s = spinf::bf16_small_splits(N, K, &kb_per);
  return s > 1 ? static_cast<int64_t>(s) * M * N * 4 : 0;
}

// spinf_bf16_gemm_ld for a decoding step's few rows (M <= 128) and few output channels: the K dimension in slices on separate
// CTAs, fp32 partial sums in `workspace` (16-byte aligned), added in slice order by a second launch. Differs from spinf_bf16_gemm_ld
// in the order of the fp32 sum only. A shape that needs no slices (workspace bytes 0) runs spinf_bf16_gemm_ld.
extern "C" int spinf_bf16_gemm_small(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t y_pitch, void* workspace,
                                     int64_t workspace_bytes, void* stream) {
  using namespace spinf;
  if (M == 0) return 0;
  const int64_t need = spinf_bf16_gemm_small_workspace_bytes(M, N, K);
  if (need == 0) return spinf_bf16_gemm_ld(x, w, y, M, N, K, y_pitch, stream);
  SPINF_CHECK_ARG(x && w && y && K % 8 == 0 && N % 8 == 0 && y_pitch >= N && y_pitch % 4 == 0 && N < (1ll << 31) && K < (1ll << 31));
  SPINF_CHECK_ARG(workspace && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 16 == 0);
  SPINF_CHECK_ARG(reinterpret_cast<uintptr_t>(y) % 8 == 0);
  constexpr int BN = 128;
  CUtensorMap tmA, tmB;
  EpiPartial<BN> epi;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, K * 2, 64, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, N, K, K * 2, 64, BN))) return r;
  epi.part = static_cast<float*>(workspace);
  GemmShape shape = make_shape(M, N, K, BN, 2);
  shape.splits = bf16_small_splits(N, K, &shape.kb_per);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((r = launch_gemm<KIND_BF16, BN>(tmA, tmB, shape, epi, st))) return r;
  const int64_t quads = M * N / 4;
  bf16_small_sum_kernel<<<static_cast<unsigned>((quads + 255) / 256), 256, 0, st>>>(epi.part, shape.splits, static_cast<int>(M),
                                                                                    static_cast<int>(N), static_cast<__nv_bfloat16*>(y), y_pitch);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_bf16_gemm(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, void* stream) {
  return spinf_bf16_gemm_ld(x, w, y, M, N, K, N, stream);
}

extern "C" int spinf_fp8_rowwise_gemm_glu(const void* x8, const float* xs, const void* w8_tiled, const float* ws_tiled, void* y,
                                          float* row_amax, int64_t M, int64_t F, int64_t K, int32_t act, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x8 && xs && w8_tiled && ws_tiled && y && row_amax && M >= 0 && F > 0 && K > 0 && K % 16 == 0 && F % 128 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && F < (1ll << 30) && K < (1ll << 31) && (act == 0 || act == 1));
  constexpr int BN = 256;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPINF_CUDA_OK(cudaMemsetAsync(row_amax, 0, static_cast<size_t>(M) * sizeof(float), st));
  CUtensorMap tmA, tmB, tmC;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8_tiled, 2 * F, K, K, 128, BN))) return r;
  if ((r = make_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, M, F, F * 2, 64, 128))) return r;
  const GemmShape shape = make_shape(M, 2 * F, K, BN);
  if (act == 0) {
    EpiGlu<BN, 0> epi;
    epi.tmC = tmC, epi.rowscale = xs, epi.colscale_g = ws_tiled, epi.row_amax = row_amax;
    return launch_gemm<KIND_F8, BN>(tmA, tmB, shape, epi, st);
  }
  EpiGlu<BN, 1> epi;
  epi.tmC = tmC, epi.rowscale = xs, epi.colscale_g = ws_tiled, epi.row_amax = row_amax;
  return launch_gemm<KIND_F8, BN>(tmA, tmB, shape, epi, st);
}

extern "C" int spinf_fp8_rowwise_gemm_qkv(const void* x8, const float* xs, const void* w8, const float* ws, void* y, int64_t M, int32_t H,
                                          int32_t Hkv, int32_t D, int64_t K, const void* wq, const void* wk, const void* cos_t,
                                          const void* sin_t, float eps, int32_t plus1, int32_t norm_v, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(x8 && xs && w8 && ws && y && wq && wk && cos_t && sin_t && M >= 0 && K > 0 && K % 16 == 0);
  SPINF_CHECK_ARG(H > 0 && Hkv > 0 && (D == 128 || D == 256) && M < (1ll << 31) && K < (1ll << 31));
  const int64_t N = static_cast<int64_t>(H + 2 * Hkv) * D;
  SPINF_CHECK_ARG(N % 256 == 0 && N < (1ll << 31));
  // rows are read and written as 32-byte pieces
  SPINF_CHECK_ARG(((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t) |
                    reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk)) & 31) == 0);
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, M, K, K, 128, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, N, K, K, 128, BN))) return r;
  const GemmShape shape = make_shape(M, N, K, BN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto fill = [&](auto& epi) {
    epi.y = static_cast<__nv_bfloat16*>(y), epi.y_pitch = N, epi.rowscale = xs, epi.colscale_g = ws;
    epi.wq = static_cast<const __nv_bfloat16*>(wq), epi.wk = static_cast<const __nv_bfloat16*>(wk);
    epi.cos_t = static_cast<const __nv_bfloat16*>(cos_t), epi.sin_t = static_cast<const __nv_bfloat16*>(sin_t);
    epi.H = H, epi.Hkv = Hkv, epi.eps = eps, epi.plus1 = plus1, epi.norm_v = norm_v;
  };
  if (D == 256) {
    EpiQkvNormRope<BN, 256> epi;
    fill(epi);
    return launch_gemm<KIND_F8, BN>(tmA, tmB, shape, epi, st);
  }
  EpiQkvNormRope<BN, 128> epi;
  fill(epi);
  return launch_gemm<KIND_F8, BN>(tmA, tmB, shape, epi, st);
}

extern "C" int spinf_fp8_quant_from_amax(const void* y, const float* row_amax, int64_t M, int64_t K, void* x8, float* xs, void* stream) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(y && row_amax && x8 && xs && M >= 0 && K > 0 && K % 8 == 0 && M < (1ll << 31) && K < (1ll << 31));
  fp8_quant_from_amax_kernel<<<static_cast<unsigned>(M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), row_amax, static_cast<int>(K), static_cast<uint8_t*>(x8), xs);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

// workspace layout: part_max [tiles_n * Mpad] f32 | part_sum [tiles_n * Mpad] f32 | col_tile_start [tiles_n + 1] i32
extern "C" int64_t spinf_option_logprobs_workspace_bytes(int64_t R, int64_t vocab, int64_t n_cols) {
  if (R < 0 || vocab <= 0 || n_cols < 0) return SPINF_ERR_BAD_ARGUMENT;
  const int64_t tiles_n = (vocab + 255) / 256, Mpad = (R + 127) / 128 * 128;
  return 2 * tiles_n * Mpad * 4 + (tiles_n + 1) * 4 + 256;
}

extern "C" int spinf_option_logprobs(const void* h, const void* W, int64_t R, int64_t hidden, int64_t vocab, const int32_t* cols,
                                     int64_t n_cols, float softcap, float* out, void* workspace,
                                     int64_t workspace_bytes, void* stream) {
  if (R == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(h && W && out && workspace && R >= 0 && hidden > 0 && hidden % 8 == 0 && vocab > 0 && n_cols >= 0);
  SPINF_CHECK_ARG(n_cols == 0 || cols);
  SPINF_CHECK_ARG(R < (1ll << 31) && vocab < (1ll << 31) && hidden < (1ll << 31) && n_cols < (1ll << 24));
  SPINF_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 15) == 0);
  if (workspace_bytes < spinf_option_logprobs_workspace_bytes(R, vocab, n_cols)) return SPINF_ERR_BAD_ARGUMENT;
  constexpr int BN = 256;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const GemmShape shape = make_shape(R, vocab, hidden, BN);
  const int64_t Mpad = static_cast<int64_t>(shape.tiles_m) * 128;
  float* part_max = static_cast<float*>(workspace);
  float* part_sum = part_max + shape.tiles_n * Mpad;
  int32_t* start_dev = reinterpret_cast<int32_t*>(part_sum + shape.tiles_n * Mpad);
  col_tile_start_kernel<<<(shape.tiles_n + 1 + 255) / 256, 256, 0, st>>>(cols, static_cast<int>(n_cols), shape.tiles_n, BN, start_dev);
  SPINF_CUDA_OK(cudaGetLastError());

  CUtensorMap tmA, tmB;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, h, R, hidden, hidden * 2, 64, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, vocab, hidden, hidden * 2, 64, BN))) return r;
  EpiLse<BN> epi;
  epi.softcap = softcap;
  epi.part_max = part_max;
  epi.part_sum = part_sum;
  epi.Mpad = static_cast<int>(Mpad);
  epi.cols = cols;
  epi.col_tile_start = start_dev;
  epi.out = out;
  epi.n_cols = static_cast<int>(n_cols);
  GemmShape sh = shape;
  sh.group_m = shape.tiles_m;  // all row tiles of one vocabulary tile run together: W is streamed from HBM once
  if ((r = launch_gemm<KIND_BF16, BN>(tmA, tmB, sh, epi, st))) return r;
  lse_finalize_kernel<<<static_cast<unsigned>(R), 128, 0, st>>>(part_max, part_sum, shape.tiles_n,
                                                                             static_cast<int>(Mpad), static_cast<int>(R), out,
                                                                             static_cast<int>(n_cols));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------ allocation-free variant
// The option log-prob read for callers that may not allocate device memory: a serving process that has handed all of its HBM to
// its own allocator, a host binding that cannot reach an allocator at all, or code running where cudaMalloc is off limits (it
// synchronises the device). The per-tile partials that spinf_option_logprobs keeps in a caller-provided workspace live here in a
// fixed array that is part of the library image: every GPU that loads the library holds these bytes until the process exits.
static constexpr size_t STATIC_SCRATCH_BYTES = (8u << 20) + 8192;  // 2 x 1 Mi partial floats + column-tile table + status slot
static __device__ __align__(256) unsigned char g_option_scratch[STATIC_SCRATCH_BYTES];

// In host code `g_option_scratch` names a host-side shadow of the symbol, not device memory: the address a kernel can use comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static unsigned char* option_scratch_device_ptr(int dev) {
  static unsigned char* ptrs[64] = {nullptr};
  static std::mutex mu;
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_option_scratch) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<unsigned char*>(p);
  }
  return ptrs[dev];
}

extern "C" int spinf_option_logprobs_static(const void* h, const void* W, int64_t R, int64_t hidden, int64_t vocab, const int32_t* cols,
                                            int64_t n_cols, float softcap, float* out, int32_t* status, void* stream) {
  if (R == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(h && W && out && R >= 0 && hidden > 0 && hidden % 8 == 0 && vocab > 0 && n_cols >= 0);
  SPINF_CHECK_ARG(n_cols == 0 || cols);
  SPINF_CHECK_ARG(R < (1ll << 31) && vocab < (1ll << 31) && hidden < (1ll << 31) && n_cols < (1ll << 24));
  constexpr int BN = 256;
  const GemmShape shape = make_shape(R, vocab, hidden, BN);
  const int64_t Mpad = static_cast<int64_t>(shape.tiles_m) * 128;
  const int64_t partial_floats = 2 * static_cast<int64_t>(shape.tiles_n) * Mpad;
  // layout: [0, 256) status slot | partial maxima | partial sums | column-tile table
  const int64_t need = 256 + partial_floats * 4 + (static_cast<int64_t>(shape.tiles_n) + 1) * 4;
  if (need > static_cast<int64_t>(STATIC_SCRATCH_BYTES)) return SPINF_ERR_TOO_LARGE;
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  unsigned char* base = option_scratch_device_ptr(dev);  // first call on a device resolves the symbol
  if (!base) return SPINF_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* status_word_p = status ? status : reinterpret_cast<int*>(base);
  float* part_max = reinterpret_cast<float*>(base + 256);
  float* part_sum = part_max + shape.tiles_n * Mpad;
  int32_t* start_dev = reinterpret_cast<int32_t*>(part_sum + shape.tiles_n * Mpad);
  // nothing in the scratch has to start at zero: every partial of every row tile and the whole column-tile table are rewritten
  // by this call before they are read; what the previous call left behind is never read
  col_tile_start_kernel<<<(shape.tiles_n + 1 + 255) / 256, 256, 0, st>>>(cols, static_cast<int>(n_cols), shape.tiles_n, BN, start_dev);
  SPINF_CUDA_OK(cudaGetLastError());
  CUtensorMap tmA, tmB;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, h, R, hidden, hidden * 2, 64, 128))) return r;
  if ((r = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, vocab, hidden, hidden * 2, 64, BN))) return r;
  EpiLse<BN> epi;
  epi.softcap = softcap;
  epi.part_max = part_max;
  epi.part_sum = part_sum;
  epi.Mpad = static_cast<int>(Mpad);
  epi.cols = cols;
  epi.col_tile_start = start_dev;
  epi.out = out;
  epi.n_cols = static_cast<int>(n_cols);
  GemmShape sh = shape;
  sh.group_m = shape.tiles_m;
  auto kern = gemm_tc_kernel<KIND_BF16, BN, EpiLse<BN>>;
  static std::atomic<bool> smem_set[64];  // the kernel's shared-memory attribute, set on this entry point's first call per device
  if (dev < 0 || dev >= 64) return SPINF_ERR_CUDA;
  if (!smem_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL));
    smem_set[dev].store(true, std::memory_order_release);
  }
  const int tiles = sh.tiles_m * sh.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 192, GemmSmem<BN>::TOTAL, st>>>(tmA, tmB, sh, epi, status_word_p);
  SPINF_CUDA_OK(cudaGetLastError());
  lse_finalize_kernel<<<static_cast<unsigned>(R), 128, 0, st>>>(part_max, part_sum, sh.tiles_n, static_cast<int>(Mpad),
                                                                             static_cast<int>(R), out, static_cast<int>(n_cols));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

