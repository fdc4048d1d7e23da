// W4A16 linear for a few rows (the extraction decoder's steps): replaces spinf_serve/quant/w4gemm.py:17-66 (`_w4_small`, `linear`).
// The int4 weights are read as the engine stores them (q uint8 [N, K/2]: byte b of a row = k 2b in the low nibble, k 2b + 1 in the
// high one, value nibble - 8; s fp16 [N, K / group] group scales) and are streamed exactly once: with M of some tens the weights
// are the traffic. Arithmetic as the reference's kernel: the activations rounded to fp16, the weight (nibble - 8) * scale formed
// and rounded in fp16, fp16 tensor-core products with fp32 accumulation, split-K partial sums in an fp32 buffer
// [splits, M, N] added in split order, the sum rounded to bf16.
//   grid (ceil(N / 128), splits), 256 threads: warp w owns 16 output channels of the block for all rows; a k-tile of 256 is staged in
//   shared memory by cp.async (two stages); a thread takes 8 consecutive k of its channel as one 32-bit word and of each of its
//   rows as one 128-bit load: the tensor-core fragment slots are filled in that (permuted) k order on both operands.
#include "common.cuh"
#include "host_util.h"

#include <cuda_fp16.h>

#include <atomic>

namespace spinf {

static constexpr int WS_BK = 256;  // k per staged tile; a CTA owns BN = 64 or 128 output channels, 16 per warp
static constexpr int WS_XLD = WS_BK * 2 + 64;   // bytes per staged activation row: 144 words, rows alternate bank halves
static constexpr int WS_QLD = WS_BK / 2 + 16;   // bytes per staged weight row: 36 words
static constexpr int WS_MAXG = WS_BK / 32;      // group scales per row and k-tile at the smallest group (32)

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async8(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4z(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}

// byte b (k even in the low nibble, k odd in the high) -> half2 ((lo - 8) * s, (hi - 8) * s), each product rounded to fp16
__device__ __forceinline__ uint32_t w4_pair(uint32_t byte, __half2 s2) {
  const uint32_t v = (byte & 0xFu) | ((byte & 0xF0u) << 12) | 0x64006400u;  // fp16 1024 + nibble, twice
  const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&v), __half2half2(__ushort_as_half(0x6408)));  // - 1032
  const __half2 w = __hmul2(h, s2);
  return *reinterpret_cast<const uint32_t*>(&w);
}

template <int MT, int WS_BN>  // row tiles of 16; output channels per CTA
__global__ void __launch_bounds__(WS_BN * 2) w4_small_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ q, const __half* __restrict__ s,
                                                        float* __restrict__ part, int M, int N, int K, int group, int k_per) {
  extern __shared__ __align__(16) uint8_t w4s_raw[];
  constexpr int BM = MT * 16;
  constexpr int WS_TH = WS_BN * 2;
  constexpr int STAGE = BM * WS_XLD + WS_BN * WS_QLD + WS_BN * WS_MAXG * 2;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int n0 = blockIdx.x * WS_BN, k_lo = blockIdx.y * k_per;
  const int tiles = k_per / WS_BK;
  const int gpt = WS_BK / group;  // scales per row and k-tile
  const int sld = K / group;

  auto stage = [&](int t, int buf) {
    uint8_t* const base = w4s_raw + buf * STAGE;
    const int k0 = k_lo + t * WS_BK;
    for (int i = tid; i < BM * (WS_BK / 8); i += WS_TH) {
      const int m = i / (WS_BK / 8), c = i % (WS_BK / 8);
      const bool ok = m < M;
      cp_async16(base + m * WS_XLD + c * 16, ok ? x + static_cast<int64_t>(m) * K + k0 + c * 8 : x, ok ? 16 : 0);
    }
    uint8_t* const qb = base + BM * WS_XLD;
    for (int i = tid; i < WS_BN * (WS_BK / 32); i += WS_TH) {
      const int n = i / (WS_BK / 32), c = i % (WS_BK / 32);
      const bool ok = n0 + n < N;
      cp_async16(qb + n * WS_QLD + c * 16, ok ? q + static_cast<int64_t>(n0 + n) * (K / 2) + k0 / 2 + c * 16 : q, ok ? 16 : 0);
    }
    // the tile's group scales ride the same asynchronous copies (a plain load here would put a global-memory latency in front of
    // every tile's products): 2 gpt bytes per row, as one 16-, 8- or 4-byte piece
    __half* const sb = reinterpret_cast<__half*>(qb + WS_BN * WS_QLD);
    if (gpt >= 2) {
      for (int n = tid; n < WS_BN; n += WS_TH) {
        const bool ok = n0 + n < N;
        const __half* src = ok ? s + static_cast<int64_t>(n0 + n) * sld + k0 / group : s;
        if (gpt == 8) cp_async16(sb + n * WS_MAXG, src, ok ? 16 : 0);
        else if (gpt == 4) cp_async8(sb + n * WS_MAXG, src, ok ? 8 : 0);
        else cp_async4z(sb + n * WS_MAXG, src, ok ? 4 : 0);
      }
    } else {
      for (int n = tid; n < WS_BN; n += WS_TH) sb[n * WS_MAXG] = n0 + n < N ? s[static_cast<int64_t>(n0 + n) * sld + k0 / group] : __float2half(0.f);
    }
  };

  float acc[MT][2][4] = {};
  stage(0, 0);
  cp_async_commit();
  for (int t = 0; t < tiles; ++t) {
    if (t + 1 < tiles) stage(t + 1, (t + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint8_t* const base = w4s_raw + (t & 1) * STAGE;
    const uint8_t* const qb = base + BM * WS_XLD;
    const __half* const sb = reinterpret_cast<const __half*>(qb + WS_BN * WS_QLD);
#pragma unroll 2
    for (int kb = 0; kb < WS_BK / 32; ++kb) {  // 32 k: two tensor-core steps
      uint32_t bw[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int n = warp * 16 + nt * 8 + gq;
        const uint32_t w = *reinterpret_cast<const uint32_t*>(qb + n * WS_QLD + kb * 16 + tq * 4);
        const __half2 s2 = __half2half2(sb[n * WS_MAXG + (kb * 32) / group]);
#pragma unroll
        for (int j = 0; j < 4; ++j) bw[nt][j] = w4_pair((w >> (8 * j)) & 0xFFu, s2);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint4 lo = *reinterpret_cast<const uint4*>(base + (mt * 16 + gq) * WS_XLD + kb * 64 + tq * 16);
        const uint4 hi = *reinterpret_cast<const uint4*>(base + (mt * 16 + gq + 8) * WS_XLD + kb * 64 + tq * 16);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          mma_f16(acc[mt][nt], lo.x, hi.x, lo.y, hi.y, bw[nt][0], bw[nt][1]);
          mma_f16(acc[mt][nt], lo.z, hi.z, lo.w, hi.w, bw[nt][2], bw[nt][3]);
        }
      }
    }
    __syncthreads();
  }
  float* const out = part + static_cast<int64_t>(blockIdx.y) * M * N;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = mt * 16 + gq + (e >> 1) * 8, n = n0 + warp * 16 + nt * 8 + tq * 2 + (e & 1);
        if (m < M && n < N) out[static_cast<int64_t>(m) * N + n] = acc[mt][nt][e];
      }
}

__global__ void w4_small_x_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xh, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) xh[i] = __float2half_rn(__bfloat162float(x[i]));
}

__global__ void w4_small_sum_kernel(const float* __restrict__ part, int splits, int64_t MN, int N, __nv_bfloat16* __restrict__ y, int64_t y_pitch) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= MN) return;
  float t = part[i];
  for (int sp = 1; sp < splits; ++sp) t += part[sp * MN + i];
  y[(i / N) * y_pitch + i % N] = __float2bfloat16_rn(t);
}

static int w4_small_splits(int64_t N, int64_t K) {
  // the reference's rule (w4gemm.py:51-56): about 512 programs, a split count that divides the k-tiles
  const int64_t n_blocks = (N + 63) / 64;  // the reference's programs are 64 channels wide
  int64_t splits = std::max<int64_t>(1, std::min<int64_t>(K / WS_BK, 512 / n_blocks));
  while ((K / WS_BK) % splits) --splits;
  return static_cast<int>(splits);
}

template <int MT, int BN>
static int w4_small_launch_bn(const __half* xh, const uint8_t* q, const __half* s, float* part, int M, int N, int K, int group, int splits,
                              cudaStream_t st) {
  constexpr int smem = 2 * (MT * 16 * WS_XLD + BN * WS_QLD + BN * WS_MAXG * 2);
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_small_kernel<MT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  w4_small_kernel<MT, BN><<<dim3(static_cast<unsigned>((N + BN - 1) / BN), static_cast<unsigned>(splits)), BN * 2, smem, st>>>(
      xh, q, s, part, M, N, K, group, K / splits);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int MT>
static int w4_small_launch(const __half* xh, const uint8_t* q, const __half* s, float* part, int M, int N, int K, int group, int splits,
                           cudaStream_t st) {
  // 128 channels per CTA halve the re-reads of the activation tile; worth it while the grid still covers the SMs one and a half times
  if (static_cast<int64_t>((N + 127) / 128) * splits * 2 >= 3 * sm_count()) return w4_small_launch_bn<MT, 128>(xh, q, s, part, M, N, K, group, splits, st);
  return w4_small_launch_bn<MT, 64>(xh, q, s, part, M, N, K, group, splits, st);
}

}  // namespace spinf

using namespace spinf;

// bytes of workspace spinf_w4_small needs: the fp16 copy of x and the [splits, M, N] fp32 partial sums
extern "C" int64_t spinf_w4_small_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || K % WS_BK) return 0;
  return ((M * K * 2 + 255) / 256) * 256 + static_cast<int64_t>(w4_small_splits(N, K)) * M * N * 4 + 256;
}

extern "C" int spinf_w4_small(const void* x, const void* q, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                              int64_t y_pitch, void* workspace, int64_t workspace_bytes, void* stream) {
  if (M == 0 || N == 0) return 0;
  SPINF_CHECK_ARG(x && q && scales && y && workspace && M > 0 && M <= 128 && N > 0 && K > 0 && K % WS_BK == 0);
  SPINF_CHECK_ARG(group >= 32 && group % 32 == 0 && WS_BK % group == 0 && y_pitch >= N && N < (1ll << 31) && K < (1ll << 31));
  SPINF_CHECK_ARG(workspace_bytes >= spinf_w4_small_workspace_bytes(M, N, K));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  ws += (256 - reinterpret_cast<uintptr_t>(ws) % 256) % 256;
  __half* const xh = reinterpret_cast<__half*>(ws);
  float* const part = reinterpret_cast<float*>(ws + ((M * K * 2 + 255) / 256) * 256);
  const int splits = w4_small_splits(N, K);
  const int64_t nx = M * K;
  w4_small_x_kernel<<<static_cast<unsigned>((nx + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), xh, nx);
  SPINF_CUDA_OK(cudaGetLastError());
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
  const uint8_t* qq = static_cast<const uint8_t*>(q);
  const __half* ss = static_cast<const __half*>(scales);
  int rc;
  if (M <= 16) rc = w4_small_launch<1>(xh, qq, ss, part, m, n, k, group, splits, st);
  else if (M <= 32) rc = w4_small_launch<2>(xh, qq, ss, part, m, n, k, group, splits, st);
  else if (M <= 48) rc = w4_small_launch<3>(xh, qq, ss, part, m, n, k, group, splits, st);
  else if (M <= 64) rc = w4_small_launch<4>(xh, qq, ss, part, m, n, k, group, splits, st);
  else rc = w4_small_launch<8>(xh, qq, ss, part, m, n, k, group, splits, st);
  if (rc) return rc;
  const int64_t MN = M * N;
  w4_small_sum_kernel<<<static_cast<unsigned>((MN + 255) / 256), 256, 0, st>>>(part, splits, MN, n, static_cast<__nv_bfloat16*>(y), y_pitch);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
