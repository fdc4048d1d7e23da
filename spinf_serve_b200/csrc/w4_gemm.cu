// int4 (GPTQ, symmetric, grouped scales) weight-only GEMM for sm_100a:  y[M,N] = bf16( x[M,K] . dq(W)[N,K]^T ),
//     dq(W)[n,k] = bf16( (nibble(n,k) - 8) * float(scale[n, k / G]) )      (one rounding, as the reference's dq_bf16)
// x bf16, fp32 accumulation in tensor memory, bf16 out. The weights stay int4 in HBM and are expanded on the way to the tensor
// core: nothing the size of the bf16 weight matrix is ever written.
//
// Persistent, one CTA per SM, 256 x 128 output tiles (two M=128 accumulators share every dequantised weight tile, halving the
// expansion work per FLOP), K in steps of 64. 14 warps:
//   warp 0     one lane: TMA loads of the activation tile (256 x 128 B, swizzled) and the raw weight tile (128 rows x 32 B) into a 4-stage ring
//   warps 6-13 dequantisers in two groups of four warps that take alternate K steps (two steps in flight), thread = weight row:
//              64 nibbles -> 64 bf16 written as a K-major 128-byte-swizzled tile into a 4-stage ring; a nibble becomes the float 128 + n with one byte permute, then one FMA gives (n - 8) * scale exactly
//   warp 1     one lane: tcgen05.mma, 2 x (M=128, N=128, K=64) per step, into one of two accumulator pairs
//   warps 2-5  epilogue: TMEM -> bf16 -> swizzled staging -> TMA store, overlapped with the next tile's main loop
// K order per output element is ascending inside one CTA and the tile shape does not depend on M: rows are batch-invariant.
#include "gemm_tc.cuh"
#include "host_util.h"

namespace spinf {

struct W4Smem {
  static constexpr int STAGES = 4, BSTAGES = 4;
  static constexpr int A_BYTES = 256 * 128;   // activations: 256 rows x 64 bf16
  static constexpr int RAW_BYTES = 128 * 32;  // raw weights: 128 rows x 64 nibbles
  static constexpr int STAGE_BYTES = A_BYTES + RAW_BYTES;
  static constexpr int B_BYTES = 128 * 128;   // dequantised weights: 128 rows x 64 bf16
  static constexpr int B_OFF = STAGES * STAGE_BYTES;
  static constexpr int EPI_OFF = B_OFF + BSTAGES * B_BYTES;
  static constexpr int BAR_OFF = EPI_OFF + 128 * 128;  // one staging tile: the epilogue has a whole main loop of slack
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

struct W4Args {
  const __half* scales;  // [N, K / G]
  int M, N, K, G;
  int tiles_m, tiles_n, group_m;
};

__global__ void __launch_bounds__(448, 1)
w4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmC,
               const W4Args a, int* __restrict__ status) {
  using L = W4Smem;
  constexpr int STAGES = L::STAGES, BSTAGES = L::BSTAGES;
  constexpr uint32_t IDESC = make_idesc(FMT_BF16, FMT_BF16, 128, 128, 0, 0);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);  // TMA landed (A + raw W)
  uint64_t* empty = full + STAGES;                                   // 1 MMA commit + 4 dequantiser-warp arrivals
  uint64_t* b_full = empty + STAGES;                                 // 4 dequantiser-warp arrivals
  uint64_t* b_empty = b_full + BSTAGES;                              // 1 MMA commit
  uint64_t* acc_full = b_empty + BSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_p + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 5);  // the MMA commit + one arrival per warp of the dequantising group
    }
    for (int s = 0; s < BSTAGES; ++s) {
      mbar_init(&b_full[s], 4);  // one arrival per warp of the dequantising group
      mbar_init(&b_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_p, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_p;
  GemmShape shape;
  shape.M = a.M, shape.N = a.N, shape.K = a.K, shape.tiles_m = a.tiles_m, shape.tiles_n = a.tiles_n, shape.group_m = a.group_m;
  const int num_tiles = a.tiles_m * a.tiles_n;
  const int num_kb = a.K / 64;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(shape, tile, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(wc, &empty[s], ph ^ 1u, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          tma_load_2d(sa, &tmA, kb * 64, tm * 256, &full[s]);
          tma_load_2d(sa + 128 * 128, &tmA, kb * 64, tm * 256 + 128, &full[s]);
          tma_load_2d(sa + L::A_BYTES, &tmW, kb * 32, tn * 128, &full[s]);
        }
      }
      if (!ok) {
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t ab = tcount & 1u, aph = (tcount >> 1) & 1u;
        if (!mbar_wait(wc, &acc_empty[ab], aph ^ 1u, ST_TIMEOUT_TMEM)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          const uint32_t bs = it % BSTAGES, bph = (it / BSTAGES) & 1u;
          if (!mbar_wait(wc, &full[s], ph, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (!mbar_wait(wc, &b_full[bs], bph, ST_TIMEOUT_OTHER)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(smem + L::B_OFF + bs * L::B_BYTES), 16, 1024);
#pragma unroll
          for (int mh = 0; mh < 2; ++mh) {
            const uint64_t adesc = make_smem_desc_sw128(sa + mh * 128 * 128, 16, 1024);
            const uint32_t d_tmem = tmem_base + ab * 256 + mh * 128;
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb | k) != 0);
          }
          umma_commit(&empty[s]);
          umma_commit(&b_empty[bs]);
        }
        if (ok) umma_commit(&acc_full[ab]);
      }
    }
  } else if (warp >= 6) {
    // dequantisers: two groups of 128 threads take alternate K steps; thread = weight row of the tile
    const int dt = threadIdx.x - 192;   // 0..255
    const int grp = dt >> 7;
    const int n_local = dt & 127;
    uint32_t it = 0;
    bool ok = true;
    const int groups = a.K / a.G;
    const bool coarse = a.G % 64 == 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(shape, tile, tm, tn);
      const int n = tn * 128 + n_local;
      const bool n_ok = n < a.N;
      const __half* srow = a.scales + static_cast<int64_t>(n_ok ? n : 0) * groups;
      int s_idx = -1;
      float sc = 0.f, off = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((it & 1u) != static_cast<uint32_t>(grp)) continue;
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        const uint32_t bs = it % BSTAGES, bph = (it / BSTAGES) & 1u;
        bool got = mbar_wait(wc, &full[s], ph, ST_TIMEOUT_FULL);
        got = got && mbar_wait(wc, &b_empty[bs], bph ^ 1u, ST_TIMEOUT_EMPTY);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        const uint4* raw = reinterpret_cast<const uint4*>(smem + s * L::STAGE_BYTES + L::A_BYTES + n_local * 32);
        const uint4 r0 = raw[0], r1 = raw[1];
        const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        uint8_t* btile = smem + L::B_OFF + bs * L::B_BYTES;
        if (coarse) {  // one scale for the whole 64-wide K step (group a multiple of 64): one division per step
          const int gi = (kb * 64) / a.G;
          if (gi != s_idx) {
            s_idx = gi;
            sc = n_ok ? __half2float(srow[gi]) : 0.f;
            off = -136.f * sc;  // exact: 136 has 5 significant bits, a half-precision scale 11
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 8 nibbles -> 8 bf16 = one 16-byte chunk of the row
          if (!coarse) {
            const int gi = (kb * 64 + c * 8) / a.G;
            if (gi != s_idx) {
              s_idx = gi;
              sc = n_ok ? __half2float(srow[gi]) : 0.f;
              off = -136.f * sc;
            }
          }
          const uint32_t even = words[c] & 0x0F0F0F0Fu;         // nibbles 0, 2, 4, 6 (k even), one per byte
          const uint32_t odd = (words[c] >> 4) & 0x0F0F0F0Fu;   // nibbles 1, 3, 5, 7
          uint32_t out[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // bytes [0, 0, nibble, 0x43] = the float 128 + nibble; fma(128 + n, s, -136 s) = (n - 8) s with no rounding
            // (the product and the sum are exact inside the FMA and the result fits fp32); then one rounding to bf16
            const float lo = fmaf(__uint_as_float(__byte_perm(even, 0x43000000u, 0x7044u | (j << 8))), sc, off);
            const float hi = fmaf(__uint_as_float(__byte_perm(odd, 0x43000000u, 0x7044u | (j << 8))), sc, off);
            out[j] = pack_bf16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(btile + sw128_offset(n_local, c)) = make_uint4(out[0], out[1], out[2], out[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();  // every lane's chunk is written and fenced: one arrival per warp instead of 32
        if (lane == 0) {
          mbar_arrive(&b_full[bs]);
          mbar_arrive(&empty[s]);  // the raw tile has been read
        }
      }
    }
  } else {
    // epilogue: warps 2-5, thread = accumulator row of each 128-row half
    const int et = threadIdx.x - 64;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint8_t* epi_stage = smem + L::EPI_OFF;
    uint32_t tcount = 0, nstores = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      int tm, tn;
      tile_coords(shape, tile, tm, tn);
      const uint32_t ab = tcount & 1u, aph = (tcount >> 1) & 1u;
      const bool got = mbar_wait(wc, &acc_full[ab], aph, ST_TIMEOUT_TMEM);
      if (!bar_red_and(1, 128, got)) break;
      tc_fence_after();
#pragma unroll 1
      for (int part = 0; part < 4; ++part) {  // (row half, 64-column chunk)
        const int mh = part >> 1, c = part & 1;
        uint32_t v0[32], v1[32];
        __syncwarp();
        const uint32_t taddr = tmem_base + ab * 256 + mh * 128 + c * 64 + (static_cast<uint32_t>(q * 32) << 16);
        tmem_ld_x32(taddr, v0);
        tmem_ld_x32(taddr + 32, v1);
        tmem_wait_ld();
        if (part == 3) {
          tc_fence_before();
          mbar_arrive(&acc_empty[ab]);
        }
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          packed[i] = pack_bf16x2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
          packed[16 + i] = pack_bf16x2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
        }
        uint8_t* buf = epi_stage;
        if (et == 0) tma_store_wait_read<0>();
        named_bar_sync(1, 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(buf + sw128_offset(row, j)) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (et == 0) {
          tma_store_2d(&tmC, buf, tn * 128 + c * 64, tm * 256 + mh * 128);
          tma_store_commit();
        }
        ++nstores;
      }
    }
    if (et == 0) tma_store_wait_all<0>();
  }

  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_w4_gemm(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                             int64_t y_pitch, void* stream) {
  SPINF_CHECK_ARG(x && qw && scales && y && M >= 0 && N > 0 && K > 0 && group > 0);
  SPINF_CHECK_ARG(K % 64 == 0 && group % 8 == 0 && K % group == 0 && N % 8 == 0 && y_pitch >= N && y_pitch % 8 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  if (M == 0) return 0;
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  CUtensorMap tmA, tmW, tmC;
  int r;
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, K * 2, 64, 128))) return r;
  if ((r = make_tmap_2d_plain(&tmW, qw, N, K / 2, K / 2, 32, 128))) return r;
  if ((r = make_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, M, N, y_pitch * 2, 64, 128))) return r;
  W4Args a;
  a.scales = static_cast<const __half*>(scales);
  a.M = static_cast<int>(M), a.N = static_cast<int>(N), a.K = static_cast<int>(K), a.G = group;
  a.tiles_m = static_cast<int>((M + 255) / 256);
  a.tiles_n = static_cast<int>((N + 127) / 128);
  // groups of row tiles as tall as about 32 MB of bf16 activations allow (4..32 tiles of 256 rows): the packed weight streams past
  // once per group
  {
    const int64_t per_tile = 256 * K * 2;
    const int64_t g = (32ll << 20) / per_tile;
    a.group_m = static_cast<int>(g < 4 ? 4 : (g > 32 ? 32 : g));
  }
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Smem::TOTAL));
    attr_set[dev] = true;
  }
  const int tiles = a.tiles_m * a.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  w4_gemm_kernel<<<grid, 448, W4Smem::TOTAL, static_cast<cudaStream_t>(stream)>>>(tmA, tmW, tmC, a, status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
