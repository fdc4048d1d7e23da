// Persistent tcgen05 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  with fp32 accumulation in tensor memory.
//
//   A: row-major [M,K] (activations, K contiguous)      B: row-major [N,K] (weights, one output channel per row)
//   element kinds: e4m3 x e4m3 (kind::f8f6f4, 128 K-elements per stage) or bf16 x bf16 (kind::f16, 64 K-elements per stage)
//
// One CTA per SM, 6 warps:
//   warp 0   one lane issues the TMA loads of A (128 x 128 B) and B (BN x 128 B) tiles into a STAGES-deep ring
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, four K-steps of 32 B per stage) into one of two
//            accumulator buffers and commits to the ring's "empty" barriers and to the accumulator's "full" barrier
//   warps 2-5  epilogue: thread = accumulator row (TMEM lane); reads 64 columns at a time with tcgen05.ld and hands them to the
//            epilogue functor, so tile i's epilogue overlaps tile i+1's main loop
//
// Batch invariance: every output element is the sum over K in ascending order inside one CTA (no split-K, no stream-K), with a
// tile shape that does not depend on M, so a row of C is bit-identical whatever other rows are in the call. The one exception is
// an epilogue that declares kSplitK (a decoding step's few rows): its work units are (tile, K slice) pairs that leave fp32
// partial sums, added in slice order by a second kernel; the slicing depends on N and K only, so rows stay independent there too.
#pragma once
#include "common.cuh"

namespace spinf {

enum : int { KIND_F8 = 0, KIND_BF16 = 1, KIND_S8 = 2 };  // operand types: e4m3 (fp32 accumulators), bf16 (fp32), int8 (int32)

struct GemmShape {
  int M, N, K;
  int tiles_m, tiles_n;
  int group_m;  // rasterisation: tiles are walked in groups of `group_m` row-tiles, column-tile fastest inside a group
  // K slices (only read by kernels whose epilogue declares kSplitK): a work unit is (tile, slice), slice = unit % splits covers
  // the K blocks [slice * kb_per, min(num_kb, (slice + 1) * kb_per))
  int splits, kb_per;
};

// an epilogue that declares `static constexpr bool kSplitK = true` receives K slices (its State has a member `ks`)
template <class E, class = void>
struct EpiSplitK {
  static constexpr bool value = false;
};
template <class E>
struct EpiSplitK<E, decltype(void(E::kSplitK))> {
  static constexpr bool value = E::kSplitK;
};

template <int BN>
struct GemmSmem {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = 2 * 128 * 128;  // two staging buffers of 128 rows x 64 bf16
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES + EPI_BYTES;
  // barriers (2*STAGES + 4) * 8 B, tmem base, abort flag, then BN floats of per-column scale
  static constexpr int COLSCALE_OFFSET = BAR_OFFSET + 256;
  static constexpr int TOTAL = COLSCALE_OFFSET + BN * 4 + 1024;  // + slack for the 1024-byte alignment of the base
};

__device__ __forceinline__ void tile_coords(const GemmShape& s, int tile, int& tm, int& tn) {
  const int per_group = s.group_m * s.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * s.group_m;
  const int rows = min(s.group_m, s.tiles_m - first_m);
  const int t = tile - g * per_group;
  tm = first_m + t % rows;
  tn = t / rows;
}

// Epilogue functor contract (all calls are made by the 128 epilogue threads, thread = row `row` of the tile; the functor is a
// __grid_constant__ kernel parameter, so it may hold a TMA descriptor; its mutable per-thread state lives in Epi::State):
//   begin_tile(st, shape, tm, tn, et, ...)       once per tile before the accumulator is ready (et = 0..127)
//   chunk(st, shape, tm, tn, row, et, c, v0, v1, ..., t_row) 64 accumulator columns [c*64, c*64+64) of this thread's row, as two x32
//                                                groups (t_row = TMEM address of the row's first column)
//   end_tile(st, ..., t_row, ...)                after the last chunk (may read single TMEM columns when kReadsTmemInEnd)
//   finish(st, et)                               once, after the last tile
template <int KIND, int BN, class Epi>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmShape shape,
               const __grid_constant__ Epi epi, int* __restrict__ status) {
  using L = GemmSmem<BN>;
  constexpr int STAGES = L::STAGES;
  constexpr int KE = KIND == KIND_BF16 ? 64 : 128;  // K elements per stage (128 bytes)
  constexpr uint32_t IDESC = KIND == KIND_F8   ? make_idesc(FMT_E4M3, FMT_E4M3, 128, BN, 0, 0)
                             : KIND == KIND_S8 ? make_idesc_s8(128, BN)
                                               : make_idesc(FMT_BF16, FMT_BF16, 128, BN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_p + 1);
  float* colscale = reinterpret_cast<float*>(smem + L::COLSCALE_OFFSET);
  uint8_t* epi_stage = smem + STAGES * L::STAGE_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_p, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_p;

  constexpr bool SPLIT = EpiSplitK<Epi>::value;
  const int splits = SPLIT ? shape.splits : 1;
  const int num_tiles = shape.tiles_m * shape.tiles_n * splits;
  const int num_kb = (shape.K + KE - 1) / KE;
  const int kb_per = SPLIT ? shape.kb_per : num_kb;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(shape, SPLIT ? tile / splits : tile, tm, tn);
        const int kb0 = SPLIT ? (tile % splits) * kb_per : 0, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(wc, &empty[s], ph ^ 1u, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          tma_load_2d(sa, &tmA, kb * KE, tm * 128, &full[s]);
          tma_load_2d(sa + L::A_BYTES, &tmB, kb * KE, tn * BN, &full[s]);
        }
      }
      if (!ok) {
        // bounded wait for this CTA's own copies still in flight before the shared memory goes away
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const uint32_t s = j % STAGES, ph = (j / STAGES) & 1u;
          for (int spin = 0; spin < 4096 && !mbar_try_wait(&full[s], ph); ++spin) {}
        }
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
        const uint32_t d_tmem = tmem_base + ab * BN;
        const int kb0 = SPLIT ? (tile % splits) * kb_per : 0, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(wc, &full[s], ph, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + L::A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes along K per step: +2 in the descriptor's 16-byte address units
            if (KIND == KIND_F8)
              umma_f8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, ((kb - kb0) | k) != 0);
            else if (KIND == KIND_S8)
              umma_i8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, ((kb - kb0) | k) != 0);
            else
              umma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, ((kb - kb0) | k) != 0);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[ab]);
      }
    }
  } else {
    const int et = threadIdx.x - 64;        // 0..127
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;          // accumulator row of this thread
    uint32_t tcount = 0;
    typename Epi::State est{};
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      int tm, tn;
      tile_coords(shape, SPLIT ? tile / splits : tile, tm, tn);
      if constexpr (SPLIT) est.ks = tile % splits;
      const uint32_t ab = tcount & 1u, aph = (tcount >> 1) & 1u;
      __syncwarp();
      epi.begin_tile(est, shape, tm, tn, et, colscale);
      const bool got = mbar_wait(wc, &acc_full[ab], aph, ST_TIMEOUT_TMEM);
      if (!bar_red_and(1, 128, got)) break;  // all 128 epilogue threads leave together
      tc_fence_after();
      const uint32_t t_row = tmem_base + ab * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        __syncwarp();
        tmem_ld_x32(t_row + c * 64, v0);
        tmem_ld_x32(t_row + c * 64 + 32, v1);
        tmem_wait_ld();
        if (c == BN / 64 - 1 && !Epi::kReadsTmemInEnd) {
          tc_fence_before();
          mbar_arrive(&acc_empty[ab]);
        }
        epi.chunk(est, shape, tm, tn, row, et, c, v0, v1, colscale, epi_stage, t_row);
      }
      __syncwarp();
      epi.end_tile(est, shape, tm, tn, row, et, t_row, colscale);
      if (Epi::kReadsTmemInEnd) {
        tc_fence_before();
        mbar_arrive(&acc_empty[ab]);
      }
    }
    epi.finish(est, et);
  }

  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------ epilogues

// bf16 output through a swizzled staging buffer and TMA stores of 128 x 64 boxes.
//   SCALED: y = bf16((acc * rowscale[m]) * colscale[n])   (the row-wise fp8 linear)       else: y = bf16(acc)
//   ACC_S32: the accumulators are 32-bit integers (int8 operands), converted to fp32 first as the reference's `.float()` does
template <int BN, bool SCALED, bool ACC_S32 = false>
struct EpiStoreBf16 {
  static constexpr bool kReadsTmemInEnd = false;
  CUtensorMap tmC;  // [M, N] bf16, box 64 x 128, 128-byte swizzle
  const float* rowscale;
  const float* colscale_g;
  int rowscale_stride = 1, colscale_stride = 1;  // 0: one scale for every row / column (the per-tensor fp8 linears)
  struct State {
    uint32_t nstores;
  };

  __device__ __forceinline__ void begin_tile(State&, const GemmShape& s, int tm, int tn, int et, float* colscale) const {
    if (SCALED) {
      named_bar_sync(2, 128);  // the previous tile's readers of colscale are done
      for (int i = et; i < BN; i += 128) {
        const int n = tn * BN + i;
        colscale[i] = n < s.N ? colscale_g[static_cast<size_t>(n) * colscale_stride] : 0.f;
      }
      named_bar_sync(2, 128);
    }
  }
  __device__ __forceinline__ void chunk(State& st, const GemmShape& s, int tm, int tn, int row, int et, int c,
                                        const uint32_t (&v0)[32], const uint32_t (&v1)[32], const float* colscale,
                                        uint8_t* epi_stage, uint32_t) const {
    float rs = 1.f;
    if (SCALED) {
      const int m = tm * 128 + row;
      rs = m < s.M ? rowscale[static_cast<size_t>(m) * rowscale_stride] : 0.f;
    }
    uint32_t packed[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a, b, d, e;
      if (ACC_S32) {
        a = __int2float_rn(static_cast<int>(v0[2 * i])), b = __int2float_rn(static_cast<int>(v0[2 * i + 1]));
        d = __int2float_rn(static_cast<int>(v1[2 * i])), e = __int2float_rn(static_cast<int>(v1[2 * i + 1]));
      } else {
        a = __uint_as_float(v0[2 * i]), b = __uint_as_float(v0[2 * i + 1]);
        d = __uint_as_float(v1[2 * i]), e = __uint_as_float(v1[2 * i + 1]);
      }
      if (SCALED) {
        a = (a * rs) * colscale[c * 64 + 2 * i];
        b = (b * rs) * colscale[c * 64 + 2 * i + 1];
        d = (d * rs) * colscale[c * 64 + 32 + 2 * i];
        e = (e * rs) * colscale[c * 64 + 32 + 2 * i + 1];
      }
      packed[i] = pack_bf16x2(a, b);
      packed[16 + i] = pack_bf16x2(d, e);
    }
    uint8_t* buf = epi_stage + (st.nstores & 1u) * (128 * 128);
    // the TMA store that last read this buffer (two stores ago) must have finished reading it
    if (et == 0) tma_store_wait_read<1>();
    named_bar_sync(1, 128);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 val = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      *reinterpret_cast<uint4*>(buf + sw128_offset(row, j)) = val;
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (et == 0) {
      tma_store_2d(&tmC, buf, tn * BN + c * 64, tm * 128);
      tma_store_commit();
    }
    ++st.nstores;
  }
  __device__ __forceinline__ void end_tile(State&, const GemmShape&, int, int, int, int, uint32_t, const float*) const {}
  __device__ __forceinline__ void finish(State&, int et) const {
    if (et == 0) tma_store_wait_all<0>();
  }
};

// fp32 partial sums of one K slice: part[ks][m][n] (the epilogue of the few-row split; scales and rounding happen in the kernel
// that adds the slices)
template <int BN>
struct EpiPartial {
  static constexpr bool kReadsTmemInEnd = false;
  static constexpr bool kSplitK = true;
  float* part;  // [splits, M, N]
  struct State {
    int ks;
  };
  __device__ __forceinline__ void begin_tile(State&, const GemmShape&, int, int, int, float*) const {}
  __device__ __forceinline__ void chunk(State& st, const GemmShape& s, int tm, int tn, int row, int, int c, const uint32_t (&v0)[32],
                                        const uint32_t (&v1)[32], const float*, uint8_t*, uint32_t) const {
    const int m = tm * 128 + row, n0 = tn * BN + c * 64;
    if (m >= s.M) return;
    float* dst = part + (static_cast<size_t>(st.ks) * s.M + m) * s.N + n0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t* v = j < 8 ? &v0[4 * j] : &v1[4 * (j - 8)];
      if (n0 + 4 * j < s.N) *reinterpret_cast<uint4*>(dst + 4 * j) = make_uint4(v[0], v[1], v[2], v[3]);
    }
  }
  __device__ __forceinline__ void end_tile(State&, const GemmShape&, int, int, int, int, uint32_t, const float*) const {}
  __device__ __forceinline__ void finish(State&, int) const {}
};

}  // namespace spinf
