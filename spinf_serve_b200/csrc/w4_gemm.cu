// int4 (GPTQ, symmetric, grouped scales) weight-only GEMM for sm_100a:  y[M,N] = bf16( x[M,K] . dq(W)[N,K]^T ),
//     dq(W)[n,k] = bf16( (nibble(n,k) - 8) * float(scale[n, k / G]) )      (one rounding, as the reference's dq_bf16)
// x bf16, fp32 accumulation in tensor memory, bf16 out. The weights stay int4 in HBM and are expanded on the way to the tensor
// core: nothing the size of the bf16 weight matrix is ever written.
//
// Persistent CTA pairs (clusters of two, tcgen05 cta_group::2), one pair per two SMs. The product is computed transposed,
// yT[n, m] = dq(W)[n, :] . x[m, :], with the WEIGHTS as the MMA's A operand, read from tensor memory: a dequantising thread owns one
// weight row = one TMEM lane and writes its 64 expanded values straight into tensor memory (tcgen05.st), so the expansion never
// passes through shared memory, and the activations (the B operand, from shared memory) are the only operand the tensor cores
// fetch there. (Expanding into a shared-memory tile instead left the tensor pipe at 44-48 %: tile writes, operand reads and TMA
// fills together saturate shared-memory bandwidth.) A pair's tile is 256 weight rows x 256 tokens: CTA r expands weight rows
// [128 r, 128 r + 128) and loads tokens [128 r, 128 r + 128) of the tile; the leader issues one M = 256, N = 256 MMA per 16 of K
// and each CTA keeps the accumulator of its own weight rows (128 lanes x 256 token columns). K in steps of 64. 14 warps per CTA:
//   warp 0     one lane: TMA loads of this CTA's half of the activation tile (128 tokens x 128 B, swizzled; completes on the
//              leader's barrier) and raw weight tile (128 rows x 32 B; completes on this CTA's barrier) into a 6-stage ring
//   warps 6-13 dequantisers in two groups of four warps that take alternate K steps, thread = weight row = TMEM lane:
//              64 nibbles -> 64 bf16 (32 packed columns of the stage's slot in tensor memory), two weights per instruction in
//              packed bf16 arithmetic that rounds the exact product (n - 8) * scale once (see the loop)
//   warp 1     leader only, one lane: tcgen05.mma (A from tensor memory), 4 x (M=256, N=256, K=16) per step, and one commit per
//              step (multicast to both CTAs) that frees the stage for the loader and the dequantisers alike
//   warps 2-5  epilogue: TMEM -> bf16 -> transposed into swizzled staging (lane pairs exchange so that every store is a pair of
//              neighbouring output channels) -> TMA store
// Tensor memory: one accumulator (256 columns) + 6 weight slots of 32 columns; the epilogue frees the accumulator as soon as its last
// chunk is in registers (a staging buffer per chunk, so no chunk waits for an earlier chunk's store): about 5 % of a tile's main
// loop at K = 5120, while loads and expansion run ahead through the ring.
// K order per output element is ascending and the tile shape does not depend on M: rows are batch-invariant.
#include <algorithm>
#include <atomic>
#include "gemm_tc.cuh"
#include "host_util.h"

namespace spinf {

template <int TOK>
struct W4Smem {
  // stage s: activation half tile + raw weight tile in shared memory, expansion in TMEM. The narrow tile (TOK = 64) moves 8 KB per
  // stage instead of 20: twice the stages keep as many weight bytes in flight per SM as the wide tile's ring (a few-row call is a
  // weight stream bound by the bytes in flight, not by the tensor pipe)
  static constexpr int STAGES = TOK == 256 ? 6 : 12;
  static constexpr int EPI_BUFS = 4;          // one staging buffer per 64-token chunk of a tile: no chunk waits for an earlier store
  static constexpr int X_BYTES = TOK / 2 * 128;  // this CTA's activations: TOK / 2 tokens x 64 bf16
  static constexpr int RAW_BYTES = 128 * 32;  // this CTA's raw weights: 128 rows x 64 nibbles
  static constexpr int STAGE_BYTES = X_BYTES + RAW_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr int EPI_BYTES = 64 * 256;  // one staging buffer: 64 tokens x 128 output channels (two swizzled 64 x 64 boxes)
  static constexpr int BAR_OFF = EPI_OFF + EPI_BUFS * EPI_BYTES;
  static constexpr int TOTAL = BAR_OFF + 1024 + 1024;  // barriers: (5 STAGES + 2) x 8 B, then the tensor-memory base and the abort flag
  static constexpr uint32_t ACC_COL = 0, W_COL = TOK;  // tensor-memory columns: accumulator (TOK), weight slots (32 columns each)
  static_assert(W_COL + STAGES * 32 <= 512, "accumulator and weight slots fit tensor memory");
  static_assert((5 * STAGES + 2) * 8 + 8 <= 1024, "barriers fit their area");
};
static_assert(W4Smem<256>::STAGE_BYTES % 1024 == 0 && W4Smem<64>::STAGE_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");

struct W4Args {
  const __half* scales;  // [N, K / G]
  int M, N, K, G;
  int tiles_m, tiles_n, group_m;  // tiles of 256 tokens x 256 output channels
  // split-K (a decoding step's few rows, where the column tiles alone do not fill the GPU): a work unit is (tile, K slice of kb_per
  // steps); the epilogue writes the slice's fp32 sums to part[slice][m][n] and a second kernel adds the slices in order. splits = 1,
  // part = nullptr: the plain kernel.
  int splits, kb_per;
  float* part;
};


// ACT: -1 = plain linear; 0 / 1 = gated linear unit in the epilogue (GELU-tanh / SiLU): the weight rows are interleaved at load
// time (row 2c = gate channel c, row 2c + 1 = up channel c), so a lane pair of the epilogue holds a channel's gate and up values
// and writes y[m, c] = bf16(bf16(act(bf16 gate)) * bf16 up): the arithmetic of the linear followed by the gated-activation pass,
// without the [M, 2F] intermediate.
// TOK: tokens per tile = the MMA's N: 256, or 64 for calls of at most 64 rows (a decoding step), where a 256-wide product would
// spend four times the tensor-pipe time on rows that do not exist; each CTA then loads 32 token rows per stage and the epilogue
// has one 64-token chunk. An output element's sum over K is the same sequence of products either way.
// COARSE: the scale group is a multiple of the 64-wide K step (one scale per step, known at compile time so that the expansion loop
// has no branch in it).
template <int ACT, int TOK, bool COARSE>
__global__ void __launch_bounds__(448, 1)
w4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmC,
               const W4Args a, int* __restrict__ status) {
  using L = W4Smem<TOK>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t IDESC = make_idesc(FMT_BF16, FMT_BF16, 256, TOK, 0, 0);  // M = weight rows, N = tokens (K-major in shared memory)
  constexpr int HALF = TOK / 2;            // token rows of a tile this CTA loads
  constexpr int CHUNKS = TOK / 64;         // 64-token chunks of the epilogue
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);  // leader's: both halves of the activation tile landed
  uint64_t* full_w = full_a + STAGES;                                  // this CTA's raw weight tile landed
  uint64_t* mma_done = full_w + STAGES;                                // 1 MMA commit: the stage's MMAs have read their operands
  uint64_t* raw_done = mma_done + STAGES;                              // 4 arrivals of this CTA's dequantiser warps: raw tile read
  uint64_t* b_full = raw_done + STAGES;                                // leader's: 4 dequantiser-warp arrivals from each CTA
  uint64_t* acc_full = b_full + STAGES;                                // 1 MMA commit
  uint64_t* acc_empty = acc_full + 1;                                  // leader's: 4 epilogue-warp arrivals from each CTA
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_p + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, status};
  const uint32_t rank = cluster_ctarank();
  const int pair0 = static_cast<int>(blockIdx.x) >> 1, pair_step = static_cast<int>(gridDim.x) >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_a[s], 1);
      mbar_init(&full_w[s], 1);
      mbar_init(&mma_done[s], 1);
      mbar_init(&raw_done[s], 4);
      mbar_init(&b_full[s], 8);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {  // the same warp in both CTAs allocates the pair's tensor memory
    tmem_alloc_pair(tmem_base_p, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival or peer-signalled copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_p;
  GemmShape shape;
  shape.M = a.M, shape.N = a.N, shape.K = a.K, shape.tiles_m = a.tiles_m, shape.tiles_n = a.tiles_n, shape.group_m = a.group_m;
  const int num_tiles = a.tiles_m * a.tiles_n * a.splits;  // work units: tile-major, a tile's K slices next to one another

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair0; tile < num_tiles && ok; tile += pair_step) {
        int tm, tn;
        tile_coords(shape, tile / a.splits, tm, tn);
        const int kb0 = (tile % a.splits) * a.kb_per;
        for (int kb = kb0; kb < kb0 + a.kb_per; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(wc, &mma_done[s], ph ^ 1u, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          if (!mbar_wait(wc, &raw_done[s], ph ^ 1u, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_a[s], 2 * L::X_BYTES);  // the leader's barrier counts both CTAs' activation bytes
          tma_load_2d_pair(sa, &tmA, kb * 64, tm * TOK + static_cast<int>(rank) * HALF, map_to_cta(&full_a[s], 0));
          mbar_expect_tx(&full_w[s], L::RAW_BYTES);
          tma_load_2d(sa + L::X_BYTES, &tmW, kb * 32, tn * 256 + static_cast<int>(rank) * 128, &full_w[s]);
        }
      }
      if (!ok) {  // bounded wait for this CTA's raw-weight copies that may still be in flight (activation copies complete on the
                  // leader's barriers; the cluster barrier at the end keeps both CTAs resident meanwhile)
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(&full_w[j % STAGES], (j / STAGES) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair0; tile < num_tiles && ok; tile += pair_step, ++tcount) {
        if (!mbar_wait(wc, acc_empty, (tcount & 1u) ^ 1u, ST_TIMEOUT_TMEM)) { ok = false; break; }
        tc_fence_after();
        const int kb0 = (tile % a.splits) * a.kb_per;
        for (int kb = kb0; kb < kb0 + a.kb_per; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(wc, &full_a[s], ph, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (!mbar_wait(wc, &b_full[s], ph, ST_TIMEOUT_OTHER)) { ok = false; break; }
          tc_fence_after();
          const uint64_t xdesc = make_smem_desc_sw128(smem_u32(smem + s * L::STAGE_BYTES), 16, 1024);
          const uint32_t w_tmem = tmem_base + L::W_COL + s * 32;  // 16 bf16 of K = 8 packed columns per MMA
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16_ts_pair(tmem_base + L::ACC_COL, w_tmem + 8 * k, xdesc + 2 * k, IDESC, kb != kb0 || k != 0);
          umma_commit_pair_both(&mma_done[s]);  // one commit per step: every commit is a bubble in the tensor pipe
        }
        if (ok) umma_commit_pair_both(acc_full);
      }
    }
  } else if (warp >= 6) {
    // dequantisers: two groups of 128 threads take alternate K steps; thread = weight row of the tile
    const int grp = (warp - 6) >> 2;
    const int n_local = (warp & 3) * 32 + lane;  // a warp reaches the 32 TMEM lanes of its quarter (warp index mod 4)
    uint32_t it = 0;
    bool ok = true;
    const int groups = a.K / a.G;
    constexpr bool coarse = COARSE;
    const uint32_t b_full_leader = map_to_cta(b_full, 0);
    for (int tile = pair0; tile < num_tiles && ok; tile += pair_step) {
      int tm, tn;
      tile_coords(shape, tile / a.splits, tm, tn);
      const int kb0 = (tile % a.splits) * a.kb_per;
      const int n = tn * 256 + static_cast<int>(rank) * 128 + n_local;
      const bool n_ok = n < a.N;
      const __half* srow = a.scales + static_cast<int64_t>(n_ok ? n : 0) * groups;
      int s_idx = -1;
      uint32_t s_hi2 = 0u, s_lo2 = 0u;  // the group's scale as two packed bf16 pairs: its top 8 significant bits and the rest
      auto load_scale = [&](int gi) {
        // a half-precision scale has 11 significant bits: the bf16 truncation keeps 8, the remainder (at most 3 bits) is a bf16 too
        const float sc = n_ok ? __half2float(srow[gi]) : 0.f;
        const uint32_t hi = __float_as_uint(sc) >> 16;
        const uint32_t lo = __float_as_uint(sc - __uint_as_float(hi << 16)) >> 16;
        s_hi2 = hi | (hi << 16), s_lo2 = lo | (lo << 16);
      };
      for (int kb = kb0; kb < kb0 + a.kb_per; ++kb, ++it) {
        if ((it & 1u) != static_cast<uint32_t>(grp)) continue;
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        bool got = mbar_wait(wc, &full_w[s], ph, ST_TIMEOUT_FULL);
        got = got && mbar_wait(wc, &mma_done[s], ph ^ 1u, ST_TIMEOUT_EMPTY);  // the stage's previous expansion has been consumed
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        const uint4* raw = reinterpret_cast<const uint4*>(smem + s * L::STAGE_BYTES + L::X_BYTES + n_local * 32);
        const uint4 r0 = raw[0], r1 = raw[1];
        const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        uint32_t out[32];  // column j of the slot = K elements (2 j, 2 j + 1) of this row
        if (coarse) {  // one scale for the whole 64-wide K step (group a multiple of 64): one division per step
          const int gi = (kb * 64) / a.G;
          if (gi != s_idx) {
            s_idx = gi;
            load_scale(gi);
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 8 nibbles -> 8 bf16 = one 16-byte chunk of the row
          if (!coarse) {
            const int gi = (kb * 64 + c * 8) / a.G;
            if (gi != s_idx) {
              s_idx = gi;
              load_scale(gi);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // the word holds its even k in the low half and its odd k in the high half (spinf_w4_repack), so one shift and one
            // mask-or give the pair (k, k + 1) as the packed bf16 values 128 + nibble (0x4300 | nibble); d = nibble - 8 exactly;
            // d * s_lo is exact (4 x 3 bits), and fma(d, s_hi, d * s_lo) rounds the exact product d * s once: the reference's
            // bf16((nibble - 8) * scale), two weights per instruction and no conversion
            const uint32_t v = ((words[c] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
            const uint32_t d = bf2_sub(v, 0x43084308u);
            out[4 * c + j] = bf2_fma(d, s_hi2, bf2_mul(d, s_lo2));
          }
        }
        tc_fence_after();  // orders the store after the commit that freed the slot
        tmem_st_x32(tmem_base + L::W_COL + s * 32 + (static_cast<uint32_t>((warp & 3) * 32) << 16), out);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();  // every lane's row is in tensor memory: one arrival per warp instead of 32
        if (lane == 0) {
          mbar_arrive_cluster(b_full_leader + s * 8);  // the leader's barrier: the pair's MMA reads both CTAs' slots
          mbar_arrive(&raw_done[s]);                   // the raw tile has been read
        }
      }
    }
  } else {
    // epilogue: warps 2-5, thread = TMEM lane = output channel of this CTA's 128; columns = the tile's 256 tokens
    const int et = threadIdx.x - 64;
    const uint32_t acc_empty_leader = map_to_cta(acc_empty, 0);
    const int q = warp & 3;
    const int ch = q * 32 + lane;            // output channel within this CTA's 128
    const int hb = ch >> 6;                  // which 64-channel box of the staging buffer
    const int ch2 = (ch & 63) & ~1;          // the even channel of this lane pair, within the box
    const uint32_t odd = lane & 1u;
    uint32_t tcount = 0, nchunks = 0;
    for (int tile = pair0; tile < num_tiles; tile += pair_step, ++tcount) {
      int tm, tn;
      tile_coords(shape, tile / a.splits, tm, tn);
      const int ks = tile % a.splits;
      const bool got = mbar_wait(wc, acc_full, tcount & 1u, ST_TIMEOUT_TMEM);
      if (!bar_red_and(1, 128, got)) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < CHUNKS; ++c, ++nchunks) {  // 64-token chunks
        uint32_t v0[32], v1[32];
        __syncwarp();
        const uint32_t taddr = tmem_base + L::ACC_COL + c * 64 + (static_cast<uint32_t>(q * 32) << 16);
        tmem_ld_x32(taddr, v0);
        tmem_ld_x32(taddr + 32, v1);
        tmem_wait_ld();
        if (c == CHUNKS - 1) {  // the accumulator is in registers: one arrival per warp on the leader's barrier
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        }
        if (ACT < 0 && a.part != nullptr) {
          // a K slice's sums, fp32, straight to part[slice][token][channel]: a warp's lanes are 32 neighbouring channels
          const int n = tn * 256 + static_cast<int>(rank) * 128 + ch;
          float* const dst = a.part + (static_cast<int64_t>(ks) * a.M + tm * TOK + c * 64) * a.N + n;
          const int rows = a.M - (tm * TOK + c * 64);  // tokens of this chunk that exist
          if (n < a.N) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i < rows) dst[static_cast<int64_t>(i) * a.N] = __uint_as_float(v0[i]);
              if (32 + i < rows) dst[static_cast<int64_t>(32 + i) * a.N] = __uint_as_float(v1[i]);
            }
          }
          continue;
        }
        // transpose through the lane pair: the even lane keeps token 2 i of both channels, the odd lane token 2 i + 1
        uint32_t packed[32];
        uint8_t* buf = smem + L::EPI_OFF + (nchunks % L::EPI_BUFS) * L::EPI_BYTES;
        if (ACT < 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t e = i < 16 ? v0[2 * i] : v1[2 * i - 32], o = i < 16 ? v0[2 * i + 1] : v1[2 * i - 31];
            const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? e : o, 1);
            packed[i] = odd ? pack_bf16x2(__uint_as_float(other), __uint_as_float(o)) : pack_bf16x2(__uint_as_float(e), __uint_as_float(other));
          }
        } else {
          // the lane pair is (gate, up) of one output channel: after the exchange both values of token 2 i + odd are here
          float yv[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t e = i < 16 ? v0[2 * i] : v1[2 * i - 32], o = i < 16 ? v0[2 * i + 1] : v1[2 * i - 31];
            const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? e : o, 1);
            const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(odd ? other : e)));
            const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(odd ? o : other)));
            const float act = ACT == 0 ? gelu_tanh_f32(g) : silu_f32(g);
            yv[i] = __bfloat162float(__float2bfloat16_rn(act)) * u;  // the product of two bf16 values is exact in fp32: rounded by the pack
          }
          // second exchange, with the neighbouring channel's lane pair: even channels keep their even i, odd channels their odd i
          const bool oddc = (lane & 2u) != 0u;
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            const float keep = oddc ? yv[2 * h + 1] : yv[2 * h], send = oddc ? yv[2 * h] : yv[2 * h + 1];
            const float other = __shfl_xor_sync(0xffffffffu, send, 2);
            packed[h] = oddc ? pack_bf16x2(other, keep) : pack_bf16x2(keep, other);
          }
        }
        if (et == 0) tma_store_wait_read<L::EPI_BUFS - 1>();  // the store that last read this buffer (a tile ago) has finished reading
        named_bar_sync(1, 128);
        if (ACT < 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t tok = 2 * i + odd;
            *reinterpret_cast<uint32_t*>(buf + hb * 8192 + sw128_offset(tok, ch2 >> 3) + (ch2 & 7) * 2) = packed[i];
          }
        } else {
          const int oc2 = (ch >> 1) & ~1;  // the even one of the two output channels this lane writes, within the CTA's 64
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            const uint32_t tok = 2 * (2 * h + ((lane >> 1) & 1u)) + odd;
            *reinterpret_cast<uint32_t*>(buf + sw128_offset(tok, oc2 >> 3) + (oc2 & 7) * 2) = packed[h];
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (et == 0) {
          const int m0 = tm * TOK + c * 64;
          if (ACT < 0) {
            const int n0 = tn * 256 + static_cast<int>(rank) * 128;
            if (m0 < a.M && n0 < a.N) tma_store_2d(&tmC, buf, n0, m0);  // boxes that lie wholly outside the output are skipped,
            if (m0 < a.M && n0 + 64 < a.N) tma_store_2d(&tmC, buf + 8192, n0 + 64, m0);  // partial ones are clipped by the copy
          } else {
            const int f0 = tn * 128 + static_cast<int>(rank) * 64;  // 128 interleaved weight rows = 64 output channels
            if (m0 < a.M && f0 < a.N / 2) tma_store_2d(&tmC, buf, f0, m0);
          }
          tma_store_commit();
        }
      }
    }
    if (et == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its peer may still signal its barriers or read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Load-time re-ordering of the packed weights for the kernel above. In: the reference's engine layout (byte b of a row holds k = 2b
// in its low nibble and k = 2b + 1 in its high nibble, qwen.py:383-389), read as 32-bit words of 8 consecutive k. Out: the same
// word with its even k in nibbles 0..3 and its odd k in nibbles 4..7, so that (word >> 4j) & 0x000F000F is the pair (2j, 2j + 1).
__global__ void __launch_bounds__(256) w4_repack_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int64_t n_words) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_words; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint32_t w = in[i];
    uint32_t r = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      r |= ((w >> (8 * j)) & 0xFu) << (4 * j);             // k = 2j
      r |= ((w >> (8 * j + 4)) & 0xFu) << (16 + 4 * j);    // k = 2j + 1
    }
    out[i] = r;
  }
}

// y[m][n] = bf16(sum over the K slices, in slice order, of part[slice][m][n])
__global__ void w4_splitk_sum_kernel(const float* __restrict__ part, int splits, int64_t MN, int N, __nv_bfloat16* __restrict__ y, int64_t y_pitch) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= MN) return;
  float t = part[i];
  for (int sp = 1; sp < splits; ++sp) t += part[sp * MN + i];
  y[(i / N) * y_pitch + i % N] = __float2bfloat16_rn(t);
}

// K slices for a product of M <= 256 rows: as many as bring the work units (column tiles x slices) up to the number of CTA pairs,
// a count that divides the K steps
static int w4_splits(int64_t N, int64_t K) {
  const int tiles_n = static_cast<int>((N + 255) / 256), pairs = sm_count() / 2, num_kb = static_cast<int>(K / 64);
  int splits = std::max(1, std::min(num_kb, pairs / tiles_n));
  while (num_kb % splits) --splits;
  return splits;
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_w4_repack(const void* q_in, void* q_out, int64_t N, int64_t K, void* stream) {
  if (N == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(q_in && q_out && N >= 0 && K > 0 && K % 8 == 0);
  SPINF_CHECK_ARG((reinterpret_cast<uintptr_t>(q_in) & 3) == 0 && (reinterpret_cast<uintptr_t>(q_out) & 3) == 0);
  const int64_t n_words = N * (K / 8);
  if (n_words == 0) return 0;
  const int64_t blocks = (n_words + 255) / 256, cap = 16ll * sm_count();
  w4_repack_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(q_in), static_cast<uint32_t*>(q_out), n_words);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int ACT>
static int launch_w4(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                     int64_t y_pitch, void* stream, int splits = 1, float* part = nullptr) {
  if (M == 0) return 0;  // nothing to do: the row pointers may be null
  const int64_t n_out = ACT < 0 ? N : N / 2;
  SPINF_CHECK_ARG(x && qw && scales && y && M >= 0 && N > 0 && K > 0 && group > 0);
  SPINF_CHECK_ARG(K % 64 == 0 && group % 8 == 0 && K % group == 0 && N % (ACT < 0 ? 8 : 16) == 0 && y_pitch >= n_out && y_pitch % 8 == 0);
  SPINF_CHECK_ARG(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31));
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  CUtensorMap tmA, tmW, tmC;
  int r;
  const int TOK = M <= 64 ? 64 : 256;  // tokens per tile (the kernel's TOK)
  if ((r = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, K * 2, 64, TOK / 2))) return r;
  if ((r = make_tmap_2d_plain(&tmW, qw, N, K / 2, K / 2, 32, 128))) return r;
  if ((r = make_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, M, n_out, y_pitch * 2, 64, 64))) return r;
  W4Args a;
  a.scales = static_cast<const __half*>(scales);
  a.M = static_cast<int>(M), a.N = static_cast<int>(N), a.K = static_cast<int>(K), a.G = group;
  a.tiles_m = static_cast<int>((M + TOK - 1) / TOK);
  a.tiles_n = static_cast<int>((N + 255) / 256);
  a.splits = splits, a.kb_per = static_cast<int>(K / 64) / splits, a.part = part;
  // groups of row tiles as tall as about 32 MB of bf16 activations allow (4..32 tiles of 256 rows): the packed weight streams past
  // once per group
  {
    const int64_t per_tile = 256 * K * 2;
    const int64_t g = (32ll << 20) / per_tile;
    a.group_m = static_cast<int>(g < 4 ? 4 : (g > 32 ? 32 : g));
  }
  const bool coarse = group % 64 == 0;
  auto kern = TOK == 64 ? (coarse ? w4_gemm_kernel<ACT, 64, true> : w4_gemm_kernel<ACT, 64, false>)
                        : (coarse ? w4_gemm_kernel<ACT, 256, true> : w4_gemm_kernel<ACT, 256, false>);
  static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice from two threads is harmless
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_gemm_kernel<ACT, 64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Smem<256>::TOTAL));
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_gemm_kernel<ACT, 64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Smem<256>::TOTAL));
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_gemm_kernel<ACT, 256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Smem<256>::TOTAL));
    SPINF_CUDA_OK(cudaFuncSetAttribute(w4_gemm_kernel<ACT, 256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Smem<256>::TOTAL));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int tiles = a.tiles_m * a.tiles_n * a.splits;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(448);
  cfg.dynamicSmemBytes = W4Smem<256>::TOTAL;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SPINF_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmA, tmW, tmC, a, status));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_w4_gemm(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                             int64_t y_pitch, void* stream) {
  return launch_w4<-1>(x, qw, scales, group, y, M, N, K, y_pitch, stream);
}

extern "C" int spinf_w4_gemm_glu(const void* x, const void* qw, const void* scales, int32_t group, int32_t act, void* y, int64_t M,
                                 int64_t N2, int64_t K, int64_t y_pitch, void* stream) {
  SPINF_CHECK_ARG(act == 0 || act == 1);
  return act == 0 ? launch_w4<0>(x, qw, scales, group, y, M, N2, K, y_pitch, stream)
                  : launch_w4<1>(x, qw, scales, group, y, M, N2, K, y_pitch, stream);
}


// bytes of workspace spinf_w4_gemm_small needs (0: the shape needs no split)
extern "C" int64_t spinf_w4_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 64) return 0;
  const int splits = w4_splits(N, K);
  return splits > 1 ? static_cast<int64_t>(splits) * M * N * 4 + 256 : 0;
}

extern "C" int spinf_w4_gemm_small(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                                   int64_t y_pitch, void* workspace, int64_t workspace_bytes, void* stream) {
  if (M == 0) return 0;
  SPINF_CHECK_ARG(M > 0 && M <= 256 && N > 0 && K > 0 && K % 64 == 0);
  const int splits = w4_splits(N, K);
  if (splits == 1) return launch_w4<-1>(x, qw, scales, group, y, M, N, K, y_pitch, stream);
  SPINF_CHECK_ARG(workspace && workspace_bytes >= spinf_w4_gemm_small_workspace_bytes(M, N, K));
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  ws += (256 - reinterpret_cast<uintptr_t>(ws) % 256) % 256;
  float* const part = reinterpret_cast<float*>(ws);
  const int r = launch_w4<-1>(x, qw, scales, group, y, M, N, K, y_pitch, stream, splits, part);
  if (r) return r;
  const int64_t MN = M * N;
  w4_splitk_sum_kernel<<<static_cast<unsigned>((MN + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      part, splits, MN, static_cast<int>(N), static_cast<__nv_bfloat16*>(y), y_pitch);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
