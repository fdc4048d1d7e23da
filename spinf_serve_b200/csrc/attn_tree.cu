// Tree-mask attention over one packed stream (prefill), tcgen05 + TMEM + TMA, for sm_100a.
//
// One CTA = one 128-row query block of one query head. It walks the block's tile list (built on the host from the packing
// metadata, copied to shared memory at start) in ascending key order, 64 keys at a time:
//   warp 0    one lane: TMA loads of Q (once) and of the K sub-tiles into a 2-deep ring, released as soon as S = Q K^T has read them
//   warp 6    one lane: TMA loads of the V sub-tiles into their own 2-deep ring, released when O += P V has read them
//   warp 1    allocates tensor memory; one lane issues  S = Q K^T  (M=128, N=64, K=D)  into one of two S buffers and
//             O += P V  (M=128, N=D, K=64)  into the O accumulator; S of sub-tile t+1 is issued before P V of sub-tile t, so the
//             tensor core works on the next scores while the softmax warps work on the current ones
//   warps 2-5 thread = query row: reads S from TMEM, applies scale and the tree mask, keeps the running reference maximum and
//             the sum in fp32, writes P (bf16) into a swizzled shared tile, and at the end divides O by the sum and stores bf16.
//             O is rescaled in TMEM only when a row's maximum grew by more than 2^8 since its reference maximum was last moved
//             (probabilities then stay below 256, exact in the final division); the decision depends on the row's own scores only.
// Numerics follow the reference's attention (bf16 Q/K/V, fp32 scores and softmax state, P rounded to bf16 before P V, fp32
// accumulation). Reduction order per row = ascending 64-key sub-tiles of the row's own job, independent of what else is packed
// in the stream; tiles flagged "no mask" only skip the mask evaluation, never change the arithmetic.
#include "common.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int KT = 64;          // keys per sub-tile
static constexpr int LIST_CAP = 512;   // tile-list entries kept in shared memory (longer lists read the rest from global)
static constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

template <int D>
struct AttnSmem {
  static constexpr int SLABS = D / 64;              // 64-element (128-byte) slabs along the head dimension
  static constexpr int Q_BYTES = SLABS * 128 * 128;
  static constexpr int KV_TILE = SLABS * KT * 128;  // one K (or V) sub-tile
  static constexpr int P_BYTES = 128 * 128;
  static constexpr int K_OFF = Q_BYTES;             // 2 stages of K then 2 stages of V
  static constexpr int V_OFF = K_OFF + 2 * KV_TILE;
  static constexpr int P_OFF = V_OFF + 2 * KV_TILE;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int LIST_OFF = BAR_OFF + 128;            // LIST_CAP ints + LIST_CAP bytes
  static constexpr int META_OFF = LIST_OFF + LIST_CAP * 5;  // per softmax warp: 2 buffers x 3 arrays x 64 ints
  static constexpr int TOTAL = META_OFF + 4 * 2 * 3 * KT * 4 + 1024;
  static constexpr int TMEM_COLS = D == 256 ? 512 : 256;    // 2 x 64 (S) + D (O), rounded up to a power of two
  static constexpr int O_COL = 128;
};

struct AttnArgs {
  __nv_bfloat16* out;
  int64_t out_pitch;
  const int32_t* art;
  const int32_t* end;
  const int32_t* pos;
  const int32_t* tile_offsets;
  const int32_t* tile_blocks;
  const uint8_t* tile_flags;  // bit 0: every pair attends under the tree rule; bit 1: no mask evaluation needed (window included)
  int nb, H, group;           // group = H / Hkv
  int window;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(224, 1)
tree_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs a, int* __restrict__ status) {
  using L = AttnSmem<D>;
  constexpr int SLABS = L::SLABS;
  constexpr uint32_t IDESC_S = make_idesc(FMT_BF16, FMT_BF16, 128, KT, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc(FMT_BF16, FMT_BF16, 128, D, 0, 1);  // B = V, MN-major (head dim contiguous)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // 2
  uint64_t* v_full = bars + 3;     // 2
  uint64_t* k_empty = bars + 5;    // 2
  uint64_t* v_empty = bars + 7;    // 2
  uint64_t* s_full = bars + 9;     // 2
  uint64_t* p_ready = bars + 11;   // 1 (128 arrivals)
  uint64_t* o_done = bars + 12;    // 1
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_p + 1);
  int* list_blocks = reinterpret_cast<int*>(smem + L::LIST_OFF);
  uint8_t* list_flags = smem + L::LIST_OFF + LIST_CAP * 4;
  int* meta = reinterpret_cast<int*>(smem + L::META_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y;
  const int g = h / a.group;
  const WaitCtx wc{abort_flag, status};
  const int e0 = a.tile_offsets[qb];
  const int n_tiles = a.tile_offsets[qb + 1] - e0;
  const int n_sub = 2 * n_tiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_p, L::TMEM_COLS);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < n_tiles && i < LIST_CAP; i += blockDim.x) {
    list_blocks[i] = a.tile_blocks[e0 + i];
    list_flags[i] = a.tile_flags[e0 + i];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_p;
  auto block_of = [&](int tile) { return tile < LIST_CAP ? list_blocks[tile] : a.tile_blocks[e0 + tile]; };
  auto flags_of = [&](int tile) { return tile < LIST_CAP ? list_flags[tile] : a.tile_flags[e0 + tile]; };

  if (warp == 0 || warp == 6) {
    // K producer (warp 0, also loads Q) and V producer (warp 6): one lane each
    if (lane == 0 && n_sub > 0) {
      const bool is_k = warp == 0;
      uint64_t* full = is_k ? k_full : v_full;
      uint64_t* empty = is_k ? k_empty : v_empty;
      const CUtensorMap* tm = is_k ? &tmK : &tmV;
      const int base = is_k ? L::K_OFF : L::V_OFF;
      if (is_k) {
        mbar_expect_tx(q_full, L::Q_BYTES);
        for (int s = 0; s < SLABS; ++s) tma_load_2d(smem + s * 128 * 128, &tmQ, h * D + s * 64, qb * 128, q_full);
      }
      int issued = 0;
      for (int t = 0; t < n_sub; ++t, ++issued) {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1u;
        const int j = block_of(t >> 1);
        if (j < 0 || j >= a.nb) {
          *abort_flag = 1;
          atomicCAS(status, 0, ST_BAD_INDEX);
          break;
        }
        if (!mbar_wait(wc, &empty[st], ph ^ 1u, ST_TIMEOUT_EMPTY)) break;
        const int kv0 = j * 128 + (t & 1) * KT;
        mbar_expect_tx(&full[st], L::KV_TILE);
        for (int s = 0; s < SLABS; ++s) tma_load_2d(smem + base + st * L::KV_TILE + s * KT * 128, tm, g * D + s * 64, kv0, &full[st]);
      }
      if (*abort_flag) {
        // bounded wait for copies of this CTA that may still be in flight
        if (is_k)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(q_full, 0); ++spin) {}
        for (int t = issued > 2 ? issued - 2 : 0; t < issued; ++t)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(&full[t & 1], (t >> 1) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_sub > 0) {
      const uint32_t q_addr = smem_u32(smem);
      const uint32_t p_addr = smem_u32(smem + L::P_OFF);
      auto issue_s = [&](int t) {
        const int st = t & 1;
        const uint32_t k_addr = smem_u32(smem + L::K_OFF + st * L::KV_TILE);
        const uint32_t d_tmem = tmem_base + (t & 1) * KT;
#pragma unroll
        for (int s = 0; s < SLABS; ++s) {
          const uint64_t ad = make_smem_desc_sw128(q_addr + s * 128 * 128, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(k_addr + s * KT * 128, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16_ss(d_tmem, ad + 2 * k, bd + 2 * k, IDESC_S, (s | k) != 0);
        }
        umma_commit(&k_empty[st]);       // the K stage may be refilled as soon as these MMAs have read it
        umma_commit(&s_full[t & 1]);
      };
      bool ok = mbar_wait(wc, q_full, 0, ST_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(wc, &k_full[0], 0, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int t = 0; t < n_sub && ok; ++t) {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1u;
        if (t + 1 < n_sub) {
          // S buffer (t+1)&1 was last read by the softmax of sub-tile t-1, which arrived on p_ready before P V (t-1) was issued
          if (!mbar_wait(wc, &k_full[(t + 1) & 1], ((t + 1) >> 1) & 1u, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
          issue_s(t + 1);
        }
        if (!mbar_wait(wc, p_ready, t & 1u, ST_TIMEOUT_OTHER)) break;
        if (!mbar_wait(wc, &v_full[st], ph, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + L::V_OFF + st * L::KV_TILE);
        const uint64_t pd = make_smem_desc_sw128(p_addr, 16, 1024);
        // V sub-tile: slab s holds head-dim columns [64 s, 64 s + 64) of 64 keys, one key per 128-byte row:
        // MN-major B operand, 64-column groups KT*128 bytes apart (LBO), 8-key groups 1024 bytes apart (SBO)
        const uint64_t vd = make_smem_desc_sw128(v_addr, KT * 128, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 keys per step: 32 bytes along P's rows, 16 rows (2048 bytes) down V
          umma_f16_ss(tmem_base + L::O_COL, pd + 2 * k, vd + 128 * k, IDESC_O, (t | k) != 0);
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
    }
  } else if (n_sub > 0) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int tq = qb * 128 + row;  // stream position of this thread's query row
    const int art_q = a.art[tq], pos_q = a.pos[tq];
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* p_smem = smem + L::P_OFF;
    int* wmeta = meta + (warp - 2) * 2 * 3 * KT;  // this warp's private copies of the key metadata
    float m_ref = -INFINITY, l_run = 0.f;
    bool alive = true;

    // key metadata of sub-tile t (art, end, pos of its 64 keys): each lane fetches 2 keys one iteration ahead
    int pre[6] = {0, 0, 0, 0, 0, 0};
    auto fetch_meta = [&](int t) {
      const int j = block_of(t >> 1);
      if (!(flags_of(t >> 1) & 2) && j >= 0 && j < a.nb) {
        const int kv0 = j * 128 + (t & 1) * KT;
        pre[0] = a.art[kv0 + lane], pre[1] = a.art[kv0 + 32 + lane];
        pre[2] = a.end[kv0 + lane], pre[3] = a.end[kv0 + 32 + lane];
        pre[4] = a.pos[kv0 + lane], pre[5] = a.pos[kv0 + 32 + lane];
      }
    };
    auto stash_meta = [&](int t) {
      int* mb = wmeta + (t & 1) * 3 * KT;
      mb[lane] = pre[0], mb[32 + lane] = pre[1];
      mb[KT + lane] = pre[2], mb[KT + 32 + lane] = pre[3];
      mb[2 * KT + lane] = pre[4], mb[2 * KT + 32 + lane] = pre[5];
    };
    fetch_meta(0);
    stash_meta(0);
    __syncwarp();

    for (int t = 0; t < n_sub; ++t) {
      const int j = block_of(t >> 1);
      const bool no_mask = (flags_of(t >> 1) & 2) != 0;
      const int kv0 = j * 128 + (t & 1) * KT;
      const int* kart = wmeta + (t & 1) * 3 * KT;
      const int* kend = kart + KT;
      const int* kpos = kend + KT;
      if (t + 1 < n_sub) fetch_meta(t + 1);  // in flight while this sub-tile is processed
      bool got = j >= 0 && j < a.nb && mbar_wait(wc, &s_full[t & 1], (t >> 1) & 1u, ST_TIMEOUT_TMEM);
      if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld_x32(tmem_base + lane_off + (t & 1) * KT, v0);
      tmem_ld_x32(tmem_base + lane_off + (t & 1) * KT + 32, v1);
      tmem_wait_ld();
      float s[KT];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        s[i] = __uint_as_float(v0[i]) * a.scale_log2;
        s[32 + i] = __uint_as_float(v1[i]) * a.scale_log2;
      }
      if (!no_mask) {
        // branch-free: every operand is loaded unconditionally (vector loads of the warp's metadata copy), the rule is a chain
        // of bitwise ANDs; short-circuit evaluation here compiles to ~200 divergent branches per sub-tile
        const bool q_real = art_q >= 0;
        const bool windowed = a.window > 0;
#pragma unroll
        for (int i4 = 0; i4 < KT / 4; ++i4) {
          const int4 ka = reinterpret_cast<const int4*>(kart)[i4];
          const int4 ke = reinterpret_cast<const int4*>(kend)[i4];
          const int4 kp = reinterpret_cast<const int4*>(kpos)[i4];
          const int kas[4] = {ka.x, ka.y, ka.z, ka.w}, kes[4] = {ke.x, ke.y, ke.z, ke.w}, kps[4] = {kp.x, kp.y, kp.z, kp.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = 4 * i4 + u;
            const int tk = kv0 + i;
            const bool tree = (tk <= tq) & q_real & (kas[u] == art_q) & (tq < kes[u]);
            const bool win = !windowed | (pos_q - kps[u] < a.window);
            const bool vis = (tree & win) | (tk == tq);
            s[i] = vis ? s[i] : -INFINITY;
          }
        }
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < KT; ++i) mx = fmaxf(mx, s[i]);
      // move the reference maximum only when the row's maximum has grown by more than the threshold
      float alpha = 1.f;
      if (mx - m_ref > RESCALE_THRESHOLD) {  // false for NaN (-inf minus -inf): a row that has seen nothing yet
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f;
      uint32_t pk[KT / 2];
#pragma unroll
      for (int i = 0; i < KT / 2; ++i) {
        const float p0 = fast_exp2(s[2 * i] - m_use), p1 = fast_exp2(s[2 * i + 1] - m_use);
        sum += p0 + p1;
        pk[i] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + sum;
      if (t > 0) {
        // P V of the previous sub-tile has completed: the P tile may be overwritten and O is stable
        got = mbar_wait(wc, o_done, (t - 1) & 1u, ST_TIMEOUT_TMEM);
        if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(p_smem + sw128_offset(row, c)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_x32(tmem_base + lane_off + L::O_COL + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(tmem_base + lane_off + L::O_COL + c * 32, o);
        }
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      if (t + 1 < n_sub) {
        stash_meta(t + 1);  // buffer (t+1)&1 was last read in iteration t-1 by this warp only
        __syncwarp();
      }
    }

    if (alive) {
      const bool got = mbar_wait(wc, o_done, (n_sub - 1) & 1u, ST_TIMEOUT_TMEM);
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        const float inv = 1.f / l_run;  // every row sees at least itself, so l_run > 0
        __nv_bfloat16* dst = a.out + static_cast<int64_t>(tq) * a.out_pitch + h * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_x32(tmem_base + lane_off + L::O_COL + c * 32, o);
          tmem_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int D>
static int launch_attn(const void* q, const void* k, const void* v, int64_t n, int H, int Hkv, int64_t q_pitch, int64_t kv_pitch,
                       const AttnArgs& args, cudaStream_t stream) {
  using L = AttnSmem<D>;
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  CUtensorMap tmQ, tmK, tmV;
  int r;
  if ((r = make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, n, static_cast<uint64_t>(H) * D, q_pitch * 2, 64, 128))) return r;
  if ((r = make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, n, static_cast<uint64_t>(Hkv) * D, kv_pitch * 2, 64, KT))) return r;
  if ((r = make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v, n, static_cast<uint64_t>(Hkv) * D, kv_pitch * 2, 64, KT))) return r;
  auto kern = tree_attn_kernel<D>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_set[dev] = true;
  }
  dim3 grid(static_cast<unsigned>(n / 128), static_cast<unsigned>(H));
  kern<<<grid, 224, L::TOTAL, stream>>>(tmQ, tmK, tmV, args, status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_tree_attn_fwd(const void* q, const void* k, const void* v, void* out, int64_t n, int32_t H, int32_t Hkv,
                                   int32_t D, int64_t q_pitch, int64_t kv_pitch, int64_t out_pitch, const int32_t* art,
                                   const int32_t* end, const int32_t* pos, int32_t window, float scale, const int32_t* tile_offsets,
                                   const int32_t* tile_blocks, const uint8_t* tile_flags, void* stream) {
  SPINF_CHECK_ARG(q && k && v && out && art && end && pos && tile_offsets && tile_blocks && tile_flags);
  SPINF_CHECK_ARG(n >= 0 && n % SPINF_BLOCK == 0 && n < (1ll << 30) && H > 0 && Hkv > 0 && H % Hkv == 0 && H <= 65535);
  SPINF_CHECK_ARG(D == 128 || D == 256);
  SPINF_CHECK_ARG(q_pitch >= static_cast<int64_t>(H) * D && kv_pitch >= static_cast<int64_t>(Hkv) * D && out_pitch >= static_cast<int64_t>(H) * D);
  SPINF_CHECK_ARG(q_pitch % 8 == 0 && kv_pitch % 8 == 0 && out_pitch % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (n == 0) return 0;
  AttnArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.out_pitch = out_pitch;
  a.art = art;
  a.end = end;
  a.pos = pos;
  a.tile_offsets = tile_offsets;
  a.tile_blocks = tile_blocks;
  a.tile_flags = tile_flags;
  a.nb = static_cast<int>(n / SPINF_BLOCK);
  a.H = H;
  a.group = H / Hkv;
  a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 256) return launch_attn<256>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st);
  return launch_attn<128>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st);
}
