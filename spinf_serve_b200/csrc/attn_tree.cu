// Tree-mask attention over one packed stream (prefill), tcgen05 + TMEM + TMA, for sm_100a.
//
// Persistent CTAs, one per SM; a work item is one 128-row tile of queries against the tile list of its 128-row query block
// (built on the host from the packing metadata), walked in ascending key order, 128 keys at a time. The 128 rows of an item are
// either one head's whole query block, or - when two query heads share a key/value head - the same 64 stream rows of both
// heads, so that every K / V tile fetched serves two heads.
//   warp 0     one lane: TMA loads of Q (per item) and of K, 64 keys at a time, into a ring
//   warp 10    one lane: TMA loads of V, 64 keys at a time, into its own ring
//   warp 1     owns tensor memory; one lane issues, per 128-key tile, S = Q K^T as two 128 x 64 halves into one of two S buffers,
//              and O += P V as two K = 64 halves with P read from tensor memory; S of tile t+1 is issued before P V of tile t
//   warps 2-9  two softmax groups of four warps; thread = query row, group A takes keys [0, 64) of the tile and group B keys
//              [64, 128): S half from TMEM, the row's 64-bit visibility word of the tile (built once per stream by
//              tile_mask_bits_kernel below: the mask is the same for every layer and head), row maximum (exchanged between the two groups through shared memory so that
//              both take the same decisions), exponentials, P as packed bf16 written back over the S half in TMEM.
//              O is rescaled in TMEM only when a row's maximum grew by more than 2^24 since its reference maximum was last moved
//              (probabilities then stay below 2^24: no overflow in bf16 P, the fp32 sum or O, and rounding to bf16 is relative, so
//              nothing is lost against a maximum that moves every tile); the decision depends on the row's own scores only.
//              At the end of an item each group divides its half of the O columns by the row sum and stores bf16.
// When two (or an even number of) query heads share a key/value head the kernel runs as CTA pairs (PAIR, below): the two 64-row
// halves of a query block form a cluster of two CTAs that split every K / V tile between them, which leaves room for two whole
// tiles of each in flight per CTA instead of one.
// Numerics follow the reference's attention (bf16 Q/K/V, fp32 scores and softmax state, P rounded to bf16 before P V, fp32
// accumulation). Reduction order per row = ascending key tiles of the row's own job, independent of what else is packed in the
// stream; tiles flagged "no mask" only skip the mask evaluation, never change the arithmetic.
#include <atomic>
#include "common.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int KH = 64;                    // keys per half tile (one softmax group's share, one ring stage)
static constexpr float RESCALE_THRESHOLD = 24.f;  // log2 units
static constexpr int ATTN_THREADS = 352;

template <int D>
struct AttnSmem {
  static constexpr int SLABS = D / 64;              // 64-element (128-byte) slabs along the head dimension
  static constexpr int Q_BYTES = SLABS * 128 * 128;
  static constexpr int KV_HALF = SLABS * KH * 128;  // one ring stage: 64 keys of K (or V)
  static constexpr int NS = D == 256 ? 2 : 4;       // ring depth in stages, a multiple of 2
  static constexpr int K_OFF = Q_BYTES;
  static constexpr int V_OFF = K_OFF + NS * KV_HALF;
  static constexpr int BAR_OFF = V_OFF + NS * KV_HALF;
  static constexpr int XCHG_OFF = BAR_OFF + 512;            // 3 x 2 x 128 floats: row maxima (two buffers), row sums
  static constexpr int ORDER_OFF = XCHG_OFF + 3 * 2 * 128 * 4;  // tile counts and the cost order of the query blocks (16 bits each)
  static constexpr int MAX_SORT = 2048;                     // streams with more query blocks are walked in natural order
  static constexpr int TOTAL = ORDER_OFF + 2 * MAX_SORT * 2 + 1024;
  static constexpr int TMEM_COLS = 512;  // S: 2 buffers x 128 columns; O: D columns from column 256
  static constexpr int O_COL = 256;
};

struct AttnArgs {
  __nv_bfloat16* out;
  int64_t out_pitch;
  float* row_amax;  // optional [n]: max |out| over a token's whole output row, merged with an integer atomic max
  const int32_t* art;
  const int32_t* end;
  const int32_t* pos;
  const int32_t* tile_offsets;
  const int32_t* tile_blocks;
  const uint8_t* tile_flags;  // bit 0: every pair attends under the tree rule; bit 1: no mask evaluation needed (window included)
  const uint64_t* tile_bits;  // per list entry, key half and query row of the block: visibility of the half's 64 keys
  int nb, H, group;           // group = H / Hkv
  int hp;                     // query heads per item: 1, or 2 (64 rows of each of two heads that share a key/value head)
  int n_items;                // nb * H
  int window;
  float scale_log2;
};

// item -> (query block, first head, first row of the block it covers)
struct AttnItem {
  int qb, h0, row0;
};
__device__ __forceinline__ AttnItem attn_item(const AttnArgs& a, int it) {
  AttnItem r;
  r.qb = it / a.H;
  const int x = it - r.qb * a.H;
  if (a.hp == 2) {
    r.h0 = (x >> 1) * 2;
    r.row0 = (x & 1) * 64;
  } else {
    r.h0 = x;
    r.row0 = 0;
  }
  return r;
}


// ---------------------------------------------------------------- CTA pairs (thread-block clusters of 2, tcgen05 cta_group::2)
// PAIR = true: the two 64-row halves of a query block (same two heads, same tile list) run in the two CTAs of a cluster and share
// every K / V tile: CTA r holds keys [64 r, 64 r + 64) of the K tile and head dimensions [D/2 r, D/2 r + D/2) of the V tile, the
// leader issues the pair's MMAs (M = 256: 128 query rows per CTA) and each CTA keeps its own S / P / O in its own tensor memory.
// Half the K / V bytes per CTA leave room for two whole tiles of each in flight. No load is multicast: each CTA fetches exactly the
// bytes it alone holds; the peer's barriers are reached through shared::cluster addresses.
template <bool PAIR>
__device__ __forceinline__ void attn_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (PAIR)
    umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, accumulate);
  else
    umma_f16_ss(d_tmem, adesc, bdesc, idesc, accumulate);
}
template <bool PAIR>
__device__ __forceinline__ void attn_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (PAIR)
    umma_f16_ts_pair(d_tmem, a_tmem, bdesc, idesc, accumulate);
  else
    umma_f16_ts(d_tmem, a_tmem, bdesc, idesc, accumulate);
}
// the MMAs issued so far by this thread arrive on `bar` when they have completed: in this CTA, or in both CTAs of the pair
template <bool PAIR>
__device__ __forceinline__ void attn_commit(uint64_t* bar) {
  if (PAIR)
    umma_commit_pair(bar);
  else
    umma_commit(bar);
}

template <int D, bool PAIR>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
tree_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs a, int* __restrict__ status) {
  using L = AttnSmem<D>;
  constexpr int SLABS = L::SLABS;
  constexpr int NS = L::NS;
  // one CTA: S in two halves of 64 keys (one K stage each); a pair: the whole 128-key tile at once, 64 keys from each CTA
  constexpr uint32_t IDESC_S = PAIR ? make_idesc(FMT_BF16, FMT_BF16, 256, 128, 0, 0) : make_idesc(FMT_BF16, FMT_BF16, 128, KH, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc(FMT_BF16, FMT_BF16, PAIR ? 256 : 128, D, 0, 1);  // B = V, MN-major (head dim contiguous)
  constexpr int V_SLABS = PAIR ? SLABS / 2 : SLABS;  // 64-dimension slabs of V this CTA holds
  constexpr int V_ROWS = PAIR ? 128 : KH;            // keys per V stage
  constexpr int STAGES_PER_TILE = PAIR ? 1 : 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;                 // 1
  uint64_t* q_empty = bars + 1;            // 1
  uint64_t* k_full = bars + 2;             // NS
  uint64_t* k_empty = k_full + NS;         // NS
  uint64_t* v_full = k_empty + NS;         // NS
  uint64_t* v_empty = v_full + NS;         // NS
  uint64_t* s_full = v_empty + NS;         // 4: [buffer][half]
  uint64_t* p_ready = s_full + 4;          // 1 (one arrival per softmax warp)
  uint64_t* o_done = p_ready + 1;          // 1
  uint64_t* o_free = o_done + 1;           // 1 (one arrival per softmax warp)
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(o_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_p + 1);
  float* xchg = reinterpret_cast<float*>(smem + L::XCHG_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, status};
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  // Work units: item = (query block, head or head pair, 64-row half); a pair's unit is both halves of one (block, head pair), each
  // CTA taking half = rank. A unit costs about its query block's tile count, which varies several-fold along a packed stream
  // (trunk blocks see 1..4 tiles, branch blocks 5..6), so units are dealt out by cost: query blocks ranked by descending tile count
  // (ties by index), units in that order handed round by round to the CTAs, every other round in reverse. Against a plain stride
  // through the stream this took the slowest CTA from 21 % above the mean to under 2 % at the 27 648-token configuration. The
  // order only moves whole items between CTAs: no item's arithmetic depends on it.
  const int n_cta = PAIR ? static_cast<int>(gridDim.x) >> 1 : static_cast<int>(gridDim.x);
  const int cta = PAIR ? static_cast<int>(blockIdx.x) >> 1 : static_cast<int>(blockIdx.x);
  const int per_block = PAIR ? a.H >> 1 : a.H;  // units per query block
  const int n_units = a.nb * per_block;
  uint16_t* blk_tiles = reinterpret_cast<uint16_t*>(smem + L::ORDER_OFF);
  uint16_t* blk_order = blk_tiles + L::MAX_SORT;
  const bool sorted = a.nb <= L::MAX_SORT;
  if (sorted) {
    for (int b = threadIdx.x; b < a.nb; b += ATTN_THREADS) {
      const int c = a.tile_offsets[b + 1] - a.tile_offsets[b];
      blk_tiles[b] = static_cast<uint16_t>(c < 0 ? 0 : (c > 65535 ? 65535 : c));
    }
    __syncthreads();
    for (int b = threadIdx.x; b < a.nb; b += ATTN_THREADS) {
      const int c = blk_tiles[b];
      int rank_b = 0;
      for (int j = 0; j < a.nb; ++j) {
        const int cj = blk_tiles[j];
        rank_b += (cj > c || (cj == c && j < b)) ? 1 : 0;
      }
      blk_order[rank_b] = static_cast<uint16_t>(b);
    }
  }
  // k-th item of this CTA, or -1 when it has no more
  auto item_of = [&](int k) -> int {
    const int64_t idx = static_cast<int64_t>(k) * n_cta + ((k & 1) ? n_cta - 1 - cta : cta);
    if (idx >= n_units) return -1;
    const int sb = static_cast<int>(idx / per_block), x = static_cast<int>(idx - static_cast<int64_t>(sb) * per_block);
    const int qb = sorted ? blk_order[sb] : sb;
    return PAIR ? (qb * per_block + x) * 2 + static_cast<int>(rank) : qb * per_block + x;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&s_full[i], 1);
    mbar_init(p_ready, PAIR ? 16 : 8);  // one arrival per softmax warp; in a pair both CTAs' warps arrive on the leader's barrier
    mbar_init(o_done, 1);
    mbar_init(o_free, PAIR ? 16 : 8);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    if (PAIR) {  // the same warp in both CTAs allocates the pair's tensor memory
      tmem_alloc_pair(tmem_base_p, L::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_p, L::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival or peer-signalled copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_p;

  if (warp == 0 || warp == 10) {
    // K producer (warp 0, also loads Q) and V producer (warp 10): one lane each
    if (lane == 0) {
      const bool is_k = warp == 0;
      uint64_t* full = is_k ? k_full : v_full;
      uint64_t* empty = is_k ? k_empty : v_empty;
      const CUtensorMap* tm = is_k ? &tmK : &tmV;
      const int base = is_k ? L::K_OFF : L::V_OFF;
      uint32_t cnt = 0, item_n = 0;  // stages issued so far; items so far
      bool ok = true;
      // in a pair every copy completes on the leader's barrier, which expects both CTAs' bytes
      const uint32_t q_bar = PAIR ? map_to_cta(q_full, 0) : 0u;
      auto load = [&](void* dst, const CUtensorMap* m, int c0, int c1, uint64_t* bar) {
        if (PAIR)
          tma_load_2d_pair(dst, m, c0, c1, map_to_cta(bar, 0));
        else
          tma_load_2d(dst, m, c0, c1, bar);
      };
      for (int ki = 0, it; (it = item_of(ki)) >= 0 && ok; ++ki) {
        const AttnItem w = attn_item(a, it);
        const int e0 = a.tile_offsets[w.qb];
        const int n_tiles = a.tile_offsets[w.qb + 1] - e0;
        if (n_tiles <= 0) continue;
        const int g = w.h0 / a.group;
        if (is_k) {
          if (!mbar_wait(wc, q_empty, (item_n & 1u) ^ 1u, ST_TIMEOUT_EMPTY)) break;
          if (!PAIR || rank == 0) mbar_expect_tx(q_full, (PAIR ? 2 : 1) * L::Q_BYTES);
          const int rows = 128 / a.hp;
          for (int hh = 0; hh < a.hp; ++hh)
            for (int s = 0; s < SLABS; ++s)
              load(smem + s * 128 * 128 + hh * rows * 128, &tmQ, (w.h0 + hh) * D + s * 64, w.qb * 128 + w.row0, q_full);
        }
        for (int t = 0; t < STAGES_PER_TILE * n_tiles; ++t, ++cnt) {
          const int j = a.tile_blocks[e0 + t / STAGES_PER_TILE];
          if (j < 0 || j >= a.nb) {
            *abort_flag = 1;
            atomicCAS(status, 0, ST_BAD_INDEX);
            ok = false;
            break;
          }
          const uint32_t st = cnt % NS, ph = (cnt / NS) & 1u;
          if (!mbar_wait(wc, &empty[st], ph ^ 1u, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          if (PAIR) {
            // K: this CTA's 64 keys of the tile, all head dimensions; V: all 128 keys, this CTA's half of the head dimensions
            if (rank == 0) mbar_expect_tx(&full[st], 2 * L::KV_HALF);
            if (is_k) {
              for (int s = 0; s < SLABS; ++s)
                load(smem + base + st * L::KV_HALF + s * KH * 128, tm, g * D + s * 64, j * 128 + static_cast<int>(rank) * KH, &full[st]);
            } else {
              for (int s = 0; s < V_SLABS; ++s)
                load(smem + base + st * L::KV_HALF + s * V_ROWS * 128, tm, g * D + static_cast<int>(rank) * (D / 2) + s * 64, j * 128, &full[st]);
            }
          } else {
            const int kv0 = j * 128 + (t & 1) * KH;
            mbar_expect_tx(&full[st], L::KV_HALF);
            for (int s = 0; s < SLABS; ++s) load(smem + base + st * L::KV_HALF + s * KH * 128, tm, g * D + s * 64, kv0, &full[st]);
          }
        }
        ++item_n;
      }
      (void)q_bar;
      if (*abort_flag && !PAIR) {
        // bounded wait for copies of this CTA that may still be in flight (in a pair they complete on the leader's barriers; the
        // cluster barrier at the end keeps both CTAs resident meanwhile)
        if (is_k)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(q_full, (item_n & 1u) ^ 1u); ++spin) {}
        for (uint32_t c = cnt > static_cast<uint32_t>(NS) ? cnt - NS : 0; c < cnt; ++c)
          for (int spin = 0; spin < 4096 && !mbar_try_wait(&full[c % NS], (c / NS) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // in a pair the leader issues for both CTAs
      const uint32_t q_addr = smem_u32(smem);
      uint32_t kc = 0, vc = 0, gt = 0, item_n = 0;  // K / V stages consumed, tiles issued, items so far
      bool ok = true;
      auto issue_s = [&](uint32_t g) -> bool {  // S for tile g into S buffer g & 1: two halves of 64 keys, or (pair) the tile at once
        for (int hf = 0; hf < STAGES_PER_TILE; ++hf, ++kc) {
          const uint32_t st = kc % NS;
          if (!mbar_wait(wc, &k_full[st], (kc / NS) & 1u, ST_TIMEOUT_FULL)) return false;
          tc_fence_after();
          const uint32_t k_addr = smem_u32(smem + L::K_OFF + st * L::KV_HALF);
          const uint32_t d_tmem = tmem_base + (g & 1u) * 128 + hf * KH;
#pragma unroll
          for (int s = 0; s < SLABS; ++s) {
            const uint64_t ad = make_smem_desc_sw128(q_addr + s * 128 * 128, 16, 1024);
            const uint64_t bd = make_smem_desc_sw128(k_addr + s * KH * 128, 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) attn_mma_ss<PAIR>(d_tmem, ad + 2 * k, bd + 2 * k, IDESC_S, (s | k) != 0);
          }
          attn_commit<PAIR>(&k_empty[st]);  // the K stage may be refilled as soon as these MMAs have read it
          attn_commit<PAIR>(&s_full[(g & 1u) * 2 + hf]);
          if (PAIR) attn_commit<PAIR>(&s_full[(g & 1u) * 2 + 1]);  // both softmax groups' halves come out of the one product
        }
        return true;
      };
      for (int ki = 0, it; (it = item_of(ki)) >= 0 && ok; ++ki) {
        const AttnItem w = attn_item(a, it);
        const int n_tiles = a.tile_offsets[w.qb + 1] - a.tile_offsets[w.qb];
        if (n_tiles <= 0) continue;
        if (!mbar_wait(wc, q_full, item_n & 1u, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        if (!issue_s(gt)) break;
        for (int i = 0; i < n_tiles && ok; ++i) {
          const uint32_t g = gt + i;
          if (i + 1 < n_tiles) {
            // S buffer (g+1)&1 last held P of tile g-1, whose P V MMAs were issued before these
            if (!issue_s(g + 1)) { ok = false; break; }
          } else {
            attn_commit<PAIR>(q_empty);  // Q may be replaced once the last S MMAs of the item have read it
          }
          if (!mbar_wait(wc, p_ready, g & 1u, ST_TIMEOUT_OTHER)) { ok = false; break; }
          if (i == 0 && item_n > 0 && !mbar_wait(wc, o_free, (item_n - 1) & 1u, ST_TIMEOUT_OTHER)) { ok = false; break; }
          for (int part = 0; part < STAGES_PER_TILE && ok; ++part, ++vc) {
            const uint32_t st = vc % NS;
            if (!mbar_wait(wc, &v_full[st], (vc / NS) & 1u, ST_TIMEOUT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t v_addr = smem_u32(smem + L::V_OFF + st * L::KV_HALF);
            // V stage: slab s holds 64 head-dim columns of the stage's keys, one key per 128-byte row: MN-major B operand,
            // 64-column groups V_ROWS*128 bytes apart (LBO), 8-key groups 1024 bytes apart (SBO)
            const uint64_t vd = make_smem_desc_sw128(v_addr, V_ROWS * 128, 1024);
#pragma unroll
            for (int hh = 0; hh < (PAIR ? 2 : 1); ++hh) {  // a pair's V stage covers both softmax groups' keys
              const int hf = PAIR ? hh : part;
              const uint32_t p_tmem = tmem_base + (g & 1u) * 128 + hf * KH;  // packed bf16 P: 16 keys per 8 columns
#pragma unroll
              for (int k = 0; k < 4; ++k)  // 16 keys per step: 8 columns along P, 16 rows (2048 bytes) down V
                attn_mma_ts<PAIR>(tmem_base + L::O_COL, p_tmem + 8 * k, vd + 128 * ((PAIR ? 4 * hh : 0) + k), IDESC_O, (i | hf | k) != 0);
            }
            attn_commit<PAIR>(&v_empty[st]);
          }
          if (ok) attn_commit<PAIR>(o_done);
        }
        gt += n_tiles;
        ++item_n;
      }
    }
  } else {
    // softmax warps 2..9
    const int wg = (warp - 2) >> 2;  // 0: keys [0, 64) of a tile, 1: keys [64, 128)
    const int qd = warp & 3;         // TMEM lane quarter this warp may access
    const int row = qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    uint32_t gt = 0, item_n = 0;
    bool alive = true;
    // the list bounds, first entry and first visibility word of an item are fetched while the item before it is processed
    const int rows_per_head = 128 / a.hp;
    int pe0 = 0, pe1 = 0, pj = 0, pf = 0;
    uint64_t pbits = 0;
    auto first_entry = [&](const AttnItem& w, int e0, int e1) {
      if (e1 > e0) {
        pj = a.tile_blocks[e0];
        pf = a.tile_flags[e0];
        pbits = a.tile_bits[(static_cast<int64_t>(e0) * 2 + wg) * 128 + w.row0 + (row % rows_per_head)];
      }
    };
    if (item_of(0) >= 0) {
      const AttnItem w = attn_item(a, item_of(0));
      pe0 = a.tile_offsets[w.qb], pe1 = a.tile_offsets[w.qb + 1];
      first_entry(w, pe0, pe1);
    }
    for (int ki = 0, it; (it = item_of(ki)) >= 0 && alive; ++ki) {
      const AttnItem w = attn_item(a, it);
      const int e0 = pe0;
      const int n_tiles = pe1 - pe0;
      int j_next = pj, f_next = pf;
      uint64_t bits_next = (pf & 2) ? ~0ull : pbits;
      const int it_n = item_of(ki + 1);
      const bool have_n = it_n >= 0;
      const AttnItem w_n = attn_item(a, have_n ? it_n : it);
      if (have_n) pe0 = a.tile_offsets[w_n.qb], pe1 = a.tile_offsets[w_n.qb + 1];  // consumed at the end of this item
      if (n_tiles <= 0) {
        if (have_n) first_entry(w_n, pe0, pe1);
        continue;
      }
      const int head = w.h0 + row / rows_per_head;
      const int tq = w.qb * 128 + w.row0 + (row % rows_per_head);  // stream position of this thread's query row
      const int rowb = w.row0 + (row % rows_per_head);            // row within the query block
      float m_ref = -INFINITY, l_run = 0.f;

      for (int i = 0; i < n_tiles; ++i) {
        const uint32_t g = gt + i;
        const int j = j_next;
        const bool no_mask = (f_next & 2) != 0;
        const uint64_t bits = bits_next;
        if (i + 1 < n_tiles) {  // in flight while this tile is processed
          j_next = a.tile_blocks[e0 + i + 1];
          f_next = a.tile_flags[e0 + i + 1];
          bits_next = (f_next & 2) ? ~0ull : a.tile_bits[(static_cast<int64_t>(e0 + i + 1) * 2 + wg) * 128 + rowb];
        }
        bool got = j >= 0 && j < a.nb && mbar_wait(wc, &s_full[(g & 1u) * 2 + wg], (g >> 1) & 1u, ST_TIMEOUT_TMEM);
        float s[KH];
        float mx = -INFINITY;
        const uint32_t s_tmem = tmem_base + lane_off + (g & 1u) * 128 + wg * KH;
        if (__all_sync(0xffffffffu, got)) {
          tc_fence_after();
          uint32_t v0[32], v1[32];
          tmem_ld_x32(s_tmem, v0);
          tmem_ld_x32(s_tmem + 32, v1);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(v0[c]), s[32 + c] = __uint_as_float(v1[c]);
          if (!no_mask) {
            const uint32_t b_lo = static_cast<uint32_t>(bits), b_hi = static_cast<uint32_t>(bits >> 32);
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              s[c] = (b_lo & (1u << c)) ? s[c] : -INFINITY;
              s[32 + c] = (b_hi & (1u << c)) ? s[32 + c] : -INFINITY;
            }
          }
#pragma unroll
          for (int c = 0; c < KH; ++c) mx = fmaxf(mx, s[c]);
        } else {
          got = false;
        }
        // the two groups exchange their halves' row maxima: every decision below is taken on the maximum over the whole tile
        float* xq = xchg + (g & 1u) * 256;
        xq[wg * 128 + row] = mx;
        if (!bar_red_and(1 + qd, 64, got)) { alive = false; break; }  // the two warps that share these rows leave together
        mx = fmaxf(mx, xq[(wg ^ 1) * 128 + row]) * a.scale_log2;
        // move the reference maximum only when the row's maximum has grown by more than the threshold
        float alpha = 1.f;
        if (mx - m_ref > RESCALE_THRESHOLD) {  // false for NaN (-inf minus -inf): a row that has seen nothing yet
          alpha = fast_exp2(m_ref - mx);
          m_ref = mx;
        }
        const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pk[KH / 2];
#pragma unroll
        for (int c = 0; c < KH / 2; ++c) {
          const float p0 = fast_exp2(fmaf(s[2 * c], a.scale_log2, neg_m)), p1 = fast_exp2(fmaf(s[2 * c + 1], a.scale_log2, neg_m));
          sum0 += p0;
          sum1 += p1;
          pk[c] = pack_bf16x2(p0, p1);
        }
        l_run = l_run * alpha + (sum0 + sum1);
        if (i > 0) {
          // P V of the previous tile is waited for at every tile, not only before a rescale: a parity wait is only unambiguous
          // while the waiter is at most one phase ahead of the barrier
          const bool done = mbar_wait(wc, o_done, (g - 1) & 1u, ST_TIMEOUT_TMEM);
          if (__any_sync(0xffffffffu, alpha != 1.f) && __all_sync(0xffffffffu, done)) {
            // every P V issued so far has completed and none is in flight until all 256 threads have arrived on p_ready:
            // this group rescales its half of the O columns
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < D / 64; ++c) {
              uint32_t o[32];
              const uint32_t o_tmem = tmem_base + lane_off + L::O_COL + wg * (D / 2) + c * 32;
              tmem_ld_x32(o_tmem, o);
              tmem_wait_ld();
#pragma unroll
              for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
              tmem_st_x32(o_tmem, o);
            }
          }
        }
        __syncwarp();
        tmem_st_x32(s_tmem, pk);  // P over the first 32 columns of the S half this thread has already read
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();  // every lane's P is in tensor memory: one arrival per warp (a remote arrival per thread costs 1 200 cycles a tile)
        if (lane == 0) {
          if (PAIR)
            mbar_arrive_cluster(map_to_cta(p_ready, 0));
          else
            mbar_arrive(p_ready);
        }
      }
      if (!alive) break;
      gt += n_tiles;

      // end of the item: O / l for this group's half of the columns
      const uint32_t g_last = gt - 1;
      float* xq = xchg + 2 * 256;  // its own buffer: the next item's first tile may already be writing maxima
      xq[wg * 128 + row] = l_run;
      if (have_n) first_entry(w_n, pe0, pe1);  // lands while O is read out
      const bool got = mbar_wait(wc, o_done, g_last & 1u, ST_TIMEOUT_TMEM);
      if (!bar_red_and(1 + qd, 64, got)) { alive = false; break; }
      tc_fence_after();
      const float inv = 1.f / (l_run + xq[(wg ^ 1) * 128 + row]);  // every row sees at least itself, so the sum is positive
      __nv_bfloat16* dst = a.out + static_cast<int64_t>(tq) * a.out_pitch + head * D + wg * (D / 2);
      uint32_t amax2 = 0u;  // running max of |out| over this thread's columns, as a packed bf16 pair
#pragma unroll 1
      for (int c = 0; c < D / 64; c += 2) {  // 64 columns at a time: both TMEM loads in flight together
        uint32_t o0[32], o1[32];
        __syncwarp();
        tmem_ld_x32(tmem_base + lane_off + L::O_COL + wg * (D / 2) + c * 32, o0);
        tmem_ld_x32(tmem_base + lane_off + L::O_COL + wg * (D / 2) + c * 32 + 32, o1);
        tmem_wait_ld();
        if (c + 2 >= D / 64) {  // O is in registers: the next item's first P V may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (PAIR)
              mbar_arrive_cluster(map_to_cta(o_free, 0));
            else
              mbar_arrive(o_free);
          }
        }
#pragma unroll
        for (int hfc = 0; hfc < 2; ++hfc) {
          const uint32_t (&o)[32] = hfc ? o1 : o0;
          uint32_t wv[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            wv[x] = pack_bf16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
            amax2 = bf2_max(amax2, wv[x] & 0x7fff7fffu);
          }
          const uint32_t lo[8] = {wv[0], wv[1], wv[2], wv[3], wv[4], wv[5], wv[6], wv[7]};
          const uint32_t hi[8] = {wv[8], wv[9], wv[10], wv[11], wv[12], wv[13], wv[14], wv[15]};
          stg_v8(dst + (c + hfc) * 32, lo);
          stg_v8(dst + (c + hfc) * 32 + 16, hi);
        }
      }
      // non-negative floats order like their bit patterns, so the merged maximum does not depend on the order of arrival
      if (a.row_amax) atomicMax(reinterpret_cast<unsigned int*>(a.row_amax + tq), __float_as_uint(fmaxf(bf2_lo(amax2), bf2_hi(amax2))));
      ++item_n;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA leaves while its peer may still signal its barriers or read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (PAIR)
      tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
    else
      tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// Visibility words of a packed stream: for list entry e (query block qb against key block j), key half hf and row r of the query
// block, bit c of bits[(e * 2 + hf) * 128 + r] says whether query t = 128 qb + r sees key k = 128 j + 64 hf + c:
//   (k <= t && art[t] >= 0 && art[k] == art[t] && t < end[k] && (window <= 0 || pos[t] - pos[k] < window)) || t == k
//   || (grp && grp[t] >= 0 && grp[k] == grp[t] && (!grp_in_window || window <= 0 || pos[t] - pos[k] < window))
// (the last line: an image's placeholder tokens see each other both ways, spinf_serve/scorer.py:178-198).
// One CTA per query block, thread = (row, half). Runs once per stream and mask type; every layer and head reads the result.
__global__ void __launch_bounds__(256) tile_mask_bits_kernel(const int32_t* __restrict__ art, const int32_t* __restrict__ end,
                                                             const int32_t* __restrict__ pos, const int32_t* __restrict__ grp, int nb,
                                                             int window, int grp_in_window, const int32_t* __restrict__ tile_offsets,
                                                             const int32_t* __restrict__ tile_blocks, uint64_t* __restrict__ bits) {
  __shared__ int k_art[128], k_end[128], k_pos[128], k_grp[128];
  const int qb = blockIdx.x;
  const int r = threadIdx.x & 127, hf = threadIdx.x >> 7;
  const int t = qb * 128 + r;
  const int art_q = art[t], pos_q = pos[t];
  const int grp_q = grp ? grp[t] : -1;
  const int e0 = tile_offsets[qb], e1 = tile_offsets[qb + 1];
  for (int e = e0; e < e1; ++e) {
    const int j = tile_blocks[e];
    const bool valid = j >= 0 && j < nb;
    __syncthreads();
    if (threadIdx.x < 128 && valid) {
      k_art[threadIdx.x] = art[j * 128 + threadIdx.x];
      k_end[threadIdx.x] = end[j * 128 + threadIdx.x];
      k_pos[threadIdx.x] = pos[j * 128 + threadIdx.x];
      k_grp[threadIdx.x] = grp ? grp[j * 128 + threadIdx.x] : -1;
    }
    __syncthreads();
    uint64_t word = 0;
    if (valid) {
      for (int c = 0; c < 64; ++c) {
        const int kk = hf * 64 + c;
        const int k = j * 128 + kk;
        const bool tree = k <= t && art_q >= 0 && k_art[kk] == art_q && t < k_end[kk];
        const bool win = window <= 0 || pos_q - k_pos[kk] < window;
        const bool img = grp_q >= 0 && k_grp[kk] == grp_q && (!grp_in_window || win);
        if ((tree && win) || k == t || img) word |= 1ull << c;
      }
    }
    bits[(static_cast<int64_t>(e) * 2 + hf) * 128 + r] = word;
  }
}

template <int D, bool PAIR>
static int launch_attn(const void* q, const void* k, const void* v, int64_t n, int H, int Hkv, int64_t q_pitch, int64_t kv_pitch,
                       const AttnArgs& args, cudaStream_t stream) {
  using L = AttnSmem<D>;
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  CUtensorMap tmQ, tmK, tmV;
  int r;
  if ((r = make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, n, static_cast<uint64_t>(H) * D, q_pitch * 2, 64, 128 / args.hp)))
    return r;
  if ((r = make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, n, static_cast<uint64_t>(Hkv) * D, kv_pitch * 2, 64, KH))) return r;
  // V boxes: 64 keys of all head dimensions for one CTA; all 128 keys of the CTA's half of the head dimensions in a pair
  if ((r = make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v, n, static_cast<uint64_t>(Hkv) * D, kv_pitch * 2, 64, PAIR ? 128 : KH)))
    return r;
  auto kern = tree_attn_kernel<D, PAIR>;
  static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice from two threads is harmless
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(ATTN_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (PAIR) {
    const int pairs = args.n_items / 2 < sm_count() / 2 ? args.n_items / 2 : sm_count() / 2;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else {
    cfg.gridDim = dim3(static_cast<unsigned>(args.n_items < sm_count() ? args.n_items : sm_count()));
  }
  SPINF_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmQ, tmK, tmV, args, status));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_tile_mask_bits_img(const int32_t* art, const int32_t* end, const int32_t* pos, const int32_t* grp, int64_t n,
                                        int32_t window, int32_t grp_in_window, const int32_t* tile_offsets, const int32_t* tile_blocks,
                                        uint64_t* bits, void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(art && end && pos && tile_offsets && tile_blocks && bits && n >= 0 && n % SPINF_BLOCK == 0 && n < (1ll << 30));
  const int nb = static_cast<int>(n / SPINF_BLOCK);
  tile_mask_bits_kernel<<<nb, 256, 0, static_cast<cudaStream_t>(stream)>>>(art, end, pos, grp, nb, window, grp_in_window, tile_offsets,
                                                                           tile_blocks, bits);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_tile_mask_bits(const int32_t* art, const int32_t* end, const int32_t* pos, int64_t n, int32_t window,
                                    const int32_t* tile_offsets, const int32_t* tile_blocks, uint64_t* bits, void* stream) {
  return spinf_tile_mask_bits_img(art, end, pos, nullptr, n, window, 0, tile_offsets, tile_blocks, bits, stream);
}

extern "C" int spinf_tree_attn_fwd(const void* q, const void* k, const void* v, void* out, int64_t n, int32_t H, int32_t Hkv,
                                   int32_t D, int64_t q_pitch, int64_t kv_pitch, int64_t out_pitch, const int32_t* art,
                                   const int32_t* end, const int32_t* pos, int32_t window, float scale, const int32_t* tile_offsets,
                                   const int32_t* tile_blocks, const uint8_t* tile_flags, const uint64_t* tile_bits, float* row_amax,
                                   void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(q && k && v && out && art && end && pos && tile_offsets && tile_blocks && tile_flags && tile_bits);
  SPINF_CHECK_ARG(n >= 0 && n % SPINF_BLOCK == 0 && n < (1ll << 30) && H > 0 && Hkv > 0 && H % Hkv == 0 && H <= 65535);
  SPINF_CHECK_ARG(D == 128 || D == 256);
  SPINF_CHECK_ARG(q_pitch >= static_cast<int64_t>(H) * D && kv_pitch >= static_cast<int64_t>(Hkv) * D && out_pitch >= static_cast<int64_t>(H) * D);
  // rows of the output are written as 32-byte pieces
  SPINF_CHECK_ARG(q_pitch % 8 == 0 && kv_pitch % 8 == 0 && out_pitch % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 31) == 0);
  SPINF_CHECK_ARG(scale > 0.f && n / SPINF_BLOCK * static_cast<int64_t>(H) < (1ll << 31));
  AttnArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.out_pitch = out_pitch;
  a.row_amax = row_amax;
  a.art = art;
  a.end = end;
  a.pos = pos;
  a.tile_offsets = tile_offsets;
  a.tile_blocks = tile_blocks;
  a.tile_flags = tile_flags;
  a.tile_bits = tile_bits;
  a.nb = static_cast<int>(n / SPINF_BLOCK);
  a.H = H;
  a.group = H / Hkv;
  a.hp = a.group % 2 == 0 ? 2 : 1;
  a.n_items = a.nb * H;
  a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // two query heads per key/value head (or a multiple): the two 64-row halves of a query block run as a CTA pair sharing K / V
  const bool pair = a.hp == 2 && a.n_items % 2 == 0 && a.n_items >= 2;
  if (D == 256)
    return pair ? launch_attn<256, true>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st)
                : launch_attn<256, false>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st);
  return pair ? launch_attn<128, true>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st)
              : launch_attn<128, false>(q, k, v, n, H, Hkv, q_pitch, kv_pitch, a, st);
}

