// Gated DeltaNet, scan of one level of a trie plan on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the operands in
// shared memory (128-byte-swizzled tiles) and the accumulators, the recurrent state among them, in tensor memory.
//
// Same arithmetic and rounding points as gdn_tree_scan_kernel in gdn_tree.cu (which runs the same units on warp-level MMAs): per
// unit of at most 64 rows, with S the state at the unit's start,
//     v' = U - W S        o = scale [(Q S) 2^G + P v']        S <- S 2^(G_last) + K^T (v' 2^(G_last - G))
// One CTA per (group of siblings, value head), the whole 128 x 128 state: it lives in tensor memory as fp32, lane = key dimension,
// column = value dimension, for the CTA's lifetime. Three products per unit, all M = 128, N = 128:
//     D1 = [W; Q] S      A = rows 0..63 W, rows 64..127 Q (K-major, 128 x 128); B = S as bf16, row = key dim (MN-major): one product
//                        gives W S in lanes 0..63 and Q S in lanes 64..127
//     D2 = [ . ; P] v'   A = rows 64..127 P (64 x 64; rows 0..63 hold finite leftovers, their lanes are never read); B = v' rows
//     S += K^T v'd       A = the K tile as it lies in memory, row = token (MN-major A); B = v' 2^(G_last - G) rows; the state was
//                        multiplied by 2^(G_last) when it was copied out for D1 (a tensor-memory round trip that the bf16 copy
//                        needs anyway)
// Roles: warps 0..3 own tensor-memory lanes 32 w .. 32 w + 31: they queue the next unit's operand tiles (cp.async into the other
// stage, writing the swizzle themselves), copy the state out, turn D1 into v' (threads 0..63, one token row each) and D1, D2 into
// output rows (threads 64..127); warp 4 issues the MMAs. Everything between the roles goes through mbarriers with bounded waits.
#include <atomic>
#include "common.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int TK = 128;   // head dimension
static constexpr int TC = 64;    // rows per unit
static constexpr int TC_THREADS = 160;
static constexpr int UNIT_WORDS_TC = 12;
static constexpr int UF_UPDATE_TC = 1, UF_PARENT_TC = 2;

struct GdnTcArgs {
  const __nv_bfloat16 *q, *k;
  __nv_bfloat16* o;
  int64_t q_pitch;
  int Hk, Hv;
  float scale;
  const __nv_bfloat16 *w_ws, *u_ws, *p_ws;
  const float* g_ws;
  const int32_t *grp_parent, *grp_ubeg, *units, *unit_rows;
  const float* h_in;
  float* h_out;
};

struct TcStage {
  uint8_t a1[2 * 128 * 128];  // [W; Q]: 128 rows x 128 key dims, K-major, two 64-column slabs
  uint8_t kt[2 * TC * 128];   // K rows [token][key dim]: the MN-major A operand of the update, two 64-dim slabs
  uint8_t a2[128 * 128];      // rows 64..127 = P (64 x 64, K-major); rows 0..63 are never written after the start
};
struct TcSmem {
  TcStage st[2];
  uint8_t b1[2 * 128 * 128];  // the state as bf16, row = key dim, two 64-value-dim slabs (MN-major B)
  uint8_t vn[2 * TC * 128];   // v' rows, two 64-value-dim slabs (MN-major B)
  uint8_t vd[2 * TC * 128];   // v' 2^(G_last - G) rows
  uint64_t ld_full[2], s_ready, d1_done, v_ready, d2_done, upd_done, d_free;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

__global__ void __launch_bounds__(TC_THREADS, 1) gdn_tree_scan_tc_kernel(const GdnTcArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t tc_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int grp = blockIdx.x, hv = blockIdx.y;
  const int hk = hv / (a.Hv / a.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u_beg = a.grp_ubeg[grp], u_end = a.grp_ubeg[grp + 1];
  const int parent = a.grp_parent[grp];
  const WaitCtx wc{&sm.abort_flag, status};

  // finite leftovers everywhere an MMA may read without a writer (rows 0..63 of a2; rows of partial units)
  for (int j = tid; j < static_cast<int>((sizeof(TcStage) * 2 + sizeof(sm.b1) + sizeof(sm.vn) + sizeof(sm.vd)) / 16); j += TC_THREADS)
    reinterpret_cast<uint4*>(&sm)[j] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    mbar_init(&sm.ld_full[0], 128);
    mbar_init(&sm.ld_full[1], 128);
    mbar_init(&sm.s_ready, 128);
    mbar_init(&sm.d1_done, 1);
    mbar_init(&sm.v_ready, 64);
    mbar_init(&sm.d2_done, 1);
    mbar_init(&sm.upd_done, 1);
    mbar_init(&sm.d_free, 128);
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  fence_proxy_async_smem();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  constexpr uint32_t COL_S = 0, COL_D1 = 128, COL_D2 = 256;
  constexpr uint32_t IDESC_NB = make_idesc(FMT_BF16, FMT_BF16, 128, 128, 0, 1);  // A K-major, B MN-major
  constexpr uint32_t IDESC_UP = make_idesc(FMT_BF16, FMT_BF16, 128, 128, 1, 1);  // A and B MN-major

  // which units copy the state out / decay it is a function of the flags alone: every role follows the same bookkeeping
  if (warp == 4) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      bool dirty = false, s_valid = false;
      uint32_t n_sready = 0, n_vready = 0, n_dfree = 0;
      int flags_n = 0, len_n = 0;
      if (u_beg < u_end) flags_n = a.units[static_cast<int64_t>(u_beg) * UNIT_WORDS_TC + 1], len_n = a.units[static_cast<int64_t>(u_beg) * UNIT_WORDS_TC + 5];
      for (int u = u_beg, i = 0; u < u_end; ++u, ++i) {
        const int flags = flags_n, len = len_n;
        if (u + 1 < u_end) flags_n = a.units[static_cast<int64_t>(u + 1) * UNIT_WORDS_TC + 1], len_n = a.units[static_cast<int64_t>(u + 1) * UNIT_WORDS_TC + 5];
        TcStage& st = sm.st[i & 1];
        if ((flags & UF_PARENT_TC) && dirty) dirty = false, s_valid = false;
        const bool touch = !s_valid || (flags & UF_UPDATE_TC);
        s_valid = true;
        if (!mbar_wait(wc, &sm.ld_full[i & 1], (i >> 1) & 1u, ST_TIMEOUT_FULL)) break;
        if (touch && !mbar_wait(wc, &sm.s_ready, (n_sready++) & 1u, ST_TIMEOUT_OTHER)) break;
        if (i > 0 && !mbar_wait(wc, &sm.d_free, (n_dfree++) & 1u, ST_TIMEOUT_OTHER)) break;
        tc_fence_after();
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          const uint64_t ad = make_smem_desc_sw128(smem_u32(st.a1) + sl * 16384, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(smem_u32(sm.b1) + sl * 8192, 16384, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16_ss(tmem + COL_D1, ad + 2 * kk, bd + 128 * kk, IDESC_NB, (sl | kk) != 0);
        }
        umma_commit(&sm.d1_done);
        if (!mbar_wait(wc, &sm.v_ready, (n_vready++) & 1u, ST_TIMEOUT_OTHER)) break;
        tc_fence_after();
        {
          const uint64_t ad = make_smem_desc_sw128(smem_u32(st.a2), 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(smem_u32(sm.vn), 8192, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16_ss(tmem + COL_D2, ad + 2 * kk, bd + 128 * kk, IDESC_NB, kk != 0);
        }
        umma_commit(&sm.d2_done);
        if (flags & UF_UPDATE_TC) {
          const uint64_t ad = make_smem_desc_sw128(smem_u32(st.kt), 8192, 1024);
          const uint64_t bd = make_smem_desc_sw128(smem_u32(sm.vd), 8192, 1024);
          for (int kk = 0; kk * 16 < len; ++kk) umma_f16_ss(tmem + COL_S, ad + 128 * kk, bd + 128 * kk, IDESC_UP, 1u);
          umma_commit(&sm.upd_done);
          dirty = true, s_valid = false;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- row threads: thread t <-> tensor-memory lane t
    const int t = tid;            // 0..127
    const int tr = t & 63;        // the token row this thread serves (W side for t < 64, Q side for t >= 64)
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const __nv_bfloat16* const any = a.w_ws;

    // A unit's row entries of the host-built table and its control words, read in two dependent steps that are issued a unit
    // apart, so that no step waits for the one before it: step 1 (the table) two units ahead, step 2 (the running log-decays,
    // addressed by step 1's tokens) one unit ahead.
    struct Meta {
      int tok, row, c0, last, ulast, flags, slot;
      float g, gl, glu;
    };
    auto step1 = [&](int u, Meta& m) {
      const int32_t* ur = a.unit_rows + static_cast<int64_t>(u) * 4 * TC;
      const int32_t* ud = a.units + static_cast<int64_t>(u) * UNIT_WORDS_TC;
      m.tok = ur[tr], m.row = ur[TC + tr], m.last = ur[2 * TC + tr], m.c0 = ur[3 * TC + tr];
      m.flags = ud[1], m.slot = ud[2], m.ulast = ud[4] + ud[5] - 1;  // the first piece's last token: the unit's, when it updates
    };
    auto step2 = [&](Meta& m) {
      m.g = m.tok >= 0 ? a.g_ws[static_cast<int64_t>(m.tok) * a.Hv + hv] : 0.f;
      m.gl = m.tok >= 0 ? a.g_ws[static_cast<int64_t>(m.last) * a.Hv + hv] : 0.f;
      m.glu = a.g_ws[static_cast<int64_t>(m.ulast) * a.Hv + hv];
    };
    // copies of one unit's tiles from this warp's rows: lanes cover consecutive 16-byte chunks, the row's table entries come
    // from the lane that holds them
    auto queue_copies = [&](TcStage& st, int tok, int row, int c0) {
      // a1: warp w writes rows 32 w .. 32 w + 31 (warps 0, 1: W rows of tokens 0..63; warps 2, 3: Q rows), two rows per instruction
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int src = 2 * j + (lane >> 4), c = lane & 15;
        const int tk = __shfl_sync(0xffffffffu, tok, src), rw = __shfl_sync(0xffffffffu, row, src);
        const uint32_t r = static_cast<uint32_t>(warp * 32 + src);
        const __nv_bfloat16* g = warp < 2 ? a.w_ws + (static_cast<int64_t>(tk) * a.Hv + hv) * TK + c * 8
                                          : a.q + static_cast<int64_t>(rw) * a.q_pitch + hk * TK + c * 8;
        cp_async16(st.a1 + (c >> 3) * 16384 + sw128(r, c & 7), tk >= 0 ? g : any, tk >= 0 ? 16 : 0);
      }
      // kt: warp w writes token rows 32 (w & 1) .. +31, key dims 64 (w >> 1) .. +63: four rows of 128 bytes per instruction
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int src = 4 * j + (lane >> 3), c = lane & 7;
        const int tk = __shfl_sync(0xffffffffu, tok, src), rw = __shfl_sync(0xffffffffu, row, src);
        const uint32_t r = static_cast<uint32_t>((warp & 1) * 32 + src);
        cp_async16(st.kt + (warp >> 1) * 8192 + sw128(r, c),
                   tk >= 0 ? a.k + static_cast<int64_t>(rw) * a.q_pitch + hk * TK + (warp >> 1) * 64 + c * 8 : any, tk >= 0 ? 16 : 0);
      }
      // a2 rows 64 + token: warp w writes token rows 32 (w & 1) .. +31, P chunks 4 (w >> 1) .. +3: eight rows per instruction
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int src = 8 * j + (lane >> 2), c = (warp >> 1) * 4 + (lane & 3);
        const int tk = __shfl_sync(0xffffffffu, tok, src), cc = __shfl_sync(0xffffffffu, c0, src);
        const uint32_t r = static_cast<uint32_t>(64 + (warp & 1) * 32 + src);
        const int cs = c - (cc >> 3);  // P's columns are relative to the piece's first row
        const bool pv = tk >= 0 && cs >= 0;
        cp_async16(st.a2 + sw128(r, c), pv ? a.p_ws + (static_cast<int64_t>(tk) * a.Hv + hv) * TC + cs * 8 : any, pv ? 16 : 0);
      }
      cp_async_commit();
    };
    auto load_parent = [&]() {  // h_in row (key dim t) -> tensor memory
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) r[e] = 0u;
        if (parent >= 0) {
          const float4* src = reinterpret_cast<const float4*>(a.h_in + ((static_cast<int64_t>(parent) * a.Hv + hv) * TK + t) * TK + 32 * c);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float4 f = src[e];
            r[4 * e] = __float_as_uint(f.x), r[4 * e + 1] = __float_as_uint(f.y), r[4 * e + 2] = __float_as_uint(f.z), r[4 * e + 3] = __float_as_uint(f.w);
          }
        }
        tmem_st_x32(lane_addr + COL_S + 32 * c, r);
      }
      tmem_wait_st();
    };

    Meta mc{-1, 0, 0, 0, 0, 0, -1, 0.f, 0.f, 0.f}, mn = mc, mp = mc;  // this unit, the next, the one after
    if (u_beg < u_end) {
      step1(u_beg, mc);
      if (u_beg + 1 < u_end) step1(u_beg + 1, mn);
      step2(mc);
      queue_copies(sm.st[0], mc.tok, mc.row, mc.c0);
    }
    load_parent();
    bool dirty = false, s_valid = false, alive = true;
    uint32_t n_d1 = 0, n_d2 = 0, n_upd = 0;
    bool upd_pending = false;
    int prev_slot = -1;

    for (int u = u_beg, i = 0; u < u_end && alive; ++u, ++i) {
      const int flags = mc.flags;
      const int m_tok = mc.tok, m_row = mc.row;
      const float m_g = mc.g, m_gl = mc.gl, m_glu = mc.glu;
      if (u + 1 < u_end) step2(mn);          // next unit's log-decays: its table entries arrived a unit ago
      if (u + 2 < u_end) step1(u + 2, mp);   // the table entries of the unit after
      // the previous unit's products are complete (its D2 was waited for below; its update here): the other stage, v' and the
      // state may be touched again
      if (upd_pending) {
        if (!mbar_wait(wc, &sm.upd_done, (n_upd++) & 1u, ST_TIMEOUT_OTHER)) break;
        tc_fence_after();
        upd_pending = false;
        if (prev_slot >= 0) {  // the state a deeper level reads
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_x32(lane_addr + COL_S + 32 * c, r);
            tmem_wait_ld();
            float4* dst = reinterpret_cast<float4*>(a.h_out + ((static_cast<int64_t>(prev_slot) * a.Hv + hv) * TK + t) * TK + 32 * c);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              dst[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]), __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
          }
        }
      }
      // this unit's U row straight from the workspace (threads 0..63), ahead of the waits
      uint4 urow[16];
      if (t < 64 && m_tok >= 0) {
        const uint4* src = reinterpret_cast<const uint4*>(a.u_ws + (static_cast<int64_t>(m_tok) * a.Hv + hv) * TK);
#pragma unroll
        for (int e = 0; e < 16; ++e) urow[e] = src[e];
      }
      if ((flags & UF_PARENT_TC) && dirty) {
        load_parent();
        dirty = false, s_valid = false;
      }
      const bool need_copy = !s_valid, need_decay = (flags & UF_UPDATE_TC) != 0;
      if (need_copy || need_decay) {
        const float eg = fast_exp2(m_glu);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_x32(lane_addr + COL_S + 32 * c, r);
          tmem_wait_ld();
          if (need_copy) {  // row t (a key dim) of the bf16 state: value dims 32 c .. 32 c + 31 = four 16-byte chunks
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint4 v = make_uint4(pack_bf16x2(__uint_as_float(r[8 * e]), __uint_as_float(r[8 * e + 1])),
                                         pack_bf16x2(__uint_as_float(r[8 * e + 2]), __uint_as_float(r[8 * e + 3])),
                                         pack_bf16x2(__uint_as_float(r[8 * e + 4]), __uint_as_float(r[8 * e + 5])),
                                         pack_bf16x2(__uint_as_float(r[8 * e + 6]), __uint_as_float(r[8 * e + 7])));
              *reinterpret_cast<uint4*>(sm.b1 + (c >> 1) * 16384 + sw128(static_cast<uint32_t>(t), (c & 1) * 4 + e)) = v;
            }
          }
          if (need_decay) {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * eg);
            tmem_st_x32(lane_addr + COL_S + 32 * c, r);
          }
        }
        if (need_decay) tmem_wait_st();
        s_valid = true;
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&sm.s_ready);
      }
      cp_async_wait<0>();  // this unit's tiles (queued a unit ago) have landed
      fence_proxy_async_smem();
      mbar_arrive(&sm.ld_full[i & 1]);
      // the next unit's tiles into the other stage, after the state has gone out: the copy instructions are off the chain
      // state -> product -> v' -> update that sets a trunk's time, and still a whole unit ahead of their use
      if (u + 1 < u_end) queue_copies(sm.st[(i & 1) ^ 1], mn.tok, mn.row, mn.c0);

      if (!mbar_wait(wc, &sm.d1_done, (n_d1++) & 1u, ST_TIMEOUT_TMEM)) break;
      tc_fence_after();
      if (t < 64) {
        // v' = U - W S for token row t, as bf16 rows of the two B operands
        const float dec = m_tok >= 0 ? fast_exp2(m_gl - m_g) : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_x32(lane_addr + COL_D1 + 32 * c, r);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t pn[4], pd[4];
            const uint32_t uw[4] = {urow[4 * c + e].x, urow[4 * c + e].y, urow[4 * c + e].z, urow[4 * c + e].w};
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const float v0 = m_tok >= 0 ? bf2_lo(uw[x]) - __uint_as_float(r[8 * e + 2 * x]) : 0.f;
              const float v1 = m_tok >= 0 ? bf2_hi(uw[x]) - __uint_as_float(r[8 * e + 2 * x + 1]) : 0.f;
              pn[x] = pack_bf16x2(v0, v1), pd[x] = pack_bf16x2(v0 * dec, v1 * dec);
            }
            const uint32_t off = (c >> 1) * 8192 + sw128(static_cast<uint32_t>(t), (c & 1) * 4 + e);
            *reinterpret_cast<uint4*>(sm.vn + off) = make_uint4(pn[0], pn[1], pn[2], pn[3]);
            *reinterpret_cast<uint4*>(sm.vd + off) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&sm.v_ready);
      }
      if (!mbar_wait(wc, &sm.d2_done, (n_d2++) & 1u, ST_TIMEOUT_TMEM)) break;
      tc_fence_after();
      if (t >= 64) {
        // o = scale [(Q S) 2^G + P v'] for token row t - 64 (the tensor-memory loads are warp-wide; only the store is per row)
        const float eg = fast_exp2(m_g) * a.scale, sc = a.scale;
        __nv_bfloat16* dst = a.o + (static_cast<int64_t>(m_tok >= 0 ? m_row : 0) * a.Hv + hv) * TK;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r1[32], r2[32];
          tmem_ld_x32(lane_addr + COL_D1 + 32 * c, r1);
          tmem_ld_x32(lane_addr + COL_D2 + 32 * c, r2);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t po[4];
#pragma unroll
            for (int x = 0; x < 4; ++x)
              po[x] = pack_bf16x2(__uint_as_float(r1[8 * e + 2 * x]) * eg + __uint_as_float(r2[8 * e + 2 * x]) * sc,
                                  __uint_as_float(r1[8 * e + 2 * x + 1]) * eg + __uint_as_float(r2[8 * e + 2 * x + 1]) * sc);
            if (m_tok >= 0) *reinterpret_cast<uint4*>(dst + 32 * c + 8 * e) = make_uint4(po[0], po[1], po[2], po[3]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&sm.d_free);  // this thread's reads of D1 / D2 are done
      if (flags & UF_UPDATE_TC) upd_pending = true, dirty = true, s_valid = false;
      prev_slot = mc.slot;
      mc = mn, mn = mp;
    }
    // the last unit's update, and its state if a deeper level reads it
    if (upd_pending && !sm.abort_flag && mbar_wait(wc, &sm.upd_done, n_upd & 1u, ST_TIMEOUT_OTHER)) {
      tc_fence_after();
      const int slot = prev_slot;
      if (slot >= 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_x32(lane_addr + COL_S + 32 * c, r);
          tmem_wait_ld();
          float4* dst = reinterpret_cast<float4*>(a.h_out + ((static_cast<int64_t>(slot) * a.Hv + hv) * TK + t) * TK + 32 * c);
#pragma unroll
          for (int e = 0; e < 8; ++e)
            dst[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]), __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
        }
      }
    }
    cp_async_wait<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 512);
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_gdn_tree_scan_tc(const void* q, const void* k, void* o, int64_t n_rows, int64_t q_pitch, int32_t Hk, int32_t Hv,
                                      int32_t K, int32_t V, float scale, int64_t plan_tokens, const int32_t* grp_parent,
                                      const int32_t* grp_ubeg, const int32_t* units, const int32_t* unit_rows, int64_t n_groups,
                                      const float* h_in, float* h_out, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_groups == 0 || plan_tokens == 0) return 0;  // an empty level
  SPINF_CHECK_ARG(q && k && o && grp_parent && grp_ubeg && units && unit_rows && workspace);
  SPINF_CHECK_ARG(K == TK && V == TK && Hk > 0 && Hv > 0 && Hv % Hk == 0 && Hv <= 65535 && n_rows >= 0 && n_rows < (1ll << 31));
  SPINF_CHECK_ARG(q_pitch >= static_cast<int64_t>(Hk) * TK && q_pitch % 8 == 0 && n_groups > 0 && n_groups < (1ll << 31));
  SPINF_CHECK_ARG(plan_tokens > 0 && plan_tokens < (1ll << 31) && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0);
  SPINF_CHECK_ARG(workspace_bytes >= spinf_gdn_tree_workspace_bytes(plan_tokens, Hv));
  GdnTcArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q), a.k = static_cast<const __nv_bfloat16*>(k), a.o = static_cast<__nv_bfloat16*>(o);
  a.q_pitch = q_pitch, a.Hk = Hk, a.Hv = Hv, a.scale = scale;
  auto align256 = [](int64_t x) { return (x + 255) / 256 * 256; };
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const int64_t wu = align256(plan_tokens * Hv * TK * 2);
  a.w_ws = reinterpret_cast<const __nv_bfloat16*>(ws), a.u_ws = reinterpret_cast<const __nv_bfloat16*>(ws + wu);
  a.p_ws = reinterpret_cast<const __nv_bfloat16*>(ws + 2 * wu);
  a.g_ws = reinterpret_cast<const float*>(ws + 2 * wu + align256(plan_tokens * Hv * TC * 2));
  a.grp_parent = grp_parent, a.grp_ubeg = grp_ubeg, a.units = units, a.unit_rows = unit_rows, a.h_in = h_in, a.h_out = h_out;
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return SPINF_ERR_CUDA;
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  const int smem = static_cast<int>(sizeof(TcSmem)) + 1024;
  static std::atomic<bool> attr_set[64];
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_tree_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev].store(true, std::memory_order_release);
  }
  gdn_tree_scan_tc_kernel<<<dim3(static_cast<unsigned>(n_groups), static_cast<unsigned>(Hv)), TC_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(a, status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
