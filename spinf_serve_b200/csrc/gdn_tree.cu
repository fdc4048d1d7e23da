// Gated DeltaNet over a whole trie plan (sm_100a): every segment of the plan, long or short, in the chunked (WY) form, with the
// state of a parent segment held on the SM while its children are read against it.
//
// The recurrence   S *= exp(g_t);  v'_t = (v_t - S^T k_t) beta_t;  S += k_t (x) v'_t;  o_t = S^T (q_t scale)
// over at most 64 tokens at a time (G_t = running sum of g inside the chunk, log2 units; Yang et al., "Gated Delta Networks"; the
// rounding points are those of the chunk pipeline the reference runs for its long segments, spinf_serve/models/qwen35/gdn.py:109-133:
// bf16 operands into every product, fp32 accumulation, fp32 state):
//     A[t,s] = beta_t (k_t . k_s) 2^(G_t - G_s)  (s < t)        T = (I + A)^-1
//     W = T (beta K 2^G)     U = T (beta V)     P = tril(Q K^T 2^(G_t - G_s))       no dependence on the state
//     v' = U - W S           o = scale [(Q S) 2^G + P v']          S <- S 2^(G_last) + K^T (v' 2^(G_last - G))
//
// Two kernels.
//   gdn_tree_prep_kernel   one CTA per (chunk, value head), four to an SM, every chunk of every segment of the plan in ONE launch:
//                          the products K K^T and Q K^T, the running log-decay G, T (a blocked inverse: the 16 x 16
//                          diagonal blocks by substitution in fp32, one column per thread; the blocks below them merged in rounds
//                          of 16 x 16 TF32 tensor-core products, one block per warp), W, U and P into a workspace indexed by plan
//                          token. Blocks past the chunk's tokens are skipped everywhere (a 20-token branch costs two blocks).
//   gdn_tree_scan_kernel   one launch per level of the trie; one CTA per (group of siblings, value head, 64-column slice of the
//                          state). The columns of S evolve independently, so slicing V multiplies the parallel chains without
//                          changing a value. The CTA loads its parent's state slice ONCE (fp32 accumulator fragments in registers,
//                          a bf16 copy in shared memory as the MMA operand) and walks the group's units:
//                            - a "light" child (one chunk, no state to keep: the 20-token question branches) only reads the state:
//                              v' and o need S, nothing writes it, so siblings are packed up to four to a 64-row unit (16-row
//                              aligned, P block-diagonal) and the state never moves;
//                            - a "heavy" child (several chunks, or a state a deeper level needs) updates the registers chunk by
//                              chunk, stores its final state where its children will find it, and the parent's state is reloaded
//                              (from L2) before the next sibling.
// A segment's values depend only on its own tokens and its parent's state: packing light siblings adds exact zeros to their sums
// (16-aligned offsets keep every product in the same MMA position), and the V slices never interact.
#include <atomic>
#include "common.cuh"
#include "gdn_mma.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int BV = 64;            // state columns per scan CTA
static constexpr int LDS = BV + 8;       // row stride of the 64-column bf16 tiles
static constexpr int UNIT_WORDS = 12;    // n_pieces, flags, store_slot, pad, 4 x (first plan token, length)
static constexpr int UF_UPDATE = 1;      // the unit's chunk updates the state (heavy child)
static constexpr int UF_PARENT = 2;      // the unit must see the parent's state (light unit, or the first chunk of a heavy child)

struct GdnTreeArgs {
  const __nv_bfloat16 *q, *k, *v, *beta;
  const float* g;
  __nv_bfloat16* o;
  int64_t q_pitch, v_pitch, g_pitch;
  int Hk, Hv;
  float scale;
  const int64_t* row_of;  // [plan_tokens] stream (or compact) row of plan token p
  int64_t n_rows, plan_tokens;
  __nv_bfloat16 *w_ws, *u_ws;  // [plan_tokens, Hv, 128]
  __nv_bfloat16* p_ws;         // [plan_tokens, Hv, 64]: row t of its chunk's P, columns relative to the chunk's first token
  float* g_ws;                 // [plan_tokens, Hv]
  // prep
  const int32_t *chunk_p0, *chunk_len;
  // scan (one level)
  const int32_t *grp_parent, *grp_ubeg, *units;
  const float* h_in;
  float* h_out;
};

// ------------------------------------------------------------------------------------------------ preparation
// The merge of the inverse's blocks runs on the tensor cores in TF32 (m16n8k8), as the chunk pipeline the reference calls does it:
// a 16 x 16 block product per warp, operands read from fp32 tiles of row stride CT + 1.
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// acc[nt] (16 x 8 each, nt = 0, 1) += A (16 x 16 at pa, row stride lda) * B (16 x 16 at pb, row stride ldb)
__device__ __forceinline__ void block16_mma(float (&acc)[2][4], const float* pa, int lda, const float* pb, int ldb, int lane) {
  const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    uint32_t fa[4];
    fa[0] = to_tf32(pa[gq * lda + 8 * ks + tq]);
    fa[1] = to_tf32(pa[(gq + 8) * lda + 8 * ks + tq]);
    fa[2] = to_tf32(pa[gq * lda + 8 * ks + tq + 4]);
    fa[3] = to_tf32(pa[(gq + 8) * lda + 8 * ks + tq + 4]);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      mma_tf32(acc[nt], fa, to_tf32(pb[(8 * ks + tq) * ldb + 8 * nt + gq]), to_tf32(pb[(8 * ks + tq + 4) * ldb + 8 * nt + gq]));
  }
}

// Shared memory of a preparation CTA, 56 832 bytes so that four CTAs share an SM. Three regions are reused as the steps go:
//   r1  K (padded rows)                      -> K~ = bf16(k beta 2^G), in place
//   r2  Q (padded rows) -> the inverse X in fp32 ([64][65]) -> T = bf16(X) as an MMA operand ([64][72])
//   r3  A in fp32 ([64][65])                 -> V (64 rows of 256 bytes, 16-byte pieces XOR-swizzled by the row) -> V~ = bf16(v beta)
static constexpr int LDA = CT + 2;  // row stride of the fp32 A and X: the two diagonal blocks a warp solves lie 16 banks apart
struct TreePrepSmem {
  __nv_bfloat16 r1[CT * LD];
  __nv_bfloat16 r2[CT * LD];
  float r3[CT * LDA];
  float m[4 * 16 * 17];       // a warp's inner sums of a merge round (one 16 x 16 block each)
  float g[CT], beta[CT];
  int64_t row[CT];
};
static_assert(sizeof(TreePrepSmem) <= 56 * 1024, "four preparation CTAs per SM");
static_assert(CT * LDA * 4 <= CT * LD * 2 && CT * CK * 2 <= CT * LDA * 4, "the aliased tiles fit their regions");

// element (row t, column c) of the swizzled V tile: 16-byte piece c / 8 of row t sits at piece (c / 8) ^ (t & 7)
__device__ __forceinline__ int vsw(int t, int c) { return t * CK + ((((c >> 3) ^ (t & 7)) << 3) | (c & 7)); }

__global__ void __launch_bounds__(128, 4) gdn_tree_prep_kernel(const GdnTreeArgs a) {
  extern __shared__ __align__(16) uint8_t tprep_raw[];
  TreePrepSmem& sm = *reinterpret_cast<TreePrepSmem*>(tprep_raw);
  __nv_bfloat16* const ktile = sm.r1;
  __nv_bfloat16* const qtile = sm.r2;
  float* const xm = reinterpret_cast<float*>(sm.r2);               // the inverse, fp32 [64][66]
  __nv_bfloat16* const tb = sm.r2;                                 // T in bf16, [64][72]
  float* const am = sm.r3;                                         // A, fp32 [64][66]
  __nv_bfloat16* const vtile = reinterpret_cast<__nv_bfloat16*>(sm.r3);
  const int chunk = blockIdx.x, hv = blockIdx.y;
  const int hk = hv / (a.Hv / a.Hk);
  const int p0 = a.chunk_p0[chunk], len = a.chunk_len[chunk];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int mtiles = (len + 15) >> 4;
  const bool active = warp < mtiles;  // this warp's 16 rows hold tokens

  if (tid < CT) {
    int64_t r = -1;
    if (tid < len) {
      r = a.row_of[p0 + tid];
      if (r < 0 || r >= a.n_rows) r = -1;  // never read outside the stream: the row counts as padding
    }
    sm.row[tid] = r;
    sm.g[tid] = r >= 0 ? a.g[r * a.g_pitch + hv] : 0.f;
    sm.beta[tid] = r >= 0 ? __bfloat162float(a.beta[r * a.g_pitch + hv]) : 0.f;
  }
  __syncthreads();
  load_tile(ktile, [&](int t) { return sm.row[t] >= 0 ? a.k + sm.row[t] * a.q_pitch + hk * CK : nullptr; }, a.k, tid, 128);
  load_tile(qtile, [&](int t) { return sm.row[t] >= 0 ? a.q + sm.row[t] * a.q_pitch + hk * CK : nullptr; }, a.q, tid, 128);
  cp_async_commit();
  if (warp == 0) {
    // inclusive running sum of g over the chunk (two tokens per lane), then log2 units
    float x0 = sm.g[2 * lane], x1 = sm.g[2 * lane + 1];
    float s = x0 + x1;
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    const float before = s - (x0 + x1);
    sm.g[2 * lane] = (before + x0) * RCP_LN2;
    sm.g[2 * lane + 1] = (before + x0 + x1) * RCP_LN2;
  }
  cp_async_wait<0>();
  __syncthreads();
  if (tid < len) a.g_ws[static_cast<int64_t>(p0 + tid) * a.Hv + hv] = sm.g[tid];

  {
    // K K^T and Q K^T for rows [16 w, 16 w + 16), in registers until A and P are formed from them
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) kk[nt][e] = qk[nt][e] = 0.f;
    if (active) {
#pragma unroll
      for (int ks = 0; ks < CK / 16; ++ks) {
        uint32_t fk[4], fq[4];
        ldsm_x4(fk, frag_a(ktile, LD, 16 * warp, 16 * ks, lane));
        ldsm_x4(fq, frag_a(qtile, LD, 16 * warp, 16 * ks, lane));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          if (np > warp) break;  // columns past the diagonal block are masked anyway
          uint32_t fb[4];
          ldsm_x4(fb, frag_b(ktile, LD, 16 * np, 16 * ks, lane));
          mma_bf16(kk[2 * np], fk, fb[0], fb[1]);
          mma_bf16(kk[2 * np + 1], fk, fb[2], fb[3]);
          mma_bf16(qk[2 * np], fq, fb[0], fb[1]);
          mma_bf16(qk[2 * np + 1], fq, fb[2], fb[3]);
        }
      }
    }
    // A (strictly lower, fp32) into shared memory; P (lower with the diagonal, bf16) straight to the workspace
    if (active)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt > 2 * warp + 1) {  // columns past this warp's diagonal block: A there is never read, P is zero (a scan that multiplies
          // whole 64 x 64 tiles reads every column of a row)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int t = 16 * warp + gq + 8 * h;
            if (t < len) *reinterpret_cast<uint32_t*>(a.p_ws + (static_cast<int64_t>(p0 + t) * a.Hv + hv) * CT + 8 * nt + 2 * tq) = 0u;
          }
          continue;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int t = 16 * warp + gq + 8 * h, s0 = 8 * nt + 2 * tq;
          const float gt = sm.g[t], bt = sm.beta[t];
          const float d0 = fast_exp2(gt - sm.g[s0]), d1 = fast_exp2(gt - sm.g[s0 + 1]);
          am[t * LDA + s0] = s0 < t ? kk[nt][2 * h] * d0 * bt : 0.f;
          am[t * LDA + s0 + 1] = s0 + 1 < t ? kk[nt][2 * h + 1] * d1 * bt : 0.f;
          if (t < len) {
            const float p0v = s0 <= t ? qk[nt][2 * h] * d0 : 0.f, p1v = s0 + 1 <= t ? qk[nt][2 * h + 1] * d1 : 0.f;
            *reinterpret_cast<uint32_t*>(a.p_ws + (static_cast<int64_t>(p0 + t) * a.Hv + hv) * CT + s0) = pack_bf16x2(p0v, p1v);
          }
        }
      }
  }
  __syncthreads();  // A is complete; every warp has read Q: its tile is free for the inverse

  // T = (I + A)^-1. Stage 1: the diagonal 16 x 16 blocks that hold tokens, one column per thread (forward substitution in
  // registers, fp32)
  if (tid < 16 * mtiles) {
    const int b = tid >> 4, c = tid & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = i == c ? 1.f : 0.f;
#pragma unroll
      for (int t = 0; t < i; ++t) s = fmaf(-am[(16 * b + i) * LDA + 16 * b + t], x[t], s);
      x[i] = s;
      xm[(16 * b + i) * LDA + 16 * b + c] = s;
    }
  }
  __syncthreads();
  // Stage 2: the blocks below the diagonal, by distance d from it: T_ij = -T_ii sum_{k = j}^{i - 1} A_ik T_kj, one block per warp
#pragma unroll 1
  for (int d = 1; d < mtiles; ++d) {
    const int jb = warp, ib = warp + d;
    if (ib < mtiles) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int kb = jb; kb < ib; ++kb)
        block16_mma(acc, am + (16 * ib) * LDA + 16 * kb, LDA, xm + (16 * kb) * LDA + 16 * jb, LDA, lane);
      float* mw = sm.m + warp * 16 * 17;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mw[gq * 17 + 8 * nt + 2 * tq] = acc[nt][0], mw[gq * 17 + 8 * nt + 2 * tq + 1] = acc[nt][1];
        mw[(gq + 8) * 17 + 8 * nt + 2 * tq] = acc[nt][2], mw[(gq + 8) * 17 + 8 * nt + 2 * tq + 1] = acc[nt][3];
      }
      __syncwarp();
      float out[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      block16_mma(out, xm + (16 * ib) * LDA + 16 * ib, LDA, mw, 17, lane);
      float* dst = xm + (16 * ib) * LDA + 16 * jb;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        dst[gq * LDA + 8 * nt + 2 * tq] = -out[nt][0], dst[gq * LDA + 8 * nt + 2 * tq + 1] = -out[nt][1];
        dst[(gq + 8) * LDA + 8 * nt + 2 * tq] = -out[nt][2], dst[(gq + 8) * LDA + 8 * nt + 2 * tq + 1] = -out[nt][3];
      }
    }
    __syncthreads();
  }
  // A is dead: V comes into its place (in flight while T and K~ are formed)
  for (int i = tid; i < CT * (CK / 8); i += 128) {
    const int t = i / (CK / 8), c = i % (CK / 8);
    const int64_t r = sm.row[t];
    cp_async16(vtile + vsw(t, c * 8), r >= 0 ? a.v + r * a.v_pitch + hv * CK + c * 8 : a.v, r >= 0 ? 16 : 0);
  }
  cp_async_commit();
  {
    // T as the bf16 A operand, over the fp32 inverse it is read from: through registers, a barrier between reading and writing
    float tx[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int i = tid + 128 * j, t = i >> 6, s = i & 63;
      tx[j] = (s >> 4) <= (t >> 4) && t < 16 * mtiles ? xm[t * LDA + s] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int i = tid + 128 * j, t = i >> 6, s = i & 63;
      tb[t * LDS + s] = __float2bfloat16_rn(tx[j]);
    }
  }
  // K~ = bf16(k beta 2^G) in place
  for (int i = tid; i < 16 * mtiles * (CK / 2); i += 128) {
    const int t = i / (CK / 2), c = (i % (CK / 2)) * 2;
    const float b = sm.beta[t], e = fast_exp2(sm.g[t]);
    uint32_t* pk = reinterpret_cast<uint32_t*>(ktile + t * LD + c);
    *pk = pack_bf16x2(bf2_lo(*pk) * b * e, bf2_hi(*pk) * b * e);
  }
  cp_async_wait<0>();
  __syncthreads();
  // V~ = bf16(v beta) in place (a row's pieces are permuted inside the row only, so the physical row is the token)
  for (int i = tid; i < 16 * mtiles * (CK / 2); i += 128) {
    const int t = i / (CK / 2), c = (i % (CK / 2)) * 2;
    const float b = sm.beta[t];
    uint32_t* pv = reinterpret_cast<uint32_t*>(vtile + t * CK + c);
    *pv = pack_bf16x2(bf2_lo(*pv) * b, bf2_hi(*pv) * b);
  }
  __syncthreads();
  // W = T K~, U = T V~ for rows [16 w, 16 w + 16); T is block lower-triangular: k-steps up to the diagonal block only
  if (active) {
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = which ? a.u_ws : a.w_ws;
      float acc[16][4];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks) {
        if (ks > warp) break;
        uint32_t fa[4];
        ldsm_x4(fa, frag_a(tb, LDS, 16 * warp, 16 * ks, lane));
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t fb[4];
          if (which) {
            // the [k][n] pattern of frag_b_t on the swizzled tile: row k0 + (lane & 7) + 8 ((lane >> 3) & 1), column n0 + 8 (lane >> 4)
            const int kr = 16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldsm_x4_t(fb, vtile + vsw(kr, 16 * np + (lane >> 4) * 8));
          } else {
            ldsm_x4_t(fb, frag_b_t(ktile, LD, 16 * ks, 16 * np, lane));
          }
          mma_bf16(acc[2 * np], fa, fb[0], fb[1]);
          mma_bf16(acc[2 * np + 1], fa, fb[2], fb[3]);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = 16 * warp + gq + 8 * h;
        if (t < len) {
          __nv_bfloat16* row = dst + (static_cast<int64_t>(p0 + t) * a.Hv + hv) * CK;
#pragma unroll
          for (int nt = 0; nt < 16; ++nt)
            *reinterpret_cast<uint32_t*>(row + 8 * nt + 2 * tq) = pack_bf16x2(acc[nt][2 * h], acc[nt][2 * h + 1]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ scan of one level
struct TreeScanSmem {
  __nv_bfloat16 w[CT * LD], k[CT * LD], q[CT * LD];
  __nv_bfloat16 p[CT * LDS];
  __nv_bfloat16 u[CT * LDS];    // the slice's U rows, then the staged output rows
  __nv_bfloat16 s[CK * LDS];    // the state slice as the bf16 operand of W S and Q S
  __nv_bfloat16 vn[CT * LDS], vd[CT * LDS];
  // the rows of a unit (plan token, stream row, running log-decay, that of the piece's last token, the piece's first row): two
  // sets, the next unit's are looked up while this unit's tiles are in flight
  float g[2][CT], glast[2][CT];
  int64_t row[2][CT];
  int32_t tok[2][CT], col0[2][CT];
};

__global__ void __launch_bounds__(256, 2) gdn_tree_scan_kernel(const GdnTreeArgs a) {
  extern __shared__ __align__(16) uint8_t tscan_raw[];
  TreeScanSmem& sm = *reinterpret_cast<TreeScanSmem*>(tscan_raw);
  const int grp = blockIdx.x, hv = blockIdx.y, vs = blockIdx.z;
  const int hk = hv / (a.Hv / a.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int mt = warp & 3, nh = warp >> 2;  // rows [16 mt, +16) of the unit, columns [32 nh, +32) of the slice
  const int parent = a.grp_parent[grp];
  const int u_beg = a.grp_ubeg[grp], u_end = a.grp_ubeg[grp + 1];

  // the state slice: warp w owns rows [16 w, 16 w + 16) x 64 columns as accumulator fragments
  float hst[8][4];
  auto load_parent = [&]() {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float2 val = make_float2(0.f, 0.f);
        if (parent >= 0)
          val = *reinterpret_cast<const float2*>(a.h_in + ((static_cast<int64_t>(parent) * a.Hv + hv) * CK + 16 * warp + gq + 8 * h) * CK + vs * BV + 8 * nt + 2 * tq);
        hst[nt][2 * h] = val.x, hst[nt][2 * h + 1] = val.y;
      }
  };
  load_parent();
  bool dirty = false, s_valid = false;

  // rows of a unit: piece p occupies rows [off_p, off_p + len_p), off_p = the 16-aligned lengths before it
  auto stage_rows = [&](int u, int mb) {
    if (tid < CT) {
      const int32_t* ud = a.units + static_cast<int64_t>(u) * UNIT_WORDS;
      const int n_pieces = ud[0];
      int tok = -1, c0 = 0, last = -1, off = 0;
      for (int pc = 0; pc < n_pieces; ++pc) {
        const int pp0 = ud[4 + 2 * pc], pl = ud[5 + 2 * pc];
        if (tid >= off && tid < off + pl) tok = pp0 + tid - off, c0 = off, last = pp0 + pl - 1;
        off += (pl + 15) & ~15;
      }
      int64_t r = -1;
      if (tok >= 0) {
        r = a.row_of[tok];
        if (r < 0 || r >= a.n_rows) r = -1, tok = -1;
      }
      sm.tok[mb][tid] = tok, sm.col0[mb][tid] = c0, sm.row[mb][tid] = r;
      sm.g[mb][tid] = tok >= 0 ? a.g_ws[static_cast<int64_t>(tok) * a.Hv + hv] : 0.f;
      sm.glast[mb][tid] = tok >= 0 ? a.g_ws[static_cast<int64_t>(last) * a.Hv + hv] : 0.f;
    }
  };
  if (u_beg < u_end) stage_rows(u_beg, 0);

  for (int u = u_beg; u < u_end; ++u) {
    const int32_t* ud = a.units + static_cast<int64_t>(u) * UNIT_WORDS;
    const int flags = ud[1], store_slot = ud[2];
    const int mb = (u - u_beg) & 1;
    __syncthreads();  // the previous unit's readers of every tile are done; this unit's rows are in place
    if ((flags & UF_PARENT) && dirty) {
      load_parent();
      dirty = false, s_valid = false;
    }
    {
      const __nv_bfloat16* any = a.w_ws;
      for (int i = tid; i < CT * (CK / 8); i += 256) {
        const int t = i / (CK / 8), c = i % (CK / 8);
        const int tok = sm.tok[mb][t];
        const int64_t r = sm.row[mb][t];
        const int64_t th = static_cast<int64_t>(tok) * a.Hv + hv;
        cp_async16(sm.w + t * LD + c * 8, tok >= 0 ? a.w_ws + th * CK + c * 8 : any, tok >= 0 ? 16 : 0);
        cp_async16(sm.k + t * LD + c * 8, tok >= 0 ? a.k + r * a.q_pitch + hk * CK + c * 8 : any, tok >= 0 ? 16 : 0);
        cp_async16(sm.q + t * LD + c * 8, tok >= 0 ? a.q + r * a.q_pitch + hk * CK + c * 8 : any, tok >= 0 ? 16 : 0);
      }
      for (int i = tid; i < CT * (BV / 8); i += 256) {
        const int t = i / (BV / 8), c = i % (BV / 8);
        const int tok = sm.tok[mb][t];
        const int64_t th = static_cast<int64_t>(tok) * a.Hv + hv;
        cp_async16(sm.u + t * LDS + c * 8, tok >= 0 ? a.u_ws + th * CK + vs * BV + c * 8 : any, tok >= 0 ? 16 : 0);
        const int cs = c - (sm.col0[mb][t] >> 3);  // P's columns are relative to the piece's first row
        const bool pv = tok >= 0 && cs >= 0;
        cp_async16(sm.p + t * LDS + c * 8, pv ? a.p_ws + th * CT + cs * 8 : any, pv ? 16 : 0);
      }
      cp_async_commit();
    }
    if (u + 1 < u_end) stage_rows(u + 1, mb ^ 1);  // global look-ups that overlap the copies in flight
    if (!s_valid) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint32_t*>(sm.s + (16 * warp + gq + 8 * h) * LDS + 8 * nt + 2 * tq) = pack_bf16x2(hst[nt][2 * h], hst[nt][2 * h + 1]);
      s_valid = true;
    }
    cp_async_wait<0>();
    __syncthreads();

    // W S and Q S for rows [16 mt, +16) x columns [32 nh, +32): one pass over the state operand feeds both
    float accw[4][4], accq[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) accw[nt][e] = accq[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < CK / 16; ++ks) {
      uint32_t fw[4], fq[4];
      ldsm_x4(fw, frag_a(sm.w, LD, 16 * mt, 16 * ks, lane));
      ldsm_x4(fq, frag_a(sm.q, LD, 16 * mt, 16 * ks, lane));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t fb[4];
        ldsm_x4_t(fb, frag_b_t(sm.s, LDS, 16 * ks, 32 * nh + 16 * np, lane));
        mma_bf16(accw[2 * np], fw, fb[0], fb[1]);
        mma_bf16(accw[2 * np + 1], fw, fb[2], fb[3]);
        mma_bf16(accq[2 * np], fq, fb[0], fb[1]);
        mma_bf16(accq[2 * np + 1], fq, fb[2], fb[3]);
      }
    }
    // v' = U - W S, as bf16 for P v' and as bf16(v' 2^(G_last - G)) for the state update
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int t = 16 * mt + gq + 8 * h;
      const float dec = sm.tok[mb][t] >= 0 ? fast_exp2(sm.glast[mb][t] - sm.g[mb][t]) : 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int c = 32 * nh + 8 * nt + 2 * tq;
        const uint32_t uu = *reinterpret_cast<const uint32_t*>(sm.u + t * LDS + c);
        const float v0 = bf2_lo(uu) - accw[nt][2 * h], v1 = bf2_hi(uu) - accw[nt][2 * h + 1];
        *reinterpret_cast<uint32_t*>(sm.vn + t * LDS + c) = pack_bf16x2(v0, v1);
        *reinterpret_cast<uint32_t*>(sm.vd + t * LDS + c) = pack_bf16x2(v0 * dec, v1 * dec);
      }
    }
    __syncthreads();

    // o = scale [(Q S) 2^G + P v']; P is lower-triangular over the unit's rows: k-steps up to this warp's own rows only
    {
      const int ta = 16 * mt + gq, tb2 = ta + 8;
      const float ea = fast_exp2(sm.g[mb][ta]), eb = fast_exp2(sm.g[mb][tb2]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) accq[nt][0] *= ea, accq[nt][1] *= ea, accq[nt][2] *= eb, accq[nt][3] *= eb;
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks) {
        if (ks > mt) break;
        uint32_t fp[4];
        ldsm_x4(fp, frag_a(sm.p, LDS, 16 * mt, 16 * ks, lane));
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.vn, LDS, 16 * ks, 32 * nh + 16 * np, lane));
          mma_bf16(accq[2 * np], fp, fb[0], fb[1]);
          mma_bf16(accq[2 * np + 1], fp, fb[2], fb[3]);
        }
      }
      // through the U tile (every warp has taken its U values: the barrier above) so that the rows leave as 16-byte pieces
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
          *reinterpret_cast<uint32_t*>(sm.u + (16 * mt + gq + 8 * h) * LDS + 32 * nh + 8 * nt + 2 * tq) =
              pack_bf16x2(accq[nt][2 * h] * a.scale, accq[nt][2 * h + 1] * a.scale);
    }
    __syncthreads();
    for (int i = tid; i < CT * (BV / 8); i += 256) {
      const int t = i / (BV / 8), c = i % (BV / 8);
      if (sm.row[mb][t] >= 0)
        *reinterpret_cast<uint4*>(a.o + (sm.row[mb][t] * a.Hv + hv) * CK + vs * BV + c * 8) = *reinterpret_cast<const uint4*>(sm.u + t * LDS + c * 8);
    }

    if (flags & UF_UPDATE) {
      // S <- S 2^(G_last) + K^T (v' 2^(G_last - G)): warp w updates its rows [16 w, +16); the unit is one piece
      const int len = ud[5];
      const float eg = fast_exp2(sm.glast[mb][0]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) hst[nt][e] *= eg;
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks) {
        if (16 * ks >= len) break;
        uint32_t fa[4];
        ldsm_x4_t(fa, frag_a_t(sm.k, LD, 16 * ks, 16 * warp, lane));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.vd, LDS, 16 * ks, 16 * np, lane));
          mma_bf16(hst[2 * np], fa, fb[0], fb[1]);
          mma_bf16(hst[2 * np + 1], fa, fb[2], fb[3]);
        }
      }
      dirty = true, s_valid = false;
      if (store_slot >= 0) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            *reinterpret_cast<float2*>(a.h_out + ((static_cast<int64_t>(store_slot) * a.Hv + hv) * CK + 16 * warp + gq + 8 * h) * CK + vs * BV + 8 * nt + 2 * tq) =
                make_float2(hst[nt][2 * h], hst[nt][2 * h + 1]);
      }
    }
  }
}

}  // namespace spinf

using namespace spinf;

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

extern "C" int64_t spinf_gdn_tree_workspace_bytes(int64_t plan_tokens, int32_t Hv) {
  if (plan_tokens < 0 || Hv <= 0) return SPINF_ERR_BAD_ARGUMENT;
  // W and U (bf16 [tokens, Hv, 128] each), P (bf16 [tokens, Hv, 64]), G (fp32 [tokens, Hv]); each part 256-byte aligned
  return 2 * align256(plan_tokens * Hv * CK * 2) + align256(plan_tokens * Hv * CT * 2) + align256(plan_tokens * Hv * 4);
}

static int tree_args(GdnTreeArgs& a, const void* q, const void* k, const void* v, const float* g, const void* beta, void* o, int64_t n_rows,
                     int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V, const int64_t* row_of,
                     int64_t plan_tokens, void* workspace, int64_t workspace_bytes) {
  SPINF_CHECK_ARG(q && k && row_of && n_rows >= 0 && plan_tokens > 0 && Hk > 0 && Hv > 0 && Hv % Hk == 0 && Hv <= 65535);
  SPINF_CHECK_ARG(K == CK && V == CK && q_pitch >= static_cast<int64_t>(Hk) * CK && q_pitch % 8 == 0);
  SPINF_CHECK_ARG(plan_tokens < (1ll << 31) && workspace && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0);
  SPINF_CHECK_ARG(workspace_bytes >= spinf_gdn_tree_workspace_bytes(plan_tokens, Hv));
  a.q = static_cast<const __nv_bfloat16*>(q), a.k = static_cast<const __nv_bfloat16*>(k), a.v = static_cast<const __nv_bfloat16*>(v);
  a.g = g, a.beta = static_cast<const __nv_bfloat16*>(beta), a.o = static_cast<__nv_bfloat16*>(o);
  a.q_pitch = q_pitch, a.v_pitch = v_pitch, a.g_pitch = g_pitch, a.Hk = Hk, a.Hv = Hv, a.scale = 0.f;
  a.row_of = row_of, a.n_rows = n_rows, a.plan_tokens = plan_tokens;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const int64_t wu = align256(plan_tokens * Hv * CK * 2);
  a.w_ws = reinterpret_cast<__nv_bfloat16*>(ws), a.u_ws = reinterpret_cast<__nv_bfloat16*>(ws + wu);
  a.p_ws = reinterpret_cast<__nv_bfloat16*>(ws + 2 * wu);
  a.g_ws = reinterpret_cast<float*>(ws + 2 * wu + align256(plan_tokens * Hv * CT * 2));
  a.chunk_p0 = a.chunk_len = a.grp_parent = a.grp_ubeg = a.units = nullptr;
  a.h_in = nullptr, a.h_out = nullptr;
  return 0;
}

static int tree_attrs() {
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  static std::atomic<bool> attr_set[64];
  if (dev < 0 || dev >= 64) return SPINF_ERR_CUDA;
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_tree_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(TreePrepSmem))));
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_tree_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(TreeScanSmem))));
    attr_set[dev].store(true, std::memory_order_release);
  }
  return 0;
}

extern "C" int spinf_gdn_tree_prep(const void* q, const void* k, const void* v, const float* g, const void* beta, int64_t n_rows,
                                   int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V,
                                   const int64_t* row_of, int64_t plan_tokens, const int32_t* chunk_p0, const int32_t* chunk_len,
                                   int64_t n_chunks, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_chunks == 0 || plan_tokens == 0) return 0;  // an empty plan: nothing to prepare
  GdnTreeArgs a;
  int r = tree_args(a, q, k, v, g, beta, nullptr, n_rows, q_pitch, v_pitch, g_pitch, Hk, Hv, K, V, row_of, plan_tokens, workspace, workspace_bytes);
  if (r) return r;
  SPINF_CHECK_ARG(v && g && beta && chunk_p0 && chunk_len && n_chunks > 0 && n_chunks < (1ll << 31));
  SPINF_CHECK_ARG(v_pitch >= static_cast<int64_t>(Hv) * CK && v_pitch % 8 == 0 && g_pitch >= Hv);
  if ((r = tree_attrs())) return r;
  a.chunk_p0 = chunk_p0, a.chunk_len = chunk_len;
  gdn_tree_prep_kernel<<<dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(Hv)), 128, sizeof(TreePrepSmem), static_cast<cudaStream_t>(stream)>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_gdn_tree_scan(const void* q, const void* k, void* o, int64_t n_rows, int64_t q_pitch, int32_t Hk, int32_t Hv, int32_t K,
                                   int32_t V, float scale, const int64_t* row_of, int64_t plan_tokens, const int32_t* grp_parent,
                                   const int32_t* grp_ubeg, const int32_t* units, int64_t n_groups, const float* h_in, float* h_out,
                                   void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_groups == 0 || plan_tokens == 0) return 0;  // an empty level
  GdnTreeArgs a;
  int r = tree_args(a, q, k, nullptr, nullptr, nullptr, o, n_rows, q_pitch, 0, 0, Hk, Hv, K, V, row_of, plan_tokens, workspace, workspace_bytes);
  if (r) return r;
  SPINF_CHECK_ARG(o && grp_parent && grp_ubeg && units && n_groups > 0 && n_groups < (1ll << 31));
  if ((r = tree_attrs())) return r;
  a.scale = scale;
  a.grp_parent = grp_parent, a.grp_ubeg = grp_ubeg, a.units = units, a.h_in = h_in, a.h_out = h_out;
  gdn_tree_scan_kernel<<<dim3(static_cast<unsigned>(n_groups), static_cast<unsigned>(Hv), CK / BV), 256, sizeof(TreeScanSmem), static_cast<cudaStream_t>(stream)>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
