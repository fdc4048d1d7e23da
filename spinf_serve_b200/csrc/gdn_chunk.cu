// Gated DeltaNet, chunked form, for long segments (sm_100a). The recurrence of gdn.cu
//     S *= exp(g_t);  v'_t = (v_t - S^T k_t) beta_t;  S += k_t (x) v'_t;  o_t = S^T (q_t scale)
// taken 64 tokens at a time in the WY representation (Yang et al., "Gated Delta Networks"; the reference runs flash-linear-attention
// 0.5.2's chunk pipeline, spinf_serve/models/qwen35/gdn.py:109-133, whose rounding points are kept: bf16 operands into every
// product, fp32 accumulation, fp32 state). With G_t the running sum of g inside the chunk (in log2 units):
//     A[t,s] = beta_t (k_t . k_s) 2^(G_t - G_s)   for s < t, else 0            T = (I + A)^-1
//     W = T (beta K 2^G)        U = T (beta V)                                  (no dependence on the state: all chunks in parallel)
//     v' = U - W S              o = scale [(Q S) 2^G + tril(Q K^T 2^(G_t - G_s)) v']
//     S <- S 2^(G_last) + K^T (v' 2^(G_last - G))                               (one chunk after the other)
// Two kernels: gdn_chunk_prep_kernel, one CTA per (chunk, value head), computes G, W and U into a workspace; gdn_chunk_scan_kernel,
// one CTA per (segment, value head), walks the segment's chunks with the 128 x 128 state in registers as the accumulator fragments
// of warp-level bf16 MMAs. The chain per chunk is five small products (64..128 rows) that depend on one another, so the kernel is
// bound by their latency, not by tensor throughput: operands stay in shared memory and registers of one CTA (ldmatrix + mma.sync),
// with no tensor-memory round trip between the steps.
#include <atomic>
#include "common.cuh"
#include "gdn_mma.cuh"
#include "host_util.h"

namespace spinf {

struct GdnChunkArgs {
  const __nv_bfloat16 *q, *k, *v, *beta;
  const float* g;
  __nv_bfloat16* o;
  int64_t q_pitch, v_pitch, g_pitch;  // row pitches in elements (g and beta share g_pitch)
  int Hk, Hv;
  float scale;
  const int64_t* cu;   // [n_seg + 1] call-order token offsets
  const int64_t* idx;  // optional: stream row of call token p
  int64_t n_rows;      // rows of the stream tensors
  const float* h0;
  const int64_t* h0_idx;
  float* ht;
  const int64_t* ht_idx;
  const int32_t* chunk_seg;  // [n_chunks] segment of the chunk
  const int32_t* chunk_t0;   // [n_chunks] first token of the chunk within its segment
  __nv_bfloat16 *w_ws, *u_ws;  // [call tokens, Hv, CK] bf16
  float* g_ws;                 // [call tokens, Hv] fp32: G in log2 units
};

// ------------------------------------------------------------------------------------------------ chunk preparation
struct PrepSmem {
  __nv_bfloat16 k[CT * LD];
  __nv_bfloat16 v[CT * LD];
  float a[CT * (CT + 1)];
  __nv_bfloat16 t[CT * (CT + 8)];
  float g[CT], beta[CT];
  int64_t row[CT];
};

__global__ void __launch_bounds__(128) gdn_chunk_prep_kernel(const GdnChunkArgs a) {
  extern __shared__ __align__(16) uint8_t prep_raw[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(prep_raw);
  const int chunk = blockIdx.x, hv = blockIdx.y;
  const int hk = hv / (a.Hv / a.Hk);
  const int seg = a.chunk_seg[chunk], t0 = a.chunk_t0[chunk];
  const int64_t bos = a.cu[seg];
  const int64_t left = a.cu[seg + 1] - bos - t0;
  const int len = left < CT ? static_cast<int>(left) : CT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;

  if (tid < CT) {
    int64_t r = -1;
    if (tid < len) {
      r = a.idx ? a.idx[bos + t0 + tid] : bos + t0 + tid;
      if (r < 0 || r >= a.n_rows) r = -1;  // never read outside the stream: the row counts as padding
    }
    sm.row[tid] = r;
    sm.g[tid] = r >= 0 ? a.g[r * a.g_pitch + hv] : 0.f;
    sm.beta[tid] = r >= 0 ? __bfloat162float(a.beta[r * a.g_pitch + hv]) : 0.f;
  }
  __syncthreads();
  load_tile(sm.k, [&](int t) { return sm.row[t] >= 0 ? a.k + sm.row[t] * a.q_pitch + hk * CK : nullptr; }, a.k, tid, 128);
  load_tile(sm.v, [&](int t) { return sm.row[t] >= 0 ? a.v + sm.row[t] * a.v_pitch + hv * CK : nullptr; }, a.v, tid, 128);
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
  if (tid < len) a.g_ws[(bos + t0 + tid) * a.Hv + hv] = sm.g[tid];

  // A = K K^T: warp w takes rows [16 w, 16 w + 16)
  {
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < CK / 16; ++kk) {
      uint32_t fa[4];
      ldsm_x4(fa, frag_a(sm.k, LD, 16 * warp, 16 * kk, lane));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t fb[4];
        ldsm_x4(fb, frag_b(sm.k, LD, 16 * np, 16 * kk, lane));
        mma_bf16(acc[2 * np], fa, fb[0], fb[1]);
        mma_bf16(acc[2 * np + 1], fa, fb[2], fb[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = 16 * warp + gq + (e >> 1) * 8, s = 8 * nt + 2 * tq + (e & 1);
        const float val = s < t ? acc[nt][e] * fast_exp2(sm.g[t] - sm.g[s]) * sm.beta[t] : 0.f;
        sm.a[t * (CT + 1) + s] = val;
      }
  }
  __syncthreads();
  // T = (I + A)^-1 by forward substitution, one column per thread: x_t = [t == c] - sum_{s < t} A[t,s] x_s
  if (tid < CT) {
    float x[CT];
#pragma unroll
    for (int t = 0; t < CT; ++t) {
      float s0 = t == tid ? 1.f : 0.f, s1 = 0.f;
#pragma unroll
      for (int s = 0; s + 1 < t; s += 2) {
        s0 = fmaf(-sm.a[t * (CT + 1) + s], x[s], s0);
        s1 = fmaf(-sm.a[t * (CT + 1) + s + 1], x[s + 1], s1);
      }
      if (t & 1) s0 = fmaf(-sm.a[t * (CT + 1) + t - 1], x[t - 1], s0);
      x[t] = s0 + s1;
      sm.t[t * (CT + 8) + tid] = __float2bfloat16_rn(x[t]);
    }
  }
  // K <- bf16(k beta 2^G), V <- bf16(v beta) in place (A has been taken from K already)
  for (int i = tid; i < CT * (CK / 2); i += 128) {
    const int t = i / (CK / 2), c = (i % (CK / 2)) * 2;
    const float b = sm.beta[t], e = fast_exp2(sm.g[t]);
    uint32_t* pk = reinterpret_cast<uint32_t*>(sm.k + t * LD + c);
    uint32_t* pv = reinterpret_cast<uint32_t*>(sm.v + t * LD + c);
    *pk = pack_bf16x2(bf2_lo(*pk) * b * e, bf2_hi(*pk) * b * e);
    *pv = pack_bf16x2(bf2_lo(*pv) * b, bf2_hi(*pv) * b);
  }
  __syncthreads();
  // W = T (k beta 2^G), U = T (v beta): warp w takes rows [16 w, 16 w + 16) of both
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = which ? sm.v : sm.k;
    __nv_bfloat16* dst = which ? a.u_ws : a.w_ws;
    float acc[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < CT / 16; ++ks) {
      uint32_t fa[4];
      ldsm_x4(fa, frag_a(sm.t, CT + 8, 16 * warp, 16 * ks, lane));
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t fb[4];
        ldsm_x4_t(fb, frag_b_t(src, LD, 16 * ks, 16 * np, lane));
        mma_bf16(acc[2 * np], fa, fb[0], fb[1]);
        mma_bf16(acc[2 * np + 1], fa, fb[2], fb[3]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int t = 16 * warp + gq + 8 * h;
      if (t < len) {
        __nv_bfloat16* row = dst + ((bos + t0 + t) * a.Hv + hv) * CK;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
          *reinterpret_cast<uint32_t*>(row + 8 * nt + 2 * tq) = pack_bf16x2(acc[nt][2 * h], acc[nt][2 * h + 1]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ scan over a segment's chunks
struct ScanIn {
  __nv_bfloat16 w[CT * LD], u[CT * LD], k[CT * LD], q[CT * LD];
  float g[CT];
  int64_t row[CT];
};
struct ScanSmem {
  ScanIn in[2];  // the next chunk's operands arrive (cp.async) while the current chunk is worked on
  __nv_bfloat16 h[CK * LD];
  __nv_bfloat16 vn[CT * LD], vd[CT * LD];
};

__global__ void __launch_bounds__(128, 1) gdn_chunk_scan_kernel(const GdnChunkArgs a) {
  extern __shared__ __align__(16) uint8_t scan_raw[];
  ScanSmem& sm = *reinterpret_cast<ScanSmem*>(scan_raw);
  const int seg = blockIdx.x / a.Hv, hv = blockIdx.x % a.Hv;
  const int hk = hv / (a.Hv / a.Hk);
  const int64_t bos = a.cu[seg];
  const int T = static_cast<int>(a.cu[seg + 1] - bos);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;

  // state: warp w owns rows [32 w, 32 w + 32) (two 16-row tiles) x 128 columns (16 tiles) as accumulator fragments
  float hst[2][16][4];
  const int64_t src = a.h0 ? a.h0_idx[seg] : -1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float2 val = make_float2(0.f, 0.f);
        if (src >= 0) val = *reinterpret_cast<const float2*>(a.h0 + ((src * a.Hv + hv) * CK + 32 * warp + 16 * mt + gq + 8 * h) * CK + 8 * nt + 2 * tq);
        hst[mt][nt][2 * h] = val.x, hst[mt][nt][2 * h + 1] = val.y;
      }

  // rows and running log-decay of a chunk, then its four operand tiles (one cp.async group per chunk)
  auto stage_rows = [&](ScanIn& in, int t0) {
    if (tid < CT) {
      const int len = min(CT, T - t0);
      int64_t r = -1;
      if (tid < len) {
        r = a.idx ? a.idx[bos + t0 + tid] : bos + t0 + tid;
        if (r < 0 || r >= a.n_rows) r = -1;  // never read outside the stream: the row counts as padding
      }
      in.row[tid] = r;
      in.g[tid] = tid < len ? a.g_ws[(bos + t0 + tid) * a.Hv + hv] : 0.f;
    }
  };
  auto stage_tiles = [&](ScanIn& in, int t0) {
    const int len = min(CT, T - t0);
    load_tile(in.w, [&](int t) { return t < len ? a.w_ws + ((bos + t0 + t) * a.Hv + hv) * CK : nullptr; }, a.w_ws, tid, 128);
    load_tile(in.u, [&](int t) { return t < len ? a.u_ws + ((bos + t0 + t) * a.Hv + hv) * CK : nullptr; }, a.u_ws, tid, 128);
    load_tile(in.k, [&](int t) { return in.row[t] >= 0 ? a.k + in.row[t] * a.q_pitch + hk * CK : nullptr; }, a.k, tid, 128);
    load_tile(in.q, [&](int t) { return in.row[t] >= 0 ? a.q + in.row[t] * a.q_pitch + hk * CK : nullptr; }, a.q, tid, 128);
    cp_async_commit();
  };
  stage_rows(sm.in[0], 0);
  __syncthreads();
  stage_tiles(sm.in[0], 0);

  for (int t0 = 0, c = 0; t0 < T; t0 += CT, ++c) {
    const int len = min(CT, T - t0);
    ScanIn& cur = sm.in[c & 1];
    ScanIn& nxt = sm.in[(c & 1) ^ 1];
    const bool more = t0 + CT < T;
    __syncthreads();  // the previous chunk's readers of the other buffer, of the state copy and of v' are done
    if (more) stage_rows(nxt, t0 + CT);
    // the state as the bf16 operand of W S and Q S
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint32_t*>(sm.h + (32 * warp + 16 * mt + gq + 8 * h) * LD + 8 * nt + 2 * tq) =
              pack_bf16x2(hst[mt][nt][2 * h], hst[mt][nt][2 * h + 1]);
    __syncthreads();
    if (more) {
      stage_tiles(nxt, t0 + CT);
      cp_async_wait<1>();  // this chunk's group has landed; the next one stays in flight
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float g_last = cur.g[len - 1];

    // v' = U - W S for rows [16 w, 16 w + 16); kept as bf16 (v') and as bf16(v' 2^(G_last - G)) for the state update
    {
      float acc[16][4];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < CK / 16; ++kk) {
        uint32_t fa[4];
        ldsm_x4(fa, frag_a(cur.w, LD, 16 * warp, 16 * kk, lane));
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.h, LD, 16 * kk, 16 * np, lane));
          mma_bf16(acc[2 * np], fa, fb[0], fb[1]);
          mma_bf16(acc[2 * np + 1], fa, fb[2], fb[3]);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = 16 * warp + gq + 8 * h;
        const float dec = t < len ? fast_exp2(g_last - cur.g[t]) : 0.f;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          const uint32_t uu = *reinterpret_cast<const uint32_t*>(cur.u + t * LD + 8 * nt + 2 * tq);
          const float v0 = bf2_lo(uu) - acc[nt][2 * h], v1 = bf2_hi(uu) - acc[nt][2 * h + 1];
          *reinterpret_cast<uint32_t*>(sm.vn + t * LD + 8 * nt + 2 * tq) = pack_bf16x2(v0, v1);
          *reinterpret_cast<uint32_t*>(sm.vd + t * LD + 8 * nt + 2 * tq) = pack_bf16x2(v0 * dec, v1 * dec);
        }
      }
    }
    __syncthreads();

    // o = scale [(Q S) 2^G + tril(Q K^T 2^(G_t - G_s)) v'] for rows [16 w, 16 w + 16)
    {
      const int ta = 16 * warp + gq, tb = ta + 8;
      const float ga = cur.g[ta], gb = cur.g[tb];
      // the decayed, causally masked scores first, as the bf16 A operand of their product with v': two 8-column score tiles
      // make one 16 x 16 block
      uint32_t pf[CT / 16][4];
      {
        float p[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) p[nt][0] = p[nt][1] = p[nt][2] = p[nt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < CK / 16; ++kk) {
          uint32_t fa[4];
          ldsm_x4(fa, frag_a(cur.q, LD, 16 * warp, 16 * kk, lane));
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            uint32_t fb[4];
            ldsm_x4(fb, frag_b(cur.k, LD, 16 * np, 16 * kk, lane));
            mma_bf16(p[2 * np], fa, fb[0], fb[1]);
            mma_bf16(p[2 * np + 1], fa, fb[2], fb[3]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int s0 = 8 * nt + 2 * tq, s1 = s0 + 1;
          const float gs0 = cur.g[s0], gs1 = cur.g[s1];
          const float a00 = s0 <= ta ? p[nt][0] * fast_exp2(ga - gs0) : 0.f, a01 = s1 <= ta ? p[nt][1] * fast_exp2(ga - gs1) : 0.f;
          const float a10 = s0 <= tb ? p[nt][2] * fast_exp2(gb - gs0) : 0.f, a11 = s1 <= tb ? p[nt][3] * fast_exp2(gb - gs1) : 0.f;
          pf[nt >> 1][2 * (nt & 1)] = pack_bf16x2(a00, a01);
          pf[nt >> 1][2 * (nt & 1) + 1] = pack_bf16x2(a10, a11);
        }
      }
      float acc[16][4];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < CK / 16; ++kk) {
        uint32_t fa[4];
        ldsm_x4(fa, frag_a(cur.q, LD, 16 * warp, 16 * kk, lane));
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.h, LD, 16 * kk, 16 * np, lane));
          mma_bf16(acc[2 * np], fa, fb[0], fb[1]);
          mma_bf16(acc[2 * np + 1], fa, fb[2], fb[3]);
        }
      }
      const float ea = fast_exp2(ga), eb = fast_exp2(gb);
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) acc[nt][0] *= ea, acc[nt][1] *= ea, acc[nt][2] *= eb, acc[nt][3] *= eb;
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.vn, LD, 16 * ks, 16 * np, lane));
          mma_bf16(acc[2 * np], pf[ks], fb[0], fb[1]);
          mma_bf16(acc[2 * np + 1], pf[ks], fb[2], fb[3]);
        }
      }
      // through the U tile (no longer needed) so that the rows leave as 16-byte pieces
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
          *reinterpret_cast<uint32_t*>(cur.u + (16 * warp + gq + 8 * h) * LD + 8 * nt + 2 * tq) =
              pack_bf16x2(acc[nt][2 * h] * a.scale, acc[nt][2 * h + 1] * a.scale);
      __syncwarp();
      for (int i = lane; i < 16 * (CK / 8); i += 32) {
        const int t = 16 * warp + i / (CK / 8), c = i % (CK / 8);
        if (cur.row[t] >= 0) *reinterpret_cast<uint4*>(a.o + (cur.row[t] * a.Hv + hv) * CK + c * 8) = *reinterpret_cast<const uint4*>(cur.u + t * LD + c * 8);
      }
    }

    // S <- S 2^(G_last) + K^T (v' 2^(G_last - G)): warp w updates its rows [32 w, 32 w + 32)
    {
      const float eg = fast_exp2(g_last);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) hst[mt][nt][e] *= eg;
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks) {
        uint32_t fa0[4], fa1[4];
        ldsm_x4_t(fa0, frag_a_t(cur.k, LD, 16 * ks, 32 * warp, lane));
        ldsm_x4_t(fa1, frag_a_t(cur.k, LD, 16 * ks, 32 * warp + 16, lane));
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t fb[4];
          ldsm_x4_t(fb, frag_b_t(sm.vd, LD, 16 * ks, 16 * np, lane));
          mma_bf16(hst[0][2 * np], fa0, fb[0], fb[1]);
          mma_bf16(hst[0][2 * np + 1], fa0, fb[2], fb[3]);
          mma_bf16(hst[1][2 * np], fa1, fb[0], fb[1]);
          mma_bf16(hst[1][2 * np + 1], fa1, fb[2], fb[3]);
        }
      }
    }
  }

  const int64_t dstrow = a.ht ? a.ht_idx[seg] : -1;
  if (dstrow >= 0) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<float2*>(a.ht + ((dstrow * a.Hv + hv) * CK + 32 * warp + 16 * mt + gq + 8 * h) * CK + 8 * nt + 2 * tq) =
              make_float2(hst[mt][nt][2 * h], hst[mt][nt][2 * h + 1]);
  }
}

}  // namespace spinf

using namespace spinf;

extern "C" int64_t spinf_gdn_chunked_workspace_bytes(int64_t call_tokens, int32_t Hv) {
  if (call_tokens < 0 || Hv <= 0) return SPINF_ERR_BAD_ARGUMENT;
  // W and U (bf16 [tokens, Hv, 128] each), then G (fp32 [tokens, Hv]); each part 256-byte aligned
  const int64_t wu = (call_tokens * Hv * CK * 2 + 255) / 256 * 256;
  return 2 * wu + (call_tokens * Hv * 4 + 255) / 256 * 256;
}

extern "C" int spinf_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o, int64_t n_rows,
                                 int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V,
                                 float scale, const int64_t* cu, int64_t n_seg, const int64_t* idx, const float* h0,
                                 const int64_t* h0_idx, float* ht, const int64_t* ht_idx, const int32_t* chunk_seg,
                                 const int32_t* chunk_t0, int64_t n_chunks, int64_t call_tokens, void* workspace,
                                 int64_t workspace_bytes, void* stream) {
  if (n_seg == 0 || n_chunks == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(q && k && v && g && beta && o && cu && n_rows >= 0 && n_seg >= 0 && Hk > 0 && Hv > 0 && Hv % Hk == 0);
  SPINF_CHECK_ARG(K == CK && V == CK);
  SPINF_CHECK_ARG(q_pitch >= static_cast<int64_t>(Hk) * CK && q_pitch % 8 == 0 && v_pitch >= static_cast<int64_t>(Hv) * CK && v_pitch % 8 == 0 && g_pitch >= Hv);
  SPINF_CHECK_ARG((h0 == nullptr) == (h0_idx == nullptr) && (ht == nullptr) == (ht_idx == nullptr));
  SPINF_CHECK_ARG(n_seg * Hv < (1ll << 31) && n_chunks >= 0 && n_chunks < (1ll << 31) && Hv <= 65535 && call_tokens >= 0);
  if (n_seg == 0 || n_chunks == 0) return 0;
  SPINF_CHECK_ARG(chunk_seg && chunk_t0 && workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0);
  SPINF_CHECK_ARG(workspace_bytes >= spinf_gdn_chunked_workspace_bytes(call_tokens, Hv));
  GdnChunkArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q), a.k = static_cast<const __nv_bfloat16*>(k), a.v = static_cast<const __nv_bfloat16*>(v);
  a.g = g, a.beta = static_cast<const __nv_bfloat16*>(beta), a.o = static_cast<__nv_bfloat16*>(o);
  a.q_pitch = q_pitch, a.v_pitch = v_pitch, a.g_pitch = g_pitch, a.Hk = Hk, a.Hv = Hv, a.scale = scale;
  a.cu = cu, a.idx = idx, a.n_rows = n_rows, a.h0 = h0, a.h0_idx = h0_idx, a.ht = ht, a.ht_idx = ht_idx;
  a.chunk_seg = chunk_seg, a.chunk_t0 = chunk_t0;
  const int64_t wu = (call_tokens * Hv * CK * 2 + 255) / 256 * 256;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  a.w_ws = reinterpret_cast<__nv_bfloat16*>(ws), a.u_ws = reinterpret_cast<__nv_bfloat16*>(ws + wu);
  a.g_ws = reinterpret_cast<float*>(ws + 2 * wu);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice from two threads is harmless
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PrepSmem))));
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(ScanSmem))));
    attr_set[dev].store(true, std::memory_order_release);
  }
  gdn_chunk_prep_kernel<<<dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(Hv)), 128, sizeof(PrepSmem), st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  gdn_chunk_scan_kernel<<<static_cast<unsigned>(n_seg * Hv), 128, sizeof(ScanSmem), st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
