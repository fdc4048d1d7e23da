// Attention of the extraction decoder's steps (spinf_serve/decode.py:71-104, `_x_attention`): a few query rows per group (slots x
// beams, one new token each) attend to three key ranges: the group's prefix (stored once per group), the templates (a slot sees
// its own prompt's template only) and the tokens the slot's own beam has generated so far. Token-major layouts throughout
// ([.., tokens, kv heads, dim]); all head dimensions that are multiples of 64 up to 512.
//
// The reference's rounding points are kept, so the product can be checked element by element: scores are bf16 products with fp32
// accumulation rounded to bf16, then scaling / soft cap / mask / softmax in fp32 over the three ranges together, the
// probabilities rounded to bf16, each range's value product rounded to bf16 and the three added in fp32. That forces the softmax
// to be complete before any value product starts, hence separate launches:
//   x_scores  (key tile of 64 | the generated range) x kv head x group : S = Q K^T on mma.sync, masked scores -> fp32 workspace
//   x_softmax one row per CTA                                          : probabilities -> bf16 workspace
//   x_values  (64 output dims x key-range part) x kv head x group      : P V per range on mma.sync, generated range on FMA -> fp32 parts
//   x_combine                                                          : the parts rounded and added as the reference adds them
// Each range is padded to a multiple of 64 columns in the workspace so every tile row starts 16-byte aligned. A decoding step is
// bound by reading the prefix K / V once per layer; these kernels read it once per (kv head, 64-dim slice) from L2.
#include "gdn_mma.cuh"
#include "host_util.h"

#include <algorithm>
#include <climits>
#include <atomic>

namespace spinf {

static constexpr int XT = 64;                // keys per tile, query rows per pass
static constexpr float X_NINF = -3.4028234663852886e38f;  // torch.finfo(float32).min: what the reference masks with

struct XAttnArgs {
  const __nv_bfloat16* q;
  int64_t q_pitch;  // elements between consecutive (group, slot) rows of q
  const __nv_bfloat16 *kp, *vp;
  const int32_t* pos_p;
  const __nv_bfloat16 *kt, *vt;
  const int32_t *pos_t, *own_t;
  __nv_bfloat16 *gk, *gv;
  const __nv_bfloat16 *k_new, *v_new;  // optional: this step's K / V rows (row g * Q + slot, head j at j * D), appended at token *step
  int64_t kv_pitch;
  const int32_t* qpos;
  const int32_t* step;
  int G, Q, H, h, D, Lp, Tt, S, beam, window;
  float scale, softcap;
  int Lp64, Tt64, S64, pitch;  // padded range widths and the workspace row pitch (their sum)
  float* scores;
  __nv_bfloat16* probs;
  float* part;   // [n_split + 2][G * H * Q][D] fp32: prefix partial sums per split, then the template's and the generated range's products
  int n_split;
  __nv_bfloat16* out;
  int64_t out_pitch;
};

__device__ __forceinline__ float x_round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float x_finish_score(float acc, float scale, float softcap) {
  float s = x_round_bf16(acc) * scale;
  if (softcap > 0.f) s = tanhf(s / softcap) * softcap;
  return s;
}

// rows m of a (group, kv head): m = slot * r + rr, query head hk * r + rr
__device__ __forceinline__ const __nv_bfloat16* x_q_row(const XAttnArgs& a, int g, int hk, int r, int m) {
  return a.q + (static_cast<int64_t>(g) * a.Q + m / r) * a.q_pitch + static_cast<int64_t>(hk * r + m % r) * a.D;
}
__device__ __forceinline__ int64_t x_ws_row(const XAttnArgs& a, int g, int hk, int r, int m) {
  return ((static_cast<int64_t>(g) * a.H + hk * r + m % r) * a.Q + m / r) * a.pitch;
}

// dynamic shared memory: [XT][D + 8] query rows, [XT][D + 8] key rows
__global__ void __launch_bounds__(128) x_scores_kernel(const XAttnArgs a) {
  extern __shared__ __align__(16) uint8_t xs_raw[];
  const int ld = a.D + 8;
  __nv_bfloat16* const qs = reinterpret_cast<__nv_bfloat16*>(xs_raw);
  __nv_bfloat16* const ks = qs + XT * ld;
  const int tile = blockIdx.x, hk = blockIdx.y, g = blockIdx.z;
  const int r = a.H / a.h, R = a.Q * r;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int np = a.Lp64 / XT, nt = a.Tt64 / XT;
  const int step = *a.step;

  if (tile >= np + nt) {
    // the generated range: slot q's rows against the keys slot q's own beam wrote; one warp per slot, four slots per CTA. The r query
    // rows of the slot stay in registers (lane l holds elements 8 l .. 8 l + 7 of every 256), the key rows stream past them.
    const int q = (tile - np - nt) * 4 + warp;
    if (q >= a.Q) return;
    const int vec = a.D / 8;
    const int n_live = min(step + 1, a.S);
    if (a.k_new && step < a.S) {
      // the slot's new token into the generated range first (GroupKV.update, spinf_serve/decode.py:60-65): each lane copies the
      // pieces it reads back below; the values are read by the value kernel, a launch later
      const int64_t dst = (((static_cast<int64_t>(g) * a.Q + q) * a.S + step) * a.h + hk) * a.D;
      const int64_t src = (static_cast<int64_t>(g) * a.Q + q) * a.kv_pitch + static_cast<int64_t>(hk) * a.D;
      for (int c = lane; c < vec; c += 32) {
        *reinterpret_cast<uint4*>(a.gk + dst + c * 8) = *reinterpret_cast<const uint4*>(a.k_new + src + c * 8);
        *reinterpret_cast<uint4*>(a.gv + dst + c * 8) = *reinterpret_cast<const uint4*>(a.v_new + src + c * 8);
      }
    }
    for (int rr = 0; rr < r; ++rr) {
      uint4 qv[2] = {};
      const __nv_bfloat16* const qr = x_q_row(a, g, hk, r, q * r + rr);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (lane + j * 32 < vec) qv[j] = *reinterpret_cast<const uint4*>(qr + (lane + j * 32) * 8);
      float* const dst = a.scores + x_ws_row(a, g, hk, r, q * r + rr) + a.Lp64 + a.Tt64;
      const __nv_bfloat16* const kbase = a.gk + (((static_cast<int64_t>(g) * a.Q + q) * a.S) * a.h + hk) * a.D;
      for (int s = n_live + lane; s < a.S64; s += 32) dst[s] = X_NINF;  // tokens not written yet, and the padding columns
      for (int s0 = 0; s0 < n_live; s0 += 4) {
        uint4 kv[4][2] = {};
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s0 + u < n_live) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              if (lane + j * 32 < vec) kv[u][j] = *reinterpret_cast<const uint4*>(kbase + static_cast<int64_t>(s0 + u) * a.h * a.D + (lane + j * 32) * 8);
          }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(&kv[u][j]);
            const __nv_bfloat162* qb = reinterpret_cast<const __nv_bfloat162*>(&qv[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 kf = __bfloat1622float2(kb[e]), qf = __bfloat1622float2(qb[e]);
              acc = fmaf(qf.x, kf.x, acc);
              acc = fmaf(qf.y, kf.y, acc);
            }
          }
          for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          if (lane == u && s0 + u < n_live) dst[s0 + u] = x_finish_score(acc, a.scale, a.softcap);
        }
      }
    }
    return;
  }

  const bool prefix = tile < np;
  const int k0 = (prefix ? tile : tile - np) * XT;
  const int L = prefix ? a.Lp : a.Tt;
  const __nv_bfloat16* const kbase = prefix ? a.kp : a.kt;
  const int32_t* const kpos = (prefix ? a.pos_p : a.pos_t) + static_cast<int64_t>(g) * L;
  const int32_t* const kown = prefix ? nullptr : a.own_t + static_cast<int64_t>(g) * L;
  const int col0 = (prefix ? 0 : a.Lp64) + k0;
  const int vec = a.D / 8;
  for (int i = tid; i < XT * vec; i += 128) {
    const int t = i / vec, c = i % vec;
    const bool ok = k0 + t < L;
    const __nv_bfloat16* p = kbase + ((static_cast<int64_t>(g) * L + (ok ? k0 + t : 0)) * a.h + hk) * a.D + c * 8;
    cp_async16(ks + t * ld + c * 8, ok ? p : kbase, ok ? 16 : 0);
  }
  cp_async_commit();
  const int gq = lane >> 2, tq = lane & 3;
  // the tile's key positions and owners once per CTA (position INT_MIN: a key nobody sees)
  __shared__ int32_t kp_s[XT], ko_s[XT];
  if (tid < XT) {
    const int key = k0 + tid;
    const bool in = key < L;
    const int kp = in ? kpos[key] : 0;
    kp_s[tid] = in && (!prefix || kp >= 0) ? kp : INT_MIN;
    ko_s[tid] = in && !prefix ? kown[key] : -1;
  }
  for (int m0 = 0; m0 < R; m0 += XT) {
    __syncthreads();  // the previous pass has read qs
    for (int i = tid; i < XT * vec; i += 128) {
      const int t = i / vec, c = i % vec;
      const bool ok = m0 + t < R;
      cp_async16(qs + t * ld + c * 8, ok ? x_q_row(a, g, hk, r, m0 + t) + c * 8 : a.q, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (m0 + warp * 16 < R) {
      float acc[8][4] = {};
      for (int kk = 0; kk < a.D; kk += 16) {
        uint32_t af[4];
        ldsm_x4(af, frag_a(qs, ld, warp * 16, kk, lane));
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          uint32_t bf[4];
          ldsm_x4(bf, frag_b(ks, ld, n2 * 16, kk, lane));
          mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
          mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
        }
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp * 16 + gq + half * 8;
        if (m >= R) continue;
        const int q = m / r;
        const int qp = a.qpos[g * a.Q + q], mine = q / a.beam;
        float* const dst = a.scores + x_ws_row(a, g, hk, r, m) + col0;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          float2 out;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = n * 8 + tq * 2 + e;
            const int kp = kp_s[c];
            bool vis = kp != INT_MIN && (prefix || ko_s[c] == mine);
            if (a.window > 0) vis = vis && (qp - kp) < a.window;
            (e ? out.y : out.x) = vis ? x_finish_score(acc[n][half * 2 + e], a.scale, a.softcap) : X_NINF;
          }
          *reinterpret_cast<float2*>(dst + n * 8 + tq * 2) = out;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(128) x_softmax_kernel(const XAttnArgs a) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const float* const s = a.scores + row * a.pitch;
  __nv_bfloat16* const p = a.probs + row * a.pitch;
  const int tid = threadIdx.x;
  constexpr int CACHE = 24;  // rows of up to 3072 columns stay in registers; longer ones are read again
  float v[CACHE];
  float m = X_NINF;
#pragma unroll
  for (int j = 0; j < CACHE; ++j) {
    const int i = tid + j * 128;
    v[j] = i < a.pitch ? s[i] : X_NINF;
    m = fmaxf(m, v[j]);
  }
  for (int i = tid + CACHE * 128; i < a.pitch; i += 128) m = fmaxf(m, s[i]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < CACHE; ++j) {
    v[j] = expf(v[j] - m);
    sum += v[j];
  }
  for (int i = tid + CACHE * 128; i < a.pitch; i += 128) sum += expf(s[i] - m);
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((tid & 31) == 0) red[4 + (tid >> 5)] = sum;
  __syncthreads();
  sum = (red[4] + red[5]) + (red[6] + red[7]);
#pragma unroll
  for (int j = 0; j < CACHE; ++j) {
    const int i = tid + j * 128;
    if (i < a.pitch) p[i] = __float2bfloat16_rn(v[j] / sum);
  }
  for (int i = tid + CACHE * 128; i < a.pitch; i += 128) p[i] = __float2bfloat16_rn(expf(s[i] - m) / sum);
}

// dynamic shared memory, two stages of: [XT][XT + 8] probabilities, [XT][XT + 8] values (keys x 64 dims of this CTA).
// blockIdx.x = dims slice * (n_split + 1) + part: parts 0 .. n_split - 1 take a run of the prefix's key tiles each (fp32 partial sums,
// added in split order by x_combine), part n_split takes the templates and the generated range.
__global__ void __launch_bounds__(128) x_values_kernel(const XAttnArgs a) {
  extern __shared__ __align__(16) uint8_t xv_raw[];
  constexpr int ld = XT + 8;
  constexpr int STAGE = 2 * XT * ld;  // elements
  __nv_bfloat16* const sm = reinterpret_cast<__nv_bfloat16*>(xv_raw);
  const int parts = a.n_split + 1;
  const int d0 = (blockIdx.x / parts) * XT, part = blockIdx.x % parts, hk = blockIdx.y, g = blockIdx.z;
  const int r = a.H / a.h, R = a.Q * r;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int step = *a.step;
  const int np = a.Lp64 / XT;
  const bool pre = part < a.n_split;
  const int t_beg = pre ? static_cast<int>(static_cast<int64_t>(np) * part / a.n_split) : 0;
  const int t_end = pre ? static_cast<int>(static_cast<int64_t>(np) * (part + 1) / a.n_split) : a.Tt64 / XT;
  const int L = pre ? a.Lp : a.Tt, col0 = pre ? 0 : a.Lp64;
  const __nv_bfloat16* const vbase = pre ? a.vp : a.vt;
  const int64_t slab = static_cast<int64_t>(a.G) * a.H * a.Q * a.D;
  for (int m0 = 0; m0 < R; m0 += XT) {
    auto stage = [&](int tile, int buf) {
      const int k0 = tile * XT;
      __nv_bfloat16* const ps = sm + buf * STAGE;
      __nv_bfloat16* const vs = ps + XT * ld;
      for (int i = tid; i < XT * 8; i += 128) {
        const int t = i >> 3, c = i & 7;
        const bool okp = m0 + t < R;
        cp_async16(ps + t * ld + c * 8, okp ? a.probs + x_ws_row(a, g, hk, r, m0 + t) + col0 + k0 + c * 8 : a.probs, okp ? 16 : 0);
        const bool okv = k0 + t < L;
        const __nv_bfloat16* p = vbase + ((static_cast<int64_t>(g) * L + (okv ? k0 + t : 0)) * a.h + hk) * a.D + d0 + c * 8;
        cp_async16(vs + t * ld + c * 8, okv ? p : vbase, okv ? 16 : 0);
      }
    };
    float acc[8][4] = {};
    __syncthreads();  // the previous pass has read both stages
    if (t_beg < t_end) stage(t_beg, 0);
    cp_async_commit();
    for (int tile = t_beg; tile < t_end; ++tile) {
      const int buf = (tile - t_beg) & 1;
      if (tile + 1 < t_end) stage(tile + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* const ps = sm + buf * STAGE;
      const __nv_bfloat16* const vs = ps + XT * ld;
      if (m0 + warp * 16 < R) {
#pragma unroll
        for (int kk = 0; kk < XT; kk += 16) {
          uint32_t af[4];
          ldsm_x4(af, frag_a(ps, ld, warp * 16, kk, lane));
#pragma unroll
          for (int n2 = 0; n2 < 4; ++n2) {
            uint32_t bf[4];
            ldsm_x4_t(bf, frag_b_t(vs, ld, kk, n2 * 16, lane));
            mma_bf16(acc[2 * n2], af, bf[0], bf[1]);
            mma_bf16(acc[2 * n2 + 1], af, bf[2], bf[3]);
          }
        }
      }
      __syncthreads();  // this stage is free for the tile after the next
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + warp * 16 + gq + half * 8;
      if (m >= R) continue;
      const int q = m / r;
      // the row of this (group, head, slot) in a slab of the partial buffer
      float* const dst = a.part + ((static_cast<int64_t>(g) * a.H + hk * r + m % r) * a.Q + q) * a.D + d0 + tq * 2;
#pragma unroll
      for (int n = 0; n < 8; ++n) *reinterpret_cast<float2*>(dst + static_cast<int64_t>(part) * slab + n * 8) = make_float2(acc[n][half * 2], acc[n][half * 2 + 1]);
      if (pre) continue;
      // the generated range: the slot's own tokens 0..step, on the FMA pipe for exactly the elements this thread holds
      const __nv_bfloat16* const pr = a.probs + x_ws_row(a, g, hk, r, m) + a.Lp64 + a.Tt64;
      const __nv_bfloat16* const vr = a.gv + ((static_cast<int64_t>(g) * a.Q + q) * a.S * a.h + hk) * a.D + d0 + tq * 2;
      float ag[8][2] = {};
      const int n_live = min(step + 1, a.S);
      for (int s = 0; s < n_live; ++s) {
        const float p = __bfloat162float(pr[s]);
        const __nv_bfloat16* const v = vr + static_cast<int64_t>(s) * a.h * a.D;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(v + n * 8));
          ag[n][0] = fmaf(p, f.x, ag[n][0]);
          ag[n][1] = fmaf(p, f.y, ag[n][1]);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) *reinterpret_cast<float2*>(dst + static_cast<int64_t>(part + 1) * slab + n * 8) = make_float2(ag[n][0], ag[n][1]);
    }
  }
}

// out = bf16( (bf16(sum of the prefix's partial sums, in split order) + bf16(templates)) + bf16(generated) ), the reference's three
// products rounded one by one and added in fp32 in its order
__global__ void x_combine_kernel(const XAttnArgs a) {
  const int64_t rows = static_cast<int64_t>(a.G) * a.H * a.Q, slab = rows * a.D;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
  if (i >= slab) return;
  float2 p = *reinterpret_cast<const float2*>(a.part + i);
  for (int sp = 1; sp < a.n_split; ++sp) {
    const float2 t = *reinterpret_cast<const float2*>(a.part + sp * slab + i);
    p.x += t.x, p.y += t.y;
  }
  const float2 t = *reinterpret_cast<const float2*>(a.part + a.n_split * slab + i);
  const float2 gn = *reinterpret_cast<const float2*>(a.part + (a.n_split + 1) * slab + i);
  const float x = (x_round_bf16(p.x) + x_round_bf16(t.x)) + x_round_bf16(gn.x);
  const float y = (x_round_bf16(p.y) + x_round_bf16(t.y)) + x_round_bf16(gn.y);
  const int64_t row = i / a.D;  // (g * H + head) * Q + q
  const int d = static_cast<int>(i % a.D);
  const int q = static_cast<int>(row % a.Q), head = static_cast<int>((row / a.Q) % a.H), g = static_cast<int>(row / (static_cast<int64_t>(a.Q) * a.H));
  *reinterpret_cast<__nv_bfloat162*>(a.out + (static_cast<int64_t>(g) * a.Q + q) * a.out_pitch + static_cast<int64_t>(head) * a.D + d) = __floats2bfloat162_rn(x, y);
}

static constexpr int X_MAX_SPLIT = 8;
static int pad64(int64_t n) { return static_cast<int>((n + XT - 1) / XT * XT); }

}  // namespace spinf

using namespace spinf;

// bytes of the workspace spinf_x_attention needs: fp32 scores and bf16 probabilities, one row per (group, query head, slot), each
// of the three key ranges padded to a multiple of 64 columns; then the fp32 partial products of the value kernel's parts
static int x_splits(int64_t Lp) {
  const int np = pad64(Lp) / XT;
  return std::max(1, std::min(X_MAX_SPLIT, (np + 5) / 6));  // about six key tiles of the prefix per CTA
}

extern "C" int64_t spinf_x_attention_workspace_bytes(int64_t G, int64_t Q, int64_t H, int64_t D, int64_t Lp, int64_t Tt, int64_t S) {
  if (G <= 0 || Q <= 0 || H <= 0 || D <= 0 || Lp < 0 || Tt < 0 || S <= 0) return 0;
  const int64_t pitch = pad64(Lp) + pad64(Tt) + pad64(S);
  return G * H * Q * (pitch * 6 + (x_splits(Lp) + 2) * D * 4) + 256;
}

extern "C" int spinf_x_attention(const void* q, int64_t q_pitch, const void* kp, const void* vp, const int32_t* pos_p, int64_t Lp,
                                 const void* kt, const void* vt, const int32_t* pos_t, const int32_t* own_t, int64_t Tt, void* gk,
                                 void* gv, int64_t S, const void* k_new, const void* v_new, int64_t kv_pitch, const int32_t* qpos,
                                 const int32_t* step, int64_t G, int64_t Q, int64_t H,
                                 int64_t h, int64_t D, int32_t beam, int32_t window, float scale, float softcap, void* out,
                                 int64_t out_pitch, void* workspace, int64_t workspace_bytes, void* stream) {
  if (G == 0 || Q == 0) return 0;
  SPINF_CHECK_ARG(q && gk && gv && qpos && step && out && workspace && G > 0 && Q > 0 && H > 0 && h > 0 && H % h == 0 && S > 0);
  SPINF_CHECK_ARG(D >= 64 && D <= 512 && D % 64 == 0 && beam > 0 && window >= 0 && Lp >= 0 && Tt >= 0 && q_pitch % 8 == 0 && out_pitch % 2 == 0);
  SPINF_CHECK_ARG((Lp == 0 || (kp && vp && pos_p)) && (Tt == 0 || (kt && vt && pos_t && own_t)) && G < 65536 && h < 65536);
  SPINF_CHECK_ARG(workspace_bytes >= spinf_x_attention_workspace_bytes(G, Q, H, D, Lp, Tt, S));
  SPINF_CHECK_ARG((k_new == nullptr) == (v_new == nullptr) && (!k_new || (kv_pitch >= h * D && kv_pitch % 8 == 0)));
  XAttnArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.q_pitch = q_pitch;
  a.kp = static_cast<const __nv_bfloat16*>(kp);
  a.vp = static_cast<const __nv_bfloat16*>(vp);
  a.pos_p = pos_p;
  a.kt = static_cast<const __nv_bfloat16*>(kt);
  a.vt = static_cast<const __nv_bfloat16*>(vt);
  a.pos_t = pos_t;
  a.own_t = own_t;
  a.gk = static_cast<__nv_bfloat16*>(gk);
  a.gv = static_cast<__nv_bfloat16*>(gv);
  a.k_new = static_cast<const __nv_bfloat16*>(k_new);
  a.v_new = static_cast<const __nv_bfloat16*>(v_new);
  a.kv_pitch = kv_pitch;
  a.qpos = qpos;
  a.step = step;
  a.G = static_cast<int>(G), a.Q = static_cast<int>(Q), a.H = static_cast<int>(H), a.h = static_cast<int>(h), a.D = static_cast<int>(D);
  a.Lp = static_cast<int>(Lp), a.Tt = static_cast<int>(Tt), a.S = static_cast<int>(S), a.beam = beam, a.window = window;
  a.scale = scale, a.softcap = softcap;
  a.Lp64 = pad64(Lp), a.Tt64 = pad64(Tt), a.S64 = pad64(S), a.pitch = a.Lp64 + a.Tt64 + a.S64;
  const int64_t rows = G * H * Q;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  ws += (256 - reinterpret_cast<uintptr_t>(ws) % 256) % 256;
  a.scores = reinterpret_cast<float*>(ws);
  a.probs = reinterpret_cast<__nv_bfloat16*>(ws + rows * a.pitch * 4);
  a.part = reinterpret_cast<float*>(ws + rows * a.pitch * 6);
  a.n_split = x_splits(Lp);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.out_pitch = out_pitch;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int smem_s = 2 * XT * (a.D + 8) * 2, smem_v = 2 * 2 * XT * (XT + 8) * 2;
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(x_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * XT * (512 + 8) * 2));
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  x_scores_kernel<<<dim3(a.Lp64 / XT + a.Tt64 / XT + (a.Q + 3) / 4, static_cast<unsigned>(h), static_cast<unsigned>(G)), 128, smem_s, st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  x_softmax_kernel<<<static_cast<unsigned>(rows), 128, 0, st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  x_values_kernel<<<dim3(static_cast<unsigned>(D / XT * (a.n_split + 1)), static_cast<unsigned>(h), static_cast<unsigned>(G)), 128, smem_v, st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  x_combine_kernel<<<static_cast<unsigned>((rows * D / 2 + 255) / 256), 256, 0, st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
