// Attention of the extraction decoder's steps (spinf_serve/decode.py:71-104, `_x_attention`): a few query rows per group (slots x
// beams, one new token each) attend to three key ranges: the group's prefix (stored once per group), the templates (a slot sees
// its own prompt's template only) and the tokens the slot's own beam has generated so far. Token-major layouts throughout
// ([.., tokens, kv heads, dim]); all head dimensions that are multiples of 64 up to 512.
//
// The reference's rounding points are kept, so the product can be checked element by element: scores are bf16 products with fp32
// accumulation rounded to bf16, then scaling / soft cap / mask / softmax in fp32 over the three ranges together, the
// probabilities rounded to bf16, each range's value product rounded to bf16 and the three added in fp32. That forces the softmax
// to be complete before any value product starts, hence three launches:
//   x_scores  (key tile of 64 | the generated range) x kv head x group : S = Q K^T on mma.sync, masked scores -> fp32 workspace
//   x_softmax one row per CTA                                          : probabilities -> bf16 workspace
//   x_values  64 output dims x kv head x group                         : P V per range on mma.sync, generated range on FMA
// Each range is padded to a multiple of 64 columns in the workspace so every tile row starts 16-byte aligned. A decoding step is
// bound by reading the prefix K / V once per layer; these kernels read it once per (kv head, 64-dim slice) from L2.
#include "gdn_mma.cuh"
#include "host_util.h"

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
  const __nv_bfloat16 *gk, *gv;
  const int32_t* qpos;
  const int32_t* step;
  int G, Q, H, h, D, Lp, Tt, S, beam, window;
  float scale, softcap;
  int Lp64, Tt64, S64, pitch;  // padded range widths and the workspace row pitch (their sum)
  float* scores;
  __nv_bfloat16* probs;
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
    for (int rr = 0; rr < r; ++rr) {
      uint4 qv[2] = {};
      const __nv_bfloat16* const qr = x_q_row(a, g, hk, r, q * r + rr);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (lane + j * 32 < vec) qv[j] = *reinterpret_cast<const uint4*>(qr + (lane + j * 32) * 8);
      float* const dst = a.scores + x_ws_row(a, g, hk, r, q * r + rr) + a.Lp64 + a.Tt64;
      const __nv_bfloat16* const kbase = a.gk + (((static_cast<int64_t>(g) * a.Q + q) * a.S) * a.h + hk) * a.D;
      for (int s0 = 0; s0 < a.S64; s0 += 4) {
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
          if (lane == u) dst[s0 + u] = s0 + u < n_live ? x_finish_score(acc, a.scale, a.softcap) : X_NINF;
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
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = n * 8 + tq * 2 + e, key = k0 + c;
            bool vis = key < L;
            if (vis) {
              const int kp = kpos[key];
              vis = prefix ? kp >= 0 : kown[key] == mine;
              if (a.window > 0) vis = vis && (qp - kp) < a.window;
            }
            dst[c] = vis ? x_finish_score(acc[n][half * 2 + e], a.scale, a.softcap) : X_NINF;
          }
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

// dynamic shared memory, two stages of: [XT][XT + 8] probabilities, [XT][XT + 8] values (keys x 64 dims of this CTA)
__global__ void __launch_bounds__(128) x_values_kernel(const XAttnArgs a) {
  extern __shared__ __align__(16) uint8_t xv_raw[];
  constexpr int ld = XT + 8;
  constexpr int STAGE = 2 * XT * ld;  // elements
  __nv_bfloat16* const sm = reinterpret_cast<__nv_bfloat16*>(xv_raw);
  const int d0 = blockIdx.x * XT, hk = blockIdx.y, g = blockIdx.z;
  const int r = a.H / a.h, R = a.Q * r;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int step = *a.step;
  const int np = a.Lp64 / XT, n_tiles = np + a.Tt64 / XT;
  for (int m0 = 0; m0 < R; m0 += XT) {
    auto stage = [&](int tile, int buf) {
      const bool pre = tile < np;
      const int L = pre ? a.Lp : a.Tt, k0 = (pre ? tile : tile - np) * XT, col0 = pre ? 0 : a.Lp64;
      const __nv_bfloat16* const vbase = pre ? a.vp : a.vt;
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
    float total[8][4] = {};
    float acc[8][4] = {};
    __syncthreads();  // the previous pass has read both stages
    if (n_tiles > 0) stage(0, 0);
    cp_async_commit();
    for (int tile = 0; tile < n_tiles; ++tile) {
      if (tile + 1 < n_tiles) stage(tile + 1, (tile + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* const ps = sm + (tile & 1) * STAGE;
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
      if (tile == np - 1 || tile == n_tiles - 1) {  // a range is complete: its product is rounded to bf16 on its own
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            total[n][e] += x_round_bf16(acc[n][e]);
            acc[n][e] = 0.f;
          }
      }
      __syncthreads();  // this stage is free for the tile after the next
    }
    // the generated range: a row's own slot's tokens 0..step, on the FMA pipe for exactly the elements this thread holds
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + warp * 16 + gq + half * 8;
      if (m >= R) continue;
      const int q = m / r;
      const __nv_bfloat16* const pr = a.probs + x_ws_row(a, g, hk, r, m) + a.Lp64 + a.Tt64;
      const __nv_bfloat16* const vr = a.gv + ((static_cast<int64_t>(g) * a.Q + q) * a.S * a.h + hk) * a.D + d0 + tq * 2;
      float acc[8][2] = {};
      const int n_live = min(step + 1, a.S);
      for (int s = 0; s < n_live; ++s) {
        const float p = __bfloat162float(pr[s]);
        const __nv_bfloat16* const v = vr + static_cast<int64_t>(s) * a.h * a.D;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(v + n * 8));
          acc[n][0] = fmaf(p, f.x, acc[n][0]);
          acc[n][1] = fmaf(p, f.y, acc[n][1]);
        }
      }
      __nv_bfloat16* const dst = a.out + (static_cast<int64_t>(g) * a.Q + q) * a.out_pitch + static_cast<int64_t>(hk * r + m % r) * a.D + d0 + tq * 2;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float x = total[n][half * 2] + x_round_bf16(acc[n][0]);
        const float y = total[n][half * 2 + 1] + x_round_bf16(acc[n][1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(x, y);
      }
    }
  }
}

static int pad64(int64_t n) { return static_cast<int>((n + XT - 1) / XT * XT); }

}  // namespace spinf

using namespace spinf;

// bytes of the workspace spinf_x_attention needs: fp32 scores and bf16 probabilities, one row per (group, query head, slot), each
// of the three key ranges padded to a multiple of 64 columns
extern "C" int64_t spinf_x_attention_workspace_bytes(int64_t G, int64_t Q, int64_t H, int64_t Lp, int64_t Tt, int64_t S) {
  if (G <= 0 || Q <= 0 || H <= 0 || Lp < 0 || Tt < 0 || S <= 0) return 0;
  const int64_t pitch = pad64(Lp) + pad64(Tt) + pad64(S);
  return G * H * Q * pitch * 6 + 256;
}

extern "C" int spinf_x_attention(const void* q, int64_t q_pitch, const void* kp, const void* vp, const int32_t* pos_p, int64_t Lp,
                                 const void* kt, const void* vt, const int32_t* pos_t, const int32_t* own_t, int64_t Tt, const void* gk,
                                 const void* gv, int64_t S, const int32_t* qpos, const int32_t* step, int64_t G, int64_t Q, int64_t H,
                                 int64_t h, int64_t D, int32_t beam, int32_t window, float scale, float softcap, void* out,
                                 int64_t out_pitch, void* workspace, int64_t workspace_bytes, void* stream) {
  if (G == 0 || Q == 0) return 0;
  SPINF_CHECK_ARG(q && gk && gv && qpos && step && out && workspace && G > 0 && Q > 0 && H > 0 && h > 0 && H % h == 0 && S > 0);
  SPINF_CHECK_ARG(D >= 64 && D <= 512 && D % 64 == 0 && beam > 0 && window >= 0 && Lp >= 0 && Tt >= 0 && q_pitch % 8 == 0 && out_pitch % 2 == 0);
  SPINF_CHECK_ARG((Lp == 0 || (kp && vp && pos_p)) && (Tt == 0 || (kt && vt && pos_t && own_t)) && G < 65536 && h < 65536);
  SPINF_CHECK_ARG(workspace_bytes >= spinf_x_attention_workspace_bytes(G, Q, H, Lp, Tt, S));
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
  a.gk = static_cast<const __nv_bfloat16*>(gk);
  a.gv = static_cast<const __nv_bfloat16*>(gv);
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
  x_values_kernel<<<dim3(static_cast<unsigned>(D / XT), static_cast<unsigned>(h), static_cast<unsigned>(G)), 128, smem_v, st>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
