// Gated DeltaNet pieces of the hybrid stack's recurrent layers, for sm_100a.
//
// gdn_recurrent_kernel: the gated delta rule, token by token, over the segments of one plan call. One CTA = one (segment, value
// head); thread c owns column c of the state S [K=128, V=128] in 128 fp32 registers, so both reductions over K (S^T k and S^T q)
// are thread-local and the state never leaves the register file between tokens. A token's operands arrive through a ring of shared
// slots filled by cp.async three tokens ahead; k and q are converted to fp32 into a double-buffered tile one token ahead. A segment starts from h0[h0_idx] (the state its parent segment left) or
// zero and writes its final state to ht[ht_idx] where a child will read it: a branch forks the trunk's state by index, the trunk
// state itself is written once.
//     S *= exp(g);  v' = (v - S^T k) beta;  S += k (x) v';  o = S^T (q scale)
// gdn_prologue_kernel / gdn_epilogue_kernel: the bandwidth-bound steps around it (path convolution + SiLU, l2 norms, beta, g;
// gated RMS norm), one pass over the rows each.
#include <atomic>
#include "common.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int GK = 128;  // key head dim
static constexpr int GV = 128;  // value head dim

struct GdnArgs {
  const __nv_bfloat16* q;   // rows x (Hk*GK), row pitch q_pitch (elements); k likewise
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;   // rows x (Hv*GV), row pitch v_pitch
  const float* g;           // rows x Hv, row pitch g_pitch
  const __nv_bfloat16* beta;
  __nv_bfloat16* o;         // rows x Hv x GV contiguous
  int64_t q_pitch, v_pitch, g_pitch;
  int Hk, Hv;
  float scale;
  const int64_t* cu;        // [n_seg + 1]
  const int64_t* idx;       // optional: token t of the call is row idx[t]
  const float* h0;          // optional [*, Hv, GK, GV]
  const int64_t* h0_idx;
  float* ht;
  const int64_t* ht_idx;
  int64_t n_rows;           // rows of the tensors (index bound)
};

static constexpr int RING = 6;  // raw operand slots: tokens t .. t + 5 in flight (the copies of token t + 2 are waited for at step t)
struct __align__(16) RawSlot {
  uint4 kqv[3 * GK * 2 / 16];  // k, q, v rows of the head, bf16
  float g;
  uint32_t beta2;              // the aligned 4-byte word that holds the head's beta
  int64_t row;
};

__global__ void __launch_bounds__(128) gdn_recurrent_kernel(const GdnArgs a, int* __restrict__ status) {
  __shared__ __align__(16) float kq[2][2][GK];  // [buffer][k | q][GK]
  __shared__ RawSlot raw[RING];
  const int seg = blockIdx.x / a.Hv, hv = blockIdx.x % a.Hv;
  const int hk = hv / (a.Hv / a.Hk);
  const int c = threadIdx.x;
  const int64_t bos = a.cu[seg], eos = a.cu[seg + 1];
  float S[GK];
  const int64_t src = (a.h0 && a.h0_idx) ? a.h0_idx[seg] : -1;
  if (src >= 0) {
    const float* p = a.h0 + (src * a.Hv + hv) * GK * GV + c;
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) S[kk] = p[kk * GV];
  } else {
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) S[kk] = 0.f;
  }
  auto row_of = [&](int64_t t) -> int64_t {
    const int64_t r = a.idx ? a.idx[t] : t;
    if (r < 0 || r >= a.n_rows) {  // never index outside the tensors: record it and read row 0
      atomicCAS(status, 0, ST_BAD_INDEX);
      return 0;
    }
    return r;
  };
  // A token's operands (k, q, v rows of the head, g, beta) travel through a ring of RING raw slots filled by cp.async three tokens
  // ahead: a token step is shorter than a trip to HBM, so one token of prefetch left every step waiting for its loads. Threads
  // 0-15 copy k, 16-31 q, 32-47 v (16 bytes each), 48 copies g, 49 the 4-byte word that holds beta.
  auto issue = [&](int64_t t, int64_t r) {
    RawSlot& sl = raw[(t - bos) % RING];
    if (c < 50) {
      if (c < 48) {
        const int part = c >> 4, j = c & 15;
        const __nv_bfloat16* src = part == 0 ? a.k + r * a.q_pitch + hk * GK : (part == 1 ? a.q + r * a.q_pitch + hk * GK : a.v + r * a.v_pitch + hv * GV);
        cp_async16(reinterpret_cast<__nv_bfloat16*>(sl.kqv) + part * GK + j * 8, src + j * 8, 16);
      } else if (c == 48) {
        cp_async4(&sl.g, a.g + r * a.g_pitch + hv);
        sl.row = r;
      } else {
        cp_async4(&sl.beta2, reinterpret_cast<const uint32_t*>(a.beta + r * a.g_pitch + (hv & ~1)));
      }
    }
    cp_async_commit();
  };
  // k and q of token t, converted to fp32 (q scaled), into the fp32 buffer the inner loops read
  auto stash = [&](int64_t t, int buf) {
    if (c < 32) {
      const RawSlot& sl = raw[(t - bos) % RING];
      const uint4 pre = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(sl.kqv) + (c >> 4) * GK + (c & 15) * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pre);
      float* dst = kq[buf][c < 16 ? 0 : 1] + (c & 15) * 8;
      const float sc = c < 16 ? 1.f : a.scale;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        dst[2 * j] = f.x * sc;
        dst[2 * j + 1] = f.y * sc;
      }
    }
  };
  const int64_t n_tok = eos - bos;
  for (int64_t t = bos; t < bos + RING - 1; ++t) {
    if (t < eos) issue(t, c < 50 ? row_of(t) : 0);
    else cp_async_commit();  // keeps the group count uniform
  }
  // the row index of the token to be issued next is read one step ahead: the copy's address must not wait for it
  int64_t r_ahead = (c < 50 && bos + RING - 1 < eos) ? row_of(bos + RING - 1) : 0;
  if (n_tok > 0) {
    cp_async_wait<RING - 3>();  // tokens 0 and 1 have landed
    __syncthreads();
    stash(bos, 0);
  }
  __syncthreads();
  for (int64_t t = bos; t < eos; ++t) {
    const int buf = static_cast<int>((t - bos) & 1);
    const RawSlot& sl = raw[(t - bos) % RING];
    // token t + 1 landed before the barrier that ended the previous step; its fp32 buffer was last read one step ago
    if (t + 1 < eos) stash(t + 1, buf ^ 1);
    const float vt = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(sl.kqv)[2 * GK + c]);
    const float eg = expf(sl.g);
    const float bt = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&sl.beta2)[hv & 1]);
    const int64_t r = sl.row;
    // the slot of token t + RING - 1 is the one token t - 1 used: every thread passed the barrier that ended that step
    if (t + RING - 1 < eos) issue(t + RING - 1, r_ahead);
    else cp_async_commit();
    if (c < 50 && t + RING < eos) r_ahead = row_of(t + RING);
    const float4* kv4 = reinterpret_cast<const float4*>(kq[buf][0]);
    const float4* qv4 = reinterpret_cast<const float4*>(kq[buf][1]);
    // four independent partial sums per reduction: a single accumulator would serialise 128 dependent FMAs per token
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
    for (int i = 0; i < GK / 4; ++i) {
      const float4 kk = kv4[i];
      S[4 * i] *= eg, S[4 * i + 1] *= eg, S[4 * i + 2] *= eg, S[4 * i + 3] *= eg;
      d0 = fmaf(S[4 * i], kk.x, d0);
      d1 = fmaf(S[4 * i + 1], kk.y, d1);
      d2 = fmaf(S[4 * i + 2], kk.z, d2);
      d3 = fmaf(S[4 * i + 3], kk.w, d3);
    }
    const float vn = (vt - ((d0 + d1) + (d2 + d3))) * bt;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int i = 0; i < GK / 4; ++i) {
      const float4 kk = kv4[i];
      const float4 qq = qv4[i];
      S[4 * i] = fmaf(kk.x, vn, S[4 * i]);
      S[4 * i + 1] = fmaf(kk.y, vn, S[4 * i + 1]);
      S[4 * i + 2] = fmaf(kk.z, vn, S[4 * i + 2]);
      S[4 * i + 3] = fmaf(kk.w, vn, S[4 * i + 3]);
      o0 = fmaf(S[4 * i], qq.x, o0);
      o1 = fmaf(S[4 * i + 1], qq.y, o1);
      o2 = fmaf(S[4 * i + 2], qq.z, o2);
      o3 = fmaf(S[4 * i + 3], qq.w, o3);
    }
    const float od = (o0 + o1) + (o2 + o3);
    a.o[(r * a.Hv + hv) * GV + c] = __float2bfloat16_rn(od);
    cp_async_wait<RING - 3>();  // this thread's copies of token t + 2 have landed; the barrier covers the other threads'
    __syncthreads();
  }
  cp_async_wait<0>();
  const int64_t dst = (a.ht && a.ht_idx) ? a.ht_idx[seg] : -1;
  if (dst >= 0) {
    float* p = a.ht + (dst * a.Hv + hv) * GK * GV + c;
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) p[kk * GV] = S[kk];
  }
}

// ------------------------------------------------------------------------------------------------ prologue
// One CTA per token. y row = [q (Hk GK) | k (Hk GK) | v (Hv GV)] (= conv_dim channels) | z (Hv GV) | b (Hv) | a (Hv).
//   c[ch] = sum_j y[conv[t][j]][ch] * conv_w[ch][j]   (fp32; tap index >= n_rows = the zero row);  x = bf16(silu(c))
//   q, k: x * rsqrt(sum_head x^2 + 1e-6) per head -> bf16;  v: x
//   beta = bf16(sigmoid(b));  g = -exp(A_log) * softplus(a + dt_bias)   (fp32)
struct GdnProArgs {
  const __nv_bfloat16* y;
  int64_t y_pitch, n_rows;
  const int64_t* conv;            // [T, 4]
  const __nv_bfloat16* conv_w;    // [conv_dim, 4]
  const float* A_log;             // [Hv]
  const float* dt_bias;           // [Hv]
  __nv_bfloat16 *q, *k, *v;       // [T, Hk, GK], [T, Hk, GK], [T, Hv, GV]
  float* g;                       // [T, Hv]
  __nv_bfloat16* beta;            // [T, Hv]
  int Hk, Hv;
};

__device__ __forceinline__ float silu_f(float x) { return silu_f32(x); }

__global__ void __launch_bounds__(256) gdn_prologue_kernel(const GdnProArgs a) {
  extern __shared__ float xs[];  // conv+silu of the q and k channels (as bf16-rounded floats): 2 Hk GK floats
  const int64_t t = blockIdx.x;
  const int kd = a.Hk * GK, vd = a.Hv * GV, conv_dim = 2 * kd + vd;
  int64_t taps[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) taps[j] = a.conv[t * 4 + j];
  for (int ch8 = threadIdx.x; ch8 < conv_dim / 8; ch8 += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // conv_w rows of these 8 channels: 32 consecutive bf16
    float w[8][4];
    {
      const uint4* wp = reinterpret_cast<const uint4*>(a.conv_w + static_cast<int64_t>(ch8) * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 u = wp[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          const int e = i * 8 + 2 * j;  // element index inside the 8 x 4 block
          w[e / 4][e % 4] = f.x;
          w[(e + 1) / 4][(e + 1) % 4] = f.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (taps[j] >= 0 && taps[j] < a.n_rows) {
        const uint4 u = *reinterpret_cast<const uint4*>(a.y + taps[j] * a.y_pitch + ch8 * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += f.x * w[2 * i][j];
          acc[2 * i + 1] += f.y * w[2 * i + 1][j];
        }
      }
    }
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(silu_f(acc[i])));
    const int ch = ch8 * 8;
    if (ch < 2 * kd) {
#pragma unroll
      for (int i = 0; i < 8; ++i) xs[ch + i] = x[i];
    } else {
      uint4 o;
      o.x = pack_bf16x2(x[0], x[1]), o.y = pack_bf16x2(x[2], x[3]), o.z = pack_bf16x2(x[4], x[5]), o.w = pack_bf16x2(x[6], x[7]);
      *reinterpret_cast<uint4*>(a.v + t * vd + (ch - 2 * kd)) = o;
    }
  }
  __syncthreads();
  // l2 norm per head of q and k: one warp per head (2 Hk heads), 4 elements per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int hd = warp; hd < 2 * a.Hk; hd += nwarps) {
    const float* src = xs + hd * GK + lane * 4;
    const float x0 = src[0], x1 = src[1], x2 = src[2], x3 = src[3];
    float ss = x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3;
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss + 1e-6f);
    __nv_bfloat16* dst = (hd < a.Hk ? a.q + t * kd + hd * GK : a.k + t * kd + (hd - a.Hk) * GK) + lane * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(x0 * inv, x1 * inv), pack_bf16x2(x2 * inv, x3 * inv));
  }
  if (threadIdx.x < a.Hv) {
    const int hv = threadIdx.x;
    const __nv_bfloat16* row = a.y + t * a.y_pitch + conv_dim + vd;
    const float b = __bfloat162float(row[hv]), av = __bfloat162float(row[a.Hv + hv]);
    a.beta[t * a.Hv + hv] = __float2bfloat16_rn(1.f / (1.f + expf(-b)));
    const float sp_in = av + a.dt_bias[hv];
    const float sp = sp_in > 20.f ? sp_in : log1pf(expf(sp_in));  // softplus with torch's threshold
    a.g[t * a.Hv + hv] = -expf(a.A_log[hv]) * sp;
  }
}

// ------------------------------------------------------------------------------------------------ epilogue
// One warp per (token, value head): of = o * rsqrt(mean(o^2) + eps);  out = bf16( float(bf16(norm_w * bf16(of))) * silu(z) )
__global__ void __launch_bounds__(256) gdn_epilogue_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                                           int64_t z_pitch, const __nv_bfloat16* __restrict__ norm_w, float eps,
                                                           int64_t T, int Hv, __nv_bfloat16* __restrict__ out) {
  const int64_t gw = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (gw >= T * Hv) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = gw / Hv;
  const int hv = static_cast<int>(gw % Hv);
  const uint2 uo = *reinterpret_cast<const uint2*>(o + (t * Hv + hv) * GV + lane * 4);
  const uint2 uz = *reinterpret_cast<const uint2*>(z + t * z_pitch + hv * GV + lane * 4);
  const uint2 uw = *reinterpret_cast<const uint2*>(norm_w + lane * 4);
  float x[4], zz[4], w[4];
  {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&uo);
    const float2 a0 = __bfloat1622float2(h[0]), a1 = __bfloat1622float2(h[1]);
    x[0] = a0.x, x[1] = a0.y, x[2] = a1.x, x[3] = a1.y;
    h = reinterpret_cast<const __nv_bfloat162*>(&uz);
    const float2 b0 = __bfloat1622float2(h[0]), b1 = __bfloat1622float2(h[1]);
    zz[0] = b0.x, zz[1] = b0.y, zz[2] = b1.x, zz[3] = b1.y;
    h = reinterpret_cast<const __nv_bfloat162*>(&uw);
    const float2 c0 = __bfloat1622float2(h[0]), c1 = __bfloat1622float2(h[1]);
    w[0] = c0.x, w[1] = c0.y, w[2] = c1.x, w[3] = c1.y;
  }
  float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float inv = rsqrtf(ss / GV + eps);
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float of = __bfloat162float(__float2bfloat16_rn(x[i] * inv));
    const float nw = __bfloat162float(__float2bfloat16_rn(w[i] * of));
    y[i] = nw * silu_f(zz[i]);
  }
  *reinterpret_cast<uint2*>(out + (t * Hv + hv) * GV + lane * 4) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                                   int64_t n_rows, int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv,
                                   int32_t K, int32_t V, float scale, const int64_t* cu, int64_t n_seg, const int64_t* idx,
                                   const float* h0, const int64_t* h0_idx, float* ht, const int64_t* ht_idx, void* stream) {
  if (n_seg == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(q && k && v && g && beta && o && cu && n_rows >= 0 && n_seg >= 0 && Hk > 0 && Hv > 0 && Hv % Hk == 0);
  SPINF_CHECK_ARG(K == GK && V == GV);  // the kernel is written for 128 x 128 states, as the reference's is for K = 128
  SPINF_CHECK_ARG(q_pitch >= static_cast<int64_t>(Hk) * GK && q_pitch % 8 == 0 && v_pitch >= static_cast<int64_t>(Hv) * GV && g_pitch >= Hv);
  SPINF_CHECK_ARG((h0 == nullptr) == (h0_idx == nullptr) && (ht == nullptr) == (ht_idx == nullptr));
  SPINF_CHECK_ARG(n_seg * Hv < (1ll << 31));
  // rows are copied in 16-byte pieces, beta as the aligned 4-byte word around it
  SPINF_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0);
  SPINF_CHECK_ARG(v_pitch % 8 == 0 && g_pitch % 2 == 0 && Hv % 2 == 0 && (reinterpret_cast<uintptr_t>(beta) & 3) == 0);
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  GdnArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q), a.k = static_cast<const __nv_bfloat16*>(k), a.v = static_cast<const __nv_bfloat16*>(v);
  a.g = g, a.beta = static_cast<const __nv_bfloat16*>(beta), a.o = static_cast<__nv_bfloat16*>(o);
  a.q_pitch = q_pitch, a.v_pitch = v_pitch, a.g_pitch = g_pitch, a.Hk = Hk, a.Hv = Hv, a.scale = scale;
  a.cu = cu, a.idx = idx, a.h0 = h0, a.h0_idx = h0_idx, a.ht = ht, a.ht_idx = ht_idx, a.n_rows = n_rows;
  gdn_recurrent_kernel<<<static_cast<unsigned>(n_seg * Hv), 128, 0, static_cast<cudaStream_t>(stream)>>>(a, status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_gdn_prologue(const void* y, int64_t y_pitch, int64_t n_rows, int64_t T, const int64_t* conv, const void* conv_w,
                                  const float* A_log, const float* dt_bias, int32_t Hk, int32_t Hv, int32_t K, int32_t V, void* q,
                                  void* k, void* v, float* g, void* beta, void* stream) {
  if (T == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(y && conv && conv_w && A_log && dt_bias && q && k && v && g && beta && T >= 0 && n_rows >= T);
  SPINF_CHECK_ARG(K == GK && V == GV && Hk > 0 && Hv > 0 && Hv <= 256 && Hk <= 96 && T < (1ll << 31));
  SPINF_CHECK_ARG(y_pitch >= 2ll * Hk * GK + 2ll * Hv * GV + 2 * Hv && y_pitch % 8 == 0);
  GdnProArgs a;
  a.y = static_cast<const __nv_bfloat16*>(y), a.y_pitch = y_pitch, a.n_rows = n_rows, a.conv = conv;
  a.conv_w = static_cast<const __nv_bfloat16*>(conv_w), a.A_log = A_log, a.dt_bias = dt_bias;
  a.q = static_cast<__nv_bfloat16*>(q), a.k = static_cast<__nv_bfloat16*>(k), a.v = static_cast<__nv_bfloat16*>(v);
  a.g = g, a.beta = static_cast<__nv_bfloat16*>(beta), a.Hk = Hk, a.Hv = Hv;
  const size_t smem = static_cast<size_t>(2) * Hk * GK * sizeof(float);
  static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice from two threads is harmless
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    SPINF_CUDA_OK(cudaFuncSetAttribute(gdn_prologue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 96 * GK * 4));
    attr_set[dev].store(true, std::memory_order_release);
  }
  gdn_prologue_kernel<<<static_cast<unsigned>(T), 256, smem, static_cast<cudaStream_t>(stream)>>>(a);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_gdn_epilogue(const void* o, const void* z, int64_t z_pitch, const void* norm_w, float eps, int64_t T, int32_t Hv,
                                  int32_t V, void* out, void* stream) {
  if (T == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(o && z && norm_w && out && T >= 0 && Hv > 0 && V == GV && z_pitch >= static_cast<int64_t>(Hv) * GV && z_pitch % 4 == 0);
  const int64_t warps = T * Hv;
  gdn_epilogue_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(z), z_pitch, static_cast<const __nv_bfloat16*>(norm_w), eps,
      T, Hv, static_cast<__nv_bfloat16*>(out));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
