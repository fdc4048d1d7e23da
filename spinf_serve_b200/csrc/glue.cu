// Bandwidth-bound layer glue of the packed forward, fused so each activation row crosses HBM once per step:
//   fused_norm      [RMSNorm] -> [+ residual] -> [RMSNorm] -> bf16 and/or per-row fp8 quantisation (feeds the next fp8 GEMM)
//   qkv_norm_rope   per-head RMSNorm of q / k (with weight) and v (without), rotary embedding of q / k, in place
//   glu_quant       act(gate) * up -> per-row fp8 quantisation (GeGLU for the Gemma stack, SwiGLU for the Qwen stack)
//   embed_scale     embedding gather times the (bf16) embedding scale
//   rope_table      cos / sin of pos * inv_freq, rounded to bf16 as the model code does before applying them
// Rounding points follow the module code the reference runs (transformers' Gemma 4 text model, called from
// spinf_serve/models/gemma4.py:134-143,407-415): every module output is bf16, norms compute in fp32 and round once, the rotary
// product is three bf16 roundings (x*cos, rot(x)*sin, their sum), residual adds are bf16 + bf16 -> bf16.
#include "common.cuh"
#include "host_util.h"

namespace spinf {

static constexpr int NORM_THREADS = 256;
static constexpr int NORM_MAX_VEC = 4;  // row cache: up to 256 * 4 * 8 = 8192 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
// One-barrier forms: each reduction of a row has its own array, so a value is only overwritten after every thread has passed a
// later barrier (the next reduction's) and so has finished reading it.
__device__ __forceinline__ float block_sum1(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max1(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int i = 1; i < NORM_THREADS / 32; ++i) t = fmaxf(t, red[i]);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < nw; ++i) t = fmaxf(t, red[i]);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
// x^-1/2 to within an ulp: hardware estimate plus one Newton step (the model code's pow(x, -0.5) costs ~10x the instructions)
__device__ __forceinline__ float inv_sqrt(float x) {
  const float y = rsqrtf(x);
  return y * fmaf(-0.5f * x * y, y, 1.5f);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint2 quant8(const float (&f)[8], const DivBy& div) {
  uint32_t o[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float q0 = fminf(fmaxf(div_by(div, f[4 * j]), -448.f), 448.f), q1 = fminf(fmaxf(div_by(div, f[4 * j + 1]), -448.f), 448.f);
    const float q2 = fminf(fmaxf(div_by(div, f[4 * j + 2]), -448.f), 448.f), q3 = fminf(fmaxf(div_by(div, f[4 * j + 3]), -448.f), 448.f);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
    o[j] = lo | (hi << 16);
  }
  return make_uint2(o[0], o[1]);
}

// RMSNorm as the model computes it: x * pow(mean(x^2) + eps, -0.5), times the weight, all in fp32, rounded once to bf16.
// plus1: the weight enters as (1 + w) (Qwen's RMSNorm, spinf_serve/models/qwen35/qwen.py:502-510).
struct FusedNormArgs {
  const __nv_bfloat16* y;         // [*, hidden] input rows
  const int64_t* rows;            // optional: output row r reads input row rows[r]
  const __nv_bfloat16* w1;        // optional first norm weight
  const __nv_bfloat16* residual;  // optional [n_out, hidden], added after the first norm
  const __nv_bfloat16* w2;        // optional second norm weight
  __nv_bfloat16* out_h;           // optional: the value after the residual add (the new residual stream)
  __nv_bfloat16* out_norm;        // optional: the second norm's output in bf16
  uint8_t* out_x8;                // optional: its per-row fp8 quantisation
  float* out_xs;
  int hidden;
  float eps;
  int plus1;
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

// One CTA per row. Both streamed loads of the row (input, residual) are issued before the first reduction, so the row costs one
// DRAM round trip instead of one per stage; the norm weights are cache hits and are loaded where they are used. The row stays in
// registers as packed bf16 pairs: a norm's output leaves the pack conversion already rounded, the residual add is the bf16x2
// add (the exact sum rounded once, as the bf16 tensor add rounds), and the running |max| is a bf16x2 max.
template <bool PLUS1>  // the weight enters as (1 + w)
__device__ __forceinline__ uint32_t scale_pair(uint32_t x, float inv, uint32_t w) {
  const float w0 = PLUS1 ? 1.f + bf2_lo(w) : bf2_lo(w), w1 = PLUS1 ? 1.f + bf2_hi(w) : bf2_hi(w);
  return pack_bf16x2(bf2_lo(x) * inv * w0, bf2_hi(x) * inv * w1);
}
__device__ __forceinline__ float sumsq4(const uint4& u, float ss) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) ss = fmaf(bf2_hi(w[j]), bf2_hi(w[j]), fmaf(bf2_lo(w[j]), bf2_lo(w[j]), ss));
  return ss;
}
// x / s for the eight values of a packed vector, converted to e4m3 with saturation (|x / s| exceeds 448 by rounding at most)
__device__ __forceinline__ uint2 quant8_packed(const uint4& u, const DivBy& div) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = __nv_cvt_float2_to_fp8x2(make_float2(div_by(div, bf2_lo(w[j])), div_by(div, bf2_hi(w[j]))), __NV_SATFINITE, __NV_E4M3);
  return make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
}

template <int NVEC, bool PLUS1>
__global__ void __launch_bounds__(NORM_THREADS, NVEC <= 2 ? 4 : 2) fused_norm_kernel(const FusedNormArgs a, int64_t n_out) {
  __shared__ float red[3][NORM_THREADS / 32];  // one array per reduction of a row
  const int nvec = a.hidden / 8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // a CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; the streamed loads of the next row are issued before the current
  // row's reductions, so every CTA keeps a row in flight while it works on another
  uint4 ny[NVEC], nr[NVEC];
  auto load_row = [&](int64_t r) {
    const int64_t rin = a.rows ? a.rows[r] : r;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      const bool on = v < nvec;
      ny[i] = on ? *reinterpret_cast<const uint4*>(a.y + rin * a.hidden + v * 8) : zero;
      nr[i] = on && a.residual ? *reinterpret_cast<const uint4*>(a.residual + r * a.hidden + v * 8) : zero;
    }
  };
  if (static_cast<int64_t>(blockIdx.x) < n_out) load_row(blockIdx.x);
  // with a single reduction per row nothing separates a row's reads of its array from the next row's writes
  const bool lone_reduction = (a.w1 != nullptr) + (a.w2 != nullptr) + (a.out_x8 != nullptr) < 2;
  for (int64_t r = blockIdx.x; r < n_out; r += gridDim.x) {
    if (lone_reduction) __syncthreads();
    uint4 cur[NVEC], rr[NVEC];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) cur[i] = ny[i], rr[i] = nr[i];
    if (r + gridDim.x < n_out) load_row(r + gridDim.x);
    if (a.w1) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NVEC; ++i) ss = sumsq4(cur[i], ss);
      const float inv = inv_sqrt(block_sum1(ss, red[0]) / a.hidden + a.eps);
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int v = threadIdx.x + i * NORM_THREADS;
        const uint4 w = v < nvec ? *reinterpret_cast<const uint4*>(a.w1 + v * 8) : zero;
        cur[i] = make_uint4(scale_pair<PLUS1>(cur[i].x, inv, w.x), scale_pair<PLUS1>(cur[i].y, inv, w.y),
                            scale_pair<PLUS1>(cur[i].z, inv, w.z), scale_pair<PLUS1>(cur[i].w, inv, w.w));
      }
    }
    if (a.residual) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i)
        cur[i] = make_uint4(bf2_add(cur[i].x, rr[i].x), bf2_add(cur[i].y, rr[i].y), bf2_add(cur[i].z, rr[i].z), bf2_add(cur[i].w, rr[i].w));
    }
    if (a.out_h) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int v = threadIdx.x + i * NORM_THREADS;
        if (v < nvec) *reinterpret_cast<uint4*>(a.out_h + r * a.hidden + v * 8) = cur[i];
      }
    }
    if (!a.w2) continue;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) ss = sumsq4(cur[i], ss);  // (lanes past the row may hold a norm of zeros times 1 + w: keep them out)
    }
    const float inv2 = inv_sqrt(block_sum1(ss, red[1]) / a.hidden + a.eps);
    uint32_t amax2 = 0u;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        const uint4 w = *reinterpret_cast<const uint4*>(a.w2 + v * 8);
        cur[i] = make_uint4(scale_pair<PLUS1>(cur[i].x, inv2, w.x), scale_pair<PLUS1>(cur[i].y, inv2, w.y),
                            scale_pair<PLUS1>(cur[i].z, inv2, w.z), scale_pair<PLUS1>(cur[i].w, inv2, w.w));
        amax2 = bf2_max(bf2_max(amax2, cur[i].x & 0x7fff7fffu),
                        bf2_max(cur[i].y & 0x7fff7fffu, bf2_max(cur[i].z & 0x7fff7fffu, cur[i].w & 0x7fff7fffu)));
        if (a.out_norm) *reinterpret_cast<uint4*>(a.out_norm + r * a.hidden + v * 8) = cur[i];
      }
    }
    if (!a.out_x8) continue;
    const float amax = fmaxf(bf2_lo(amax2), bf2_hi(amax2));
    const float s = __fdiv_rn(fmaxf(block_max1(amax, red[2]), 1e-12f), 448.f);
    if (threadIdx.x == 0) a.out_xs[r] = s;
    const DivBy div = make_div_by(s);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) *reinterpret_cast<uint2*>(a.out_x8 + r * a.hidden + v * 8) = quant8_packed(cur[i], div);
    }
  }
}

// ------------------------------------------------------------------------------------------------ q/k/v head norms + rotary
// One warp per (token, head) of the fused projection output [n, (H + 2 Hkv) * D]; lane l holds elements [l*V, l*V + V), V = D/32,
// whose rotary partners (offset D/2) sit in lane l ^ 16.
template <int V>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&f)[V]) {
  if constexpr (V == 8) {
    load8(p, f);
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
  }
}
template <int V>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&f)[V]) {
  if constexpr (V == 8) {
    store8(p, f);
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
  }
}

// One warp per two consecutive (token, head) items: both heads' rows are loaded before either is reduced (twice the bytes in
// flight per warp); norm weights and the rotary table are cache hits and are loaded where they are used.
template <int D>
__global__ void __launch_bounds__(256) qkv_norm_rope_kernel(__nv_bfloat16* __restrict__ qkv, int64_t pitch, int64_t n, int H, int Hkv,
                                                            const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                                                            const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                                                            float eps, int plus1, int norm_v, int rot_dim, int q_stride, int k_off,
                                                            __nv_bfloat16* __restrict__ q_out) {
  constexpr int V = D / 32;
  const int heads = H + 2 * Hkv;
  const int64_t total = n * heads;
  const int64_t first = ((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * 2;
  if (first >= total) return;
  const int lane = threadIdx.x & 31;
  // rotate_half over the first R = rot_dim dimensions: out[i] = x[i] cos[i] - x[i + R/2] sin[i]  (i < R/2),
  //                                                    out[i] = x[i] cos[i] + x[i - R/2] sin[i]  (R/2 <= i < R),
  // cos / sin repeat with period R/2; dimensions >= R pass through. R/2 is a multiple of V, so a lane's partners sit in
  // one other lane, `hl` lanes away, and its V cos / sin values are contiguous in the table.
  const int half = rot_dim / 2;
  const int hl = half / V;
  const bool low = lane < hl;
  float x[2][V];
  const __nv_bfloat16* src[2];
  __nv_bfloat16* dst[2];
  int hd[2];
  int64_t tok[2];
  bool live[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int64_t item = first + u;
    live[u] = item < total;
    tok[u] = live[u] ? item / heads : 0;
    hd[u] = live[u] ? static_cast<int>(item % heads) : 0;
    if (hd[u] >= H + Hkv && !norm_v) live[u] = false;  // value heads without a norm are left untouched
    // query head hd sits at column hd * q_stride (q_stride = D for a dense q block, 2 D when each head is followed by its
    // gate); key / value heads follow from column k_off; a query head may be written to a separate dense tensor
    src[u] = qkv + tok[u] * pitch + (hd[u] < H ? static_cast<int64_t>(hd[u]) * q_stride : k_off + static_cast<int64_t>(hd[u] - H) * D) + lane * V;
    dst[u] = (hd[u] < H && q_out) ? q_out + (tok[u] * H + hd[u]) * D + lane * V : const_cast<__nv_bfloat16*>(src[u]);
    if (live[u]) load_vec<V>(src[u], x[u]);
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (!live[u]) continue;  // uniform across the warp
    const bool is_v = hd[u] >= H + Hkv;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) ss += x[u][j] * x[u][j];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = inv_sqrt(ss / D + eps);
    if (is_v) {
#pragma unroll
      for (int j = 0; j < V; ++j) x[u][j] = round_bf16(x[u][j] * inv);
    } else {
      float w[V];
      load_vec<V>((hd[u] < H ? wq : wk) + lane * V, w);
#pragma unroll
      for (int j = 0; j < V; ++j) x[u][j] = round_bf16(x[u][j] * inv * (plus1 ? 1.f + w[j] : w[j]));
      const bool rotates = lane < 2 * hl;
      const int partner_lane = !rotates ? lane : (low ? lane + hl : lane - hl);
      float c[V], sn[V];
      if (rotates) {
        const int f0 = (low ? lane : lane - hl) * V;
        load_vec<V>(cos_t + tok[u] * half + f0, c);
        load_vec<V>(sin_t + tok[u] * half + f0, sn);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float partner = __shfl_sync(0xffffffffu, x[u][j], partner_lane);
        if (rotates) x[u][j] = round_bf16(round_bf16(x[u][j] * c[j]) + round_bf16((low ? -partner : partner) * sn[j]));
      }
    }
    store_vec<V>(dst[u], x[u]);
  }
}

// ------------------------------------------------------------------------------------------------ gated activation + quantiser
enum : int { ACT_GELU_TANH = 0, ACT_SILU = 1 };
template <int ACT>
__device__ __forceinline__ float act_fn(float x) {
  if (ACT == ACT_GELU_TANH) return gelu_tanh_f32(x);
  return silu_f32(x);
}

// gu [n, 2F]: gate = columns [0, F), up = columns [F, 2F). y = bf16(bf16(act(gate)) * up); then the per-row fp8 quantisation of y
// (out_x8 / out_xs), or y itself in bf16 (out_y) when the next linear takes bf16 activations.
template <int ACT>
__global__ void __launch_bounds__(512) glu_quant_kernel(const __nv_bfloat16* __restrict__ gu, int F, uint8_t* __restrict__ out_x8,
                                                        float* __restrict__ out_xs, __nv_bfloat16* __restrict__ out_y) {
  __shared__ float red[16];
  const int64_t r = blockIdx.x;
  const __nv_bfloat16* g = gu + r * 2 * F;
  const __nv_bfloat16* u = g + F;
  const int nvec = F / 8;
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float a[8], b[8];
    load8(g + v * 8, a);
    load8(u + v * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[j] = round_bf16(round_bf16(act_fn<ACT>(a[j])) * b[j]);
      amax = fmaxf(amax, fabsf(a[j]));
    }
    if (out_y) store8(out_y + r * F + v * 8, a);
  }
  if (!out_x8) return;
  const float s = __fdiv_rn(fmaxf(block_max(amax, red), 1e-12f), 448.f);
  if (threadIdx.x == 0) out_xs[r] = s;
  const DivBy div = make_div_by(s);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float a[8], b[8];
    load8(g + v * 8, a);
    load8(u + v * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = round_bf16(round_bf16(act_fn<ACT>(a[j])) * b[j]);
    *reinterpret_cast<uint2*>(out_x8 + r * F + v * 8) = quant8(a, div);
  }
}

// ------------------------------------------------------------------------------------------------ embedding, rotary table
__global__ void embed_scale_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ emb, int hidden, int64_t vocab,
                                   float scale, __nv_bfloat16* __restrict__ out) {
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // never read outside the table
  const __nv_bfloat16* src = emb + id * hidden;
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    float x[8];
    load8(src + v * 8, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= scale;
    store8(out + t * hidden + v * 8, x);
  }
}

// cos / sin of pos[t] * inv_freq[f] in fp32, rounded to bf16 (the model casts them to the activations' dtype before use)
__global__ void rope_table_kernel(const int32_t* __restrict__ pos, int64_t n, int half, const float* __restrict__ inv_freq,
                                  __nv_bfloat16* __restrict__ cos_t, __nv_bfloat16* __restrict__ sin_t) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n * half) return;
  const int64_t t = i / half;
  const int f = static_cast<int>(i % half);
  const float ang = static_cast<float>(pos[t]) * inv_freq[f];
  cos_t[i] = __float2bfloat16_rn(cosf(ang));
  sin_t[i] = __float2bfloat16_rn(sinf(ang));
}

// ------------------------------------------------------------------------------------------------ self-test of the bounded wait
// One CTA waits on a barrier that nothing will ever complete, with the limit the caller gives: the wait gives up, records
// ST_TIMEOUT_OTHER in the device status word and the kernel returns normally, which is what every pipeline role of the library
// does when a peer stops. Lets a test see the error path end to end without a fault and without a hang.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(uint64_t limit_ns, int* __restrict__ status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const WaitCtx wc{&abort_flag, status};
    mbar_wait(wc, &bar, 0u, ST_TIMEOUT_OTHER, limit_ns);
  }
}

}  // namespace spinf

using namespace spinf;

extern "C" int spinf_selftest_bounded_wait(int64_t limit_ns, void* stream) {
  SPINF_CHECK_ARG(limit_ns > 0 && limit_ns <= 1000000000ll);
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  int* status = status_word(dev);
  if (!status) return SPINF_ERR_CUDA;
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t>(limit_ns), status);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_fused_norm(const void* y, const int64_t* rows, const void* w1, const void* residual, const void* w2, int64_t n_out,
                                int64_t hidden, float eps, int32_t plus1, void* out_h, void* out_norm, void* out_x8, float* out_xs,
                                void* stream) {
  if (n_out == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(y && n_out >= 0 && hidden > 0 && hidden % 8 == 0 && hidden <= NORM_THREADS * NORM_MAX_VEC * 8);
  SPINF_CHECK_ARG((out_x8 == nullptr) == (out_xs == nullptr));
  SPINF_CHECK_ARG(!(out_norm || out_x8) || w2);
  SPINF_CHECK_ARG(n_out < (1ll << 31));
  FusedNormArgs a;
  a.y = static_cast<const __nv_bfloat16*>(y);
  a.rows = rows;
  a.w1 = static_cast<const __nv_bfloat16*>(w1);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.w2 = static_cast<const __nv_bfloat16*>(w2);
  a.out_h = static_cast<__nv_bfloat16*>(out_h);
  a.out_norm = static_cast<__nv_bfloat16*>(out_norm);
  a.out_x8 = static_cast<uint8_t*>(out_x8);
  a.out_xs = out_xs;
  a.hidden = static_cast<int>(hidden);
  a.eps = eps;
  a.plus1 = plus1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int per_thread = static_cast<int>((hidden / 8 + NORM_THREADS - 1) / NORM_THREADS);
  // resident CTAs only (4 per SM at up to 2 vectors per thread, else 2): each walks its share of the rows
  const int64_t resident = static_cast<int64_t>(sm_count()) * (per_thread <= 2 ? 4 : 2);
  const unsigned grid = static_cast<unsigned>(n_out < resident ? n_out : resident);
#define SPINF_NORM_CASE(NV)                                                      \
  if (plus1)                                                                     \
    fused_norm_kernel<NV, true><<<grid, NORM_THREADS, 0, st>>>(a, n_out);        \
  else                                                                           \
    fused_norm_kernel<NV, false><<<grid, NORM_THREADS, 0, st>>>(a, n_out);       \
  break;
  switch (per_thread) {
    case 1: SPINF_NORM_CASE(1)
    case 2: SPINF_NORM_CASE(2)
    case 3: SPINF_NORM_CASE(3)
    default: SPINF_NORM_CASE(4)
  }
#undef SPINF_NORM_CASE
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_qkv_norm_rope(void* qkv, int64_t pitch, int64_t n, int32_t H, int32_t Hkv, int32_t D, const void* wq,
                                   const void* wk, const void* cos_t, const void* sin_t, int32_t rot_dim, float eps, int32_t plus1,
                                   int32_t norm_v, void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(qkv && wq && wk && cos_t && sin_t && n >= 0 && H > 0 && Hkv > 0 && (D == 128 || D == 256));
  SPINF_CHECK_ARG(rot_dim > 0 && rot_dim <= D && rot_dim % (2 * (D / 32)) == 0);
  SPINF_CHECK_ARG(pitch >= static_cast<int64_t>(H + 2 * Hkv) * D);
  const int64_t warps = (n * (H + 2 * Hkv) + 1) / 2;  // two (token, head) items per warp
  const unsigned grid = static_cast<unsigned>((warps + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* p = static_cast<__nv_bfloat16*>(qkv);
  auto* q = static_cast<const __nv_bfloat16*>(wq);
  auto* k = static_cast<const __nv_bfloat16*>(wk);
  auto* c = static_cast<const __nv_bfloat16*>(cos_t);
  auto* s = static_cast<const __nv_bfloat16*>(sin_t);
  if (D == 256)
    qkv_norm_rope_kernel<256><<<grid, 256, 0, st>>>(p, pitch, n, H, Hkv, q, k, c, s, eps, plus1, norm_v, rot_dim, D, H * D, nullptr);
  else
    qkv_norm_rope_kernel<128><<<grid, 256, 0, st>>>(p, pitch, n, H, Hkv, q, k, c, s, eps, plus1, norm_v, rot_dim, D, H * D, nullptr);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_qkv_norm_rope_gated(void* y, int64_t pitch, int64_t n, int32_t H, int32_t Hkv, int32_t D, const void* wq, const void* wk,
                                         const void* cos_t, const void* sin_t, int32_t rot_dim, float eps, int32_t plus1, void* q_out,
                                         void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(y && wq && wk && cos_t && sin_t && q_out && n >= 0 && H > 0 && Hkv > 0 && (D == 128 || D == 256));
  SPINF_CHECK_ARG(rot_dim > 0 && rot_dim <= D && rot_dim % (2 * (D / 32)) == 0);
  SPINF_CHECK_ARG(pitch >= static_cast<int64_t>(2 * H + 2 * Hkv) * D && pitch % 8 == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* p = static_cast<__nv_bfloat16*>(y);
  auto* q = static_cast<const __nv_bfloat16*>(wq);
  auto* k = static_cast<const __nv_bfloat16*>(wk);
  auto* c = static_cast<const __nv_bfloat16*>(cos_t);
  auto* s = static_cast<const __nv_bfloat16*>(sin_t);
  auto* qo = static_cast<__nv_bfloat16*>(q_out);
  // one warp per (token, head); the value heads' warps return at once (norm_v = 0: no norm, no rotary on values)
  const int64_t warps_all = (n * (H + 2 * Hkv) + 1) / 2;
  const unsigned grid_all = static_cast<unsigned>((warps_all + 7) / 8);
  if (D == 256)
    qkv_norm_rope_kernel<256><<<grid_all, 256, 0, st>>>(p, pitch, n, H, Hkv, q, k, c, s, eps, plus1, 0, rot_dim, 2 * D, 2 * H * D, qo);
  else
    qkv_norm_rope_kernel<128><<<grid_all, 256, 0, st>>>(p, pitch, n, H, Hkv, q, k, c, s, eps, plus1, 0, rot_dim, 2 * D, 2 * H * D, qo);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

// o[t, h, :] *= sigmoid(gate[t, h, :]) with the gate read from the interleaved projection output (column h * 2 D + D): the
// sigmoid is rounded to bf16, then the product (both as the reference's bf16 tensor ops round them)
__global__ void attn_gate_kernel(__nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ y, int64_t pitch, int64_t n, int H, int D) {
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  const int64_t per_tok = static_cast<int64_t>(H) * D;
  if (i >= n * per_tok) return;
  const int64_t t = i / per_tok;
  const int r = static_cast<int>(i % per_tok);
  const int h = r / D, d = r % D;
  float x[8], g[8];
  load8(o + i, x);
  load8(y + t * pitch + static_cast<int64_t>(h) * 2 * D + D + d, g);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = x[j] * round_bf16(1.f / (1.f + expf(-g[j])));
  store8(o + i, x);
}

extern "C" int spinf_attn_gate(void* o, const void* y, int64_t pitch, int64_t n, int32_t H, int32_t D, void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(o && y && n >= 0 && H > 0 && D > 0 && D % 8 == 0 && pitch >= 2ll * H * D && pitch % 8 == 0);
  const int64_t vecs = n * H * D / 8;
  attn_gate_kernel<<<static_cast<unsigned>((vecs + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(y), pitch, n, H, D);
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_glu_quant(const void* gu, int64_t n, int64_t F, int32_t act, void* out_x8, float* out_xs, void* out_y,
                               void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(gu && n >= 0 && F > 0 && F % 8 == 0 && (act == 0 || act == 1) && n < (1ll << 31) && F < (1ll << 28));
  SPINF_CHECK_ARG((out_x8 == nullptr) == (out_xs == nullptr) && (out_x8 || out_y));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* g = static_cast<const __nv_bfloat16*>(gu);
  if (act == ACT_GELU_TANH)
    glu_quant_kernel<ACT_GELU_TANH><<<static_cast<unsigned>(n), 512, 0, st>>>(g, static_cast<int>(F), static_cast<uint8_t*>(out_x8), out_xs,
                                                                            static_cast<__nv_bfloat16*>(out_y));
  else
    glu_quant_kernel<ACT_SILU><<<static_cast<unsigned>(n), 512, 0, st>>>(g, static_cast<int>(F), static_cast<uint8_t*>(out_x8), out_xs,
                                                                       static_cast<__nv_bfloat16*>(out_y));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_embed_scale(const int64_t* ids, const void* emb, int64_t n, int64_t hidden, int64_t vocab, float scale, void* out,
                                 void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(ids && emb && out && n >= 0 && hidden > 0 && hidden % 8 == 0 && vocab > 0 && n < (1ll << 31));
  embed_scale_kernel<<<static_cast<unsigned>(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(emb), static_cast<int>(hidden), vocab, scale, static_cast<__nv_bfloat16*>(out));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int spinf_rope_table(const int32_t* pos, int64_t n, int32_t rot_dim, const float* inv_freq, void* cos_t, void* sin_t,
                                void* stream) {
  if (n == 0) return 0;  // nothing to do: the row pointers may be null
  SPINF_CHECK_ARG(pos && cos_t && sin_t && inv_freq && n >= 0 && rot_dim > 0 && rot_dim % 2 == 0);
  const int half = rot_dim / 2;
  const int64_t total = n * half;
  rope_table_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pos, n, half, inv_freq, static_cast<__nv_bfloat16*>(cos_t), static_cast<__nv_bfloat16*>(sin_t));
  SPINF_CUDA_OK(cudaGetLastError());
  return 0;
}
