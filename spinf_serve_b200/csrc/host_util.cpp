#include "host_util.h"

#include <mutex>

namespace spinf {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return SPINF_ERR_TENSORMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || box_cols * elem_bytes != 128 || box_rows > 256)
    return SPINF_ERR_TENSORMAP;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SPINF_ERR_TENSORMAP;
}

int make_tmap_2d_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                       uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return SPINF_ERR_TENSORMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || (box_cols & 15) || box_cols > 256 || box_rows > 256)
    return SPINF_ERR_TENSORMAP;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SPINF_ERR_TENSORMAP;
}

int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return SPINF_ERR_TENSORMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15) || b0 * elem_bytes != 128 || b1 > 256)
    return SPINF_ERR_TENSORMAP;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SPINF_ERR_TENSORMAP;
}

static int* g_status[64] = {nullptr};
static int g_sms[64] = {0};
static std::mutex g_mu;

int* status_word(int device) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[device]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[device] = p;
  }
  return g_status[device];
}

int read_and_clear_status(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SPINF_ERR_CUDA;
  int* w = status_word(dev);
  if (!w) return SPINF_ERR_CUDA;
  int h = 0;
  if (cudaMemcpyAsync(&h, w, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return SPINF_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return SPINF_ERR_CUDA;
  if (h != 0) cudaMemsetAsync(w, 0, sizeof(int), stream);
  return h;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

}  // namespace spinf
