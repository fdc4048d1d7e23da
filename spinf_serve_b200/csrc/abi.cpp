// Library-level entry points: version, per-device preparation, status read-back.
#include "host_util.h"

using namespace spinf;

extern "C" int spinf_version(void) { return 200; }  // 0.2.0: the int4 weight layout of spinf_w4_gemm changed (spinf_w4_repack); per-tensor fp8, int8 and GLU entry points added

extern "C" int spinf_init(void) {
  int dev = 0;
  SPINF_CUDA_OK(cudaGetDevice(&dev));
  cudaDeviceProp p;
  SPINF_CUDA_OK(cudaGetDeviceProperties(&p, dev));
  if (p.major != 10) return SPINF_ERR_CUDA;  // sm_100a code only
  if (!status_word(dev)) return SPINF_ERR_CUDA;
  if (!encode_tiled_fn()) return SPINF_ERR_TENSORMAP;
  return 0;
}

extern "C" int spinf_last_status(void* stream) { return read_and_clear_status(static_cast<cudaStream_t>(stream)); }
