// Library-wide entry points: version, error strings, per-device set-up.
#include "pe_common.cuh"

namespace pe {
thread_local int g_last_cuda_error = 0;

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (dev < 64) cached[dev] = n;
  return n;
}
}  // namespace pe

extern "C" int pe_version(void) { return 100; }

extern "C" int pe_last_cuda_error(void) { return pe::g_last_cuda_error; }

extern "C" const char* pe_error_string(int code) {
  switch (code) {
    case PE_OK: return "ok";
    case PE_ERR_ARG: return "invalid argument";
    case PE_ERR_SHAPE: return "unsupported shape";
    case PE_ERR_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case PE_ERR_WORKSPACE: return "scratch buffer too small";
    case PE_ERR_CUDA: return "CUDA runtime error";
    case PE_ERR_DEVICE: return "device is not sm_100";
    case PE_ERR_LIMIT: return "size beyond a compiled-in maximum";
    default: return "unknown error";
  }
}

extern "C" int pe_init(int device) {
  PE_CUDA_TRY(cudaSetDevice(device));
  int major = 0;
  PE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10) return PE_ERR_DEVICE;
  return pe::sm_count() > 0 ? PE_OK : PE_ERR_CUDA;
}
