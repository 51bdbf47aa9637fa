// Library-wide entry points: version, error strings, per-device set-up.
#include "pe_common.cuh"

namespace pe {
thread_local int g_last_cuda_error = 0;

// Limit of the device-side waits on another party (a peer's flag, a bulk copy), in clock cycles.
static long long g_wait_limit_cycles = 2000000000ll;  // about one second at 2 GHz
long long wait_limit_cycles() { return g_wait_limit_cycles; }

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

extern "C" int pe_set_wait_limit_us(int64_t microseconds) {
  if (microseconds < 1 || microseconds > 60ll * 1000 * 1000) return PE_ERR_ARG;
  pe::g_wait_limit_cycles = microseconds * 2000;  // SM clocks run at up to 2 GHz: an upper bound in cycles
  return PE_OK;
}

extern "C" int pe_init(int device) {
  PE_CUDA_TRY(cudaSetDevice(device));
  int major = 0;
  PE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10) return PE_ERR_DEVICE;
  return pe::sm_count() > 0 ? PE_OK : PE_ERR_CUDA;
}
