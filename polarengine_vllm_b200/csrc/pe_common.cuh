// Shared device/host helpers for the sm_100a PolarEngine kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/polar_b200.h"

namespace pe {

constexpr int kBlock = 128;  // quantization block = FWHT length

// ---- host-side error plumbing ------------------------------------------------
extern thread_local int g_last_cuda_error;
inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return PE_ERR_CUDA;
}
#define PE_CUDA_TRY(expr)                        \
  do {                                           \
    cudaError_t _e = (expr);                     \
    if (_e != cudaSuccess) return pe::cuda_fail(_e); \
  } while (0)

int sm_count();  // SM count of the current device (cached per device)
long long wait_limit_cycles();  // limit of device-side waits on another party (pe_set_wait_limit_us)

// Launch with programmatic stream serialization: the grid may start while its predecessor
// in the stream is still draining.  The kernel must call pdl_enter() (or its own
// griddepcontrol.wait) before it touches anything the predecessor reads or writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- small device helpers ----------------------------------------------------
// Let the next kernel of the stream start its own prologue now, then wait until the
// previous kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// streaming 16-byte load that does not pollute L1
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// element load as fp32 from an fp32 / fp16 / bf16 array
__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t idx) {
  if (dtype == PE_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == PE_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

__device__ __forceinline__ void store_from_float(void* base, int dtype, int64_t idx, float v) {
  if (dtype == PE_F32) reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == PE_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}

// 4 consecutive elements starting at a multiple of 4, zero beyond `limit`, in two steps so
// that a caller can issue the loads of several items before converting any of them (the
// hardware issues in program order: a conversion right behind its load makes the next load
// wait a full memory round trip).
struct Raw4 { uint32_t w[4]; };  // fp32: four words; fp16 / bf16: two words

__device__ __forceinline__ Raw4 load4_raw(const void* base, int dtype, int64_t row_off, int col, int limit, bool vec_ok) {
  Raw4 r = {{0u, 0u, 0u, 0u}};
  if (vec_ok && col + 4 <= limit) {
    if (dtype == PE_F32) {
      asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
                   : "l"(reinterpret_cast<const float*>(base) + row_off + col));
    } else {
      asm volatile("ld.global.v2.u32 {%0,%1}, [%2];"
                   : "=r"(r.w[0]), "=r"(r.w[1])
                   : "l"(reinterpret_cast<const uint16_t*>(base) + row_off + col));
    }
  } else {  // ragged edge or unaligned rows: element loads
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (col + i < limit) {
        if (dtype == PE_F32) {
          r.w[i] = reinterpret_cast<const uint32_t*>(base)[row_off + col + i];
        } else {
          const uint32_t h = reinterpret_cast<const uint16_t*>(base)[row_off + col + i];
          r.w[i >> 1] |= h << (16 * (i & 1));
        }
      }
    }
  }
  return r;
}

__device__ __forceinline__ void cvt4(const Raw4& r, int dtype, float v[4]) {
  if (dtype == PE_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r.w[i]);
  } else if (dtype == PE_F16) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.w[0]));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.w[1]));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.w[0]));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.w[1]));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}

__device__ __forceinline__ void load4_as_float(const void* base, int dtype, int64_t row_off, int col, int limit,
                                               bool vec_ok, float v[4]) {
  cvt4(load4_raw(base, dtype, row_off, col, limit, vec_ok), dtype, v);
}

// FWHT-128 across one warp.  Lane l holds elements 4l..4l+3 of the block on entry and
// the same positions of the rotated block on return (scaled by 1/sqrt(128)).
// Strides 1 and 2 are in-register; strides 4..64 are lane exchanges with masks 1..16.
__device__ __forceinline__ void warp_fwht128(float v[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m <= 16; m <<= 1) {
    const float sgn = (lane & m) ? -1.f : 1.f;  // upper half of the pair: partner - own (one FMA, exact)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = fmaf(sgn, v[i], o);
    }
  }
  const float s = 0.08838834764831845f;  // 1/sqrt(128)
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= s;
}

}  // namespace pe
