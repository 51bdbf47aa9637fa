// Row-parallel epilogue across tensor-parallel ranks, as ONE kernel per rank:
//   all-reduce of the partial projection outputs (o_proj / down_proj shards) over peer
//   memory  +  residual add  +  RMSNorm of the next layer input.
// In the reference's deployment this is an NCCL all-reduce issued by vLLM after the
// row-parallel linear layer (the reference itself only slices the weights:
// loader.py:558-638) followed by the framework's add + norm kernels.
//
// Protocol (one CTA per activation row, every rank runs the same launch):
//  push   the rank's fp32 partial row is stored into slot [parity][rank][row] of EVERY
//         rank's exchange buffer (plain peer stores over NVLink, 16 bytes per thread and
//         peer), then a system-scope fence, then thread r raises flag [rank][row] in
//         rank r's buffer to the call's sequence number (release store);
//  wait   thread r polls the local flag [r][row] (acquire loads, bounded: after ~1 s
//         the status word is set and the kernel carries on with what it has);
//  reduce the world partials of the row are read from LOCAL memory (L1 bypassed) and
//         summed in rank order -- every rank gets the same bits -- then x += fp16(sum),
//         out = fp16(x * rsqrt(mean(x^2) + eps)) * weight.
// Slots are double-buffered by the parity of the sequence number, which lives in device
// memory (graph replays advance it): a rank can be at most one call ahead of a peer,
// because finishing a call needs every peer's flag of that call.
// No multicast, no TMA: ordinary loads and stores on peer-mapped addresses.
#include "pe_common.cuh"

namespace pe {

constexpr int kArThreads = 256;
constexpr int kArMaxIter = 8;     // hidden <= 256 x 8 x 8 = 16384
constexpr int kArMaxWorld = 16;
constexpr size_t kArFlagBytes = 4096;  // flags [world][max_rows] uint32 at the start of the buffer

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_add_rmsnorm_kernel(const float* partial, __half* x, const __half* w, __half* out,
                                                                           int hidden, float eps, const uint64_t* peers, int rank,
                                                                           int world, int max_rows, unsigned* seq, int* status,
                                                                           long long wait_limit) {
  __shared__ float warp_sums[kArThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  pdl_enter();
  const unsigned s = seq[row] + 1u;
  const unsigned parity = s & 1u;
  const size_t slot_floats = (size_t)hidden;
  auto data_of = [&](uint64_t base, int src) {
    return reinterpret_cast<float*>(base + kArFlagBytes) + (((size_t)parity * world + src) * max_rows + row) * slot_floats;
  };
  // ---- push
  const float* mine = partial + (size_t)row * hidden;
#pragma unroll
  for (int it = 0; it < kArMaxIter; ++it) {
    const int col = (it * kArThreads + tid) * 8;
    if (col < hidden) {
      const float4 a = *reinterpret_cast<const float4*>(mine + col);
      const float4 b = *reinterpret_cast<const float4*>(mine + col + 4);
      for (int r = 0; r < world; ++r) {
        float* dst = data_of(peers[r], rank) + col;
        *reinterpret_cast<float4*>(dst) = a;
        *reinterpret_cast<float4*>(dst + 4) = b;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) st_release_sys(reinterpret_cast<unsigned*>(peers[tid]) + (size_t)rank * max_rows + row, s);
  // ---- wait (bounded)
  if (tid < world) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(peers[rank]) + (size_t)tid * max_rows + row;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(flag) - s) < 0) {
      if (clock64() - t0 > wait_limit) {  // about a second unless the host set another limit: a peer never arrived
        atomicExch(status, 1);
        break;
      }
    }
  }
  __syncthreads();
  // ---- reduce + residual add + norm
  __half* xr = x + (size_t)row * hidden;
  const uint64_t local = peers[rank];
  float v[kArMaxIter][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kArMaxIter; ++it) {
    const int col = (it * kArThreads + tid) * 8;
    if (col < hidden) {
      float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        const float* src = data_of(local, r) + col;
        const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(src + 4));
        d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w; d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
      }
      const uint4 u = *reinterpret_cast<const uint4*>(xr + col);
      const __half2* h2 = reinterpret_cast<const __half2*>(&u);
      uint4 o;
      __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h2[i]);
        const float a = f.x + __half2float(__float2half_rn(d[2 * i]));
        const float b = f.y + __half2float(__float2half_rn(d[2 * i + 1]));
        o2[i] = __floats2half2_rn(a, b);
        const float2 g = __half22float2(o2[i]);
        v[it][2 * i] = g.x;
        v[it][2 * i + 1] = g.y;
      }
      *reinterpret_cast<uint4*>(xr + col) = o;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[it][i] * v[it][i];
    }
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
  if ((tid & 31) == 0) warp_sums[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kArThreads / 32; ++i) tot += warp_sums[i];
  const float scale = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < kArMaxIter; ++it) {
    const int col = (it * kArThreads + tid) * 8;
    if (col < hidden) {
      const uint4 wu = *reinterpret_cast<const uint4*>(w + col);
      const __half2* w2 = reinterpret_cast<const __half2*>(&wu);
      uint4 o;
      __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) o2[i] = __hmul2(__floats2half2_rn(v[it][2 * i] * scale, v[it][2 * i + 1] * scale), w2[i]);
      *reinterpret_cast<uint4*>(out + (size_t)row * hidden + col) = o;
    }
  }
  if (tid == 0) seq[row] = s;
}

}  // namespace pe

using namespace pe;

extern "C" size_t pe_allreduce_buffer_bytes(int world, int max_rows, int hidden) {
  if (world < 1 || world > kArMaxWorld || max_rows < 1 || hidden < 8) return 0;
  if ((size_t)world * max_rows * 4 > kArFlagBytes) return 0;
  return kArFlagBytes + (size_t)2 * world * max_rows * hidden * sizeof(float);
}

extern "C" int pe_allreduce_add_rmsnorm(const float* partial, void* x, const void* weight, void* out, int rows, int hidden, float eps,
                                        const uint64_t* peer_buffers, int rank, int world, int max_rows, unsigned* seq,
                                        int* status, void* stream) {
  if (!partial || !x || !weight || !out || !peer_buffers || !seq || !status) return PE_ERR_ARG;
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || rows < 1 || rows > max_rows) return PE_ERR_ARG;
  if (hidden % 8 || hidden < 8 || hidden > kArThreads * 8 * kArMaxIter) return PE_ERR_SHAPE;
  if ((size_t)world * max_rows * 4 > kArFlagBytes) return PE_ERR_LIMIT;
  if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return PE_ERR_ALIGN;
  PE_CUDA_TRY(launch_pdl(allreduce_add_rmsnorm_kernel, dim3(rows), dim3(kArThreads), 0, static_cast<cudaStream_t>(stream), partial,
                         static_cast<__half*>(x), static_cast<const __half*>(weight), static_cast<__half*>(out), hidden, eps,
                         peer_buffers, rank, world, max_rows, seq, status, wait_limit_cycles()));
  return PE_OK;
}
