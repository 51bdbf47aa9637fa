// Glue ops of a decoder layer around the quantized projections: residual add + RMSNorm,
// rotary embedding + KV-cache write, SiLU * up.  They exist so that the end-to-end decode
// measurement is not dominated by dozens of tiny framework kernels; in a vLLM deployment
// the server's own fused ops play this role.  fp16 activations, fp32 arithmetic, results
// rounded where the op-by-op torch formulation rounds.
#include "pe_common.cuh"

namespace pe {

constexpr int kNormThreads = 256;
constexpr int kNormMaxIter = 8;  // hidden <= 256 threads x 8 elements x 8 iterations = 16384

// x[row] += half(delta[row]) (if delta), out[row] = half(x * rsqrt(mean(x^2) + eps)) * w
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(__half* x, const void* delta, int delta_dtype, const __half* w,
                                                                   __half* out, int hidden, float eps) {
  __shared__ float warp_sums[kNormThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  __half* xr = x + (int64_t)row * hidden;
  float v[kNormMaxIter][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kNormMaxIter; ++it) {
    const int col = (it * kNormThreads + tid) * 8;
    if (col < hidden) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + col);
      const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h2[i]);
        v[it][2 * i] = f.x;
        v[it][2 * i + 1] = f.y;
      }
      if (delta) {
        float d[8];
        if (delta_dtype == PE_F32) {
          const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(delta) + (int64_t)row * hidden + col);
          const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(delta) + (int64_t)row * hidden + col + 4);
          d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w; d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
        } else {
          const uint4 du = *reinterpret_cast<const uint4*>(static_cast<const __half*>(delta) + (int64_t)row * hidden + col);
          const __half2* d2 = reinterpret_cast<const __half2*>(&du);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(d2[i]);
            d[2 * i] = f.x;
            d[2 * i + 1] = f.y;
          }
        }
        uint4 o;
        __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // the delta is rounded to fp16 first, then added in fp16 (round to nearest of the exact sum)
          const float a = v[it][2 * i] + __half2float(__float2half_rn(d[2 * i]));
          const float b = v[it][2 * i + 1] + __half2float(__float2half_rn(d[2 * i + 1]));
          o2[i] = __floats2half2_rn(a, b);
          const float2 f = __half22float2(o2[i]);
          v[it][2 * i] = f.x;
          v[it][2 * i + 1] = f.y;
        }
        *reinterpret_cast<uint4*>(xr + col) = o;
      }
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
  for (int i = 0; i < kNormThreads / 32; ++i) tot += warp_sums[i];
  const float scale = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < kNormMaxIter; ++it) {
    const int col = (it * kNormThreads + tid) * 8;
    if (col < hidden) {
      const uint4 wu = *reinterpret_cast<const uint4*>(w + col);
      const __half2* w2 = reinterpret_cast<const __half2*>(&wu);
      uint4 o;
      __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 n = __floats2half2_rn(v[it][2 * i] * scale, v[it][2 * i + 1] * scale);
        o2[i] = __hmul2(n, w2[i]);
      }
      *reinterpret_cast<uint4*>(out + (int64_t)row * hidden + col) = o;
    }
  }
}

// One block per (token, head); thread j rotates the pair (j, j + d/2) (rotate-half form).
// Query heads go to q_out (batch, hq, t, d); key heads (rotated) and value heads (copied)
// go into the caches (batch, hkv, max_len, d) at position base + token index.
__global__ void rope_cache_kernel(const __half* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, __half* q_out,
                                  __half* k_cache, __half* v_cache, int t, int hq, int hkv, int d, int max_len,
                                  float theta) {
  const int tok = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
  const int b = tok / t, i = tok - b * t;
  const int64_t pos = (pos_dev ? *pos_dev : pos_host) + i;
  const __half* src = qkv + (int64_t)tok * ld_qkv + (int64_t)head * d;
  const int half_d = d >> 1;
  if (head < hq + hkv) {
    const float inv = 1.f / powf(theta, (float)(2 * j) / (float)d);
    const float ang = (float)pos * inv;
    const float c = cosf(ang), s = sinf(ang);
    const float x1 = __half2float(src[j]), x2 = __half2float(src[j + half_d]);
    const __half o1 = __float2half_rn(x1 * c - x2 * s), o2 = __float2half_rn(x2 * c + x1 * s);
    if (head < hq) {
      __half* dst = q_out + (((int64_t)b * hq + head) * t + i) * d;
      dst[j] = o1;
      dst[j + half_d] = o2;
    } else if (pos >= 0 && pos < max_len) {
      __half* dst = k_cache + (((int64_t)b * hkv + (head - hq)) * max_len + pos) * d;
      dst[j] = o1;
      dst[j + half_d] = o2;
    }
  } else if (pos >= 0 && pos < max_len) {
    __half* dst = v_cache + (((int64_t)b * hkv + (head - hq - hkv)) * max_len + pos) * d;
    dst[j] = src[j];
    dst[j + half_d] = src[j + half_d];
  }
}

// out[r, i] = half(silu(gate)) * up in fp16, gate = gu[r, i], up = gu[r, inter + i]; 8 elements per thread
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* gu, int64_t ld_gu, __half* out, int64_t ld_out, int inter,
                                                       int64_t n_vec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_vec) return;
  const int per_row = inter >> 3;
  const int64_t r = idx / per_row;
  const int col = (int)(idx - r * per_row) * 8;
  const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld_gu + col);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld_gu + inter + col);
  const __half2* g2 = reinterpret_cast<const __half2*>(&g);
  const __half2* u2 = reinterpret_cast<const __half2*>(&u);
  uint4 o;
  __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(g2[i]);
    const __half2 s = __floats2half2_rn(f.x / (1.f + expf(-f.x)), f.y / (1.f + expf(-f.y)));
    o2[i] = __hmul2(s, u2[i]);
  }
  *reinterpret_cast<uint4*>(out + r * ld_out + col) = o;
}

}  // namespace pe

using namespace pe;

extern "C" int pe_add_rmsnorm(void* x, const void* delta, int delta_dtype, const void* weight, void* out, int rows, int hidden,
                              float eps, void* stream) {
  if (!x || !weight || !out || rows < 1 || hidden < 8) return PE_ERR_ARG;
  if (delta && delta_dtype != PE_F32 && delta_dtype != PE_F16) return PE_ERR_ARG;
  if (hidden % 8 || hidden > kNormThreads * 8 * kNormMaxIter) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return PE_ERR_ALIGN;
  add_rmsnorm_kernel<<<rows, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__half*>(x), delta, delta_dtype, static_cast<const __half*>(weight), static_cast<__half*>(out), hidden, eps);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_rope_cache(const void* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, void* q_out,
                             void* k_cache, void* v_cache, int batch, int t, int hq, int hkv, int head_dim, int max_len,
                             float theta, void* stream) {
  if (!qkv || !q_out || !k_cache || !v_cache || batch < 1 || t < 1 || hq < 1 || hkv < 1 || max_len < 1) return PE_ERR_ARG;
  if (head_dim < 2 || head_dim > 2048 || (head_dim & 1)) return PE_ERR_SHAPE;
  if (ld_qkv < (int64_t)(hq + 2 * hkv) * head_dim) return PE_ERR_ARG;
  if ((int64_t)batch * t > 0x7fffffff || hq + 2 * hkv > 65535) return PE_ERR_LIMIT;
  rope_cache_kernel<<<dim3((unsigned)(batch * t), (unsigned)(hq + 2 * hkv)), head_dim / 2, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(qkv), ld_qkv, pos_dev, pos_host, static_cast<__half*>(q_out), static_cast<__half*>(k_cache),
      static_cast<__half*>(v_cache), t, hq, hkv, head_dim, max_len, theta);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_silu_mul(const void* gate_up, int64_t ld_gu, void* out, int64_t ld_out, int rows, int inter, void* stream) {
  if (!gate_up || !out || rows < 1 || inter < 8) return PE_ERR_ARG;
  if (inter % 8 || ld_gu % 8 || ld_out % 8) return PE_ERR_SHAPE;
  if (ld_gu < 2 * (int64_t)inter || ld_out < inter) return PE_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) return PE_ERR_ALIGN;
  const int64_t n_vec = (int64_t)rows * (inter / 8);
  const int64_t blocks = (n_vec + 255) / 256;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(gate_up), ld_gu,
                                                                                 static_cast<__half*>(out), ld_out, inter, n_vec);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}
