// Stand-alone rotation and nibble-packing kernels (small, HBM-trivial).
#include "pe_common.cuh"

namespace pe {

// One warp per 128-block: pad, rotate (register + shuffle butterflies), convert, store.
__global__ void __launch_bounds__(256) fwht128_kernel(const void* x, int x_dtype, int64_t ld_x, void* out,
                                                      int out_dtype, int64_t ld_out, int batch, int in_f,
                                                      int nb) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t total = (int64_t)batch * nb;
  if (warp >= total) return;  // whole warps leave together
  const int m = (int)(warp / nb), blk = (int)(warp - (int64_t)m * nb);
  const bool vin = (ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  float v[4];
  load4_as_float(x, x_dtype, (int64_t)m * ld_x, blk * kBlock + lane * 4, in_f, vin, v);
  warp_fwht128(v, lane);
  const int64_t o = (int64_t)m * ld_out + blk * kBlock + lane * 4;
  const bool vout = (ld_out % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (vout && out_dtype == PE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = make_float4(v[0], v[1], v[2], v[3]);
  } else if (vout && out_dtype == PE_F16) {
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + o) = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) store_from_float(out, out_dtype, o + i, v[i]);
  }
}

// One thread per 16 output bytes: 16 codes of the first half, 16 of the second half.
__global__ void __launch_bounds__(256) pack_nibble_kernel(const int8_t* codes, uint8_t* packed, int64_t n_chunks) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_chunks) return;
  // chunk i covers packed bytes [16 i, 16 i + 16): block = i / 4, offset (i % 4) * 16 inside its 64 bytes
  const int64_t blk = i >> 2;
  const int off = (int)(i & 3) * 16;
  const uint4 lo = *reinterpret_cast<const uint4*>(codes + blk * kBlock + off);
  const uint4 hi = *reinterpret_cast<const uint4*>(codes + blk * kBlock + 64 + off);
  uint4 r;
  r.x = (lo.x & 0x0f0f0f0fu) | ((hi.x & 0x0f0f0f0fu) << 4);
  r.y = (lo.y & 0x0f0f0f0fu) | ((hi.y & 0x0f0f0f0fu) << 4);
  r.z = (lo.z & 0x0f0f0f0fu) | ((hi.z & 0x0f0f0f0fu) << 4);
  r.w = (lo.w & 0x0f0f0f0fu) | ((hi.w & 0x0f0f0f0fu) << 4);
  *reinterpret_cast<uint4*>(packed + i * 16) = r;
}

// Quantizer: one warp per (weight row, 128-block).  Zero-pad, L2 norm clamped at 1e-10, divide, rotate, scale by
// sqrt(128), nearest Lloyd-Max level by distance (first minimum wins, as the reference's argmin does), int8 code
// and fp16 norm out.  The butterfly rotation and the warp-order sum of squares round differently from the
// reference's matrix product and torch.norm, so a value that sits on a cell boundary to within fp32 rounding can
// land on the other side: a few codes per million differ from the CPU quantizer.
__global__ void __launch_bounds__(256) quantize_kernel(const void* w, int w_dtype, int64_t ld_w, int64_t rows, int in_f, int nb,
                                                       const float* levels, int n_levels, int8_t* codes, int64_t ld_codes,
                                                       __half* norms, int64_t ld_norms) {
  extern __shared__ float lv[];
  for (int i = threadIdx.x; i < n_levels; i += blockDim.x) lv[i] = levels[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= rows * nb) return;  // whole warps leave together
  const int64_t r = warp / nb;
  const int blk = (int)(warp - r * nb);
  const bool vin = (ld_w % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
  float v[4];
  load4_as_float(w, w_dtype, r * ld_w, blk * kBlock + lane * 4, in_f, vin, v);
  float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
  const float nrm = fmaxf(sqrtf(ss), 1e-10f);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __fdiv_rn(v[i], nrm);
  warp_fwht128(v, lane);  // includes the 1/sqrt(128) of the normalised Hadamard matrix
  const float root = 11.313708498984761f;  // sqrt(128)
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float x = v[i] * root;
    int best = 0;
    float bd = fabsf(x - lv[0]);
    for (int j = 1; j < n_levels; ++j) {
      const float d = fabsf(x - lv[j]);
      if (d < bd) { bd = d; best = j; }
    }
    packed |= (uint32_t)(best & 0xff) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(codes + r * ld_codes + blk * kBlock + lane * 4) = packed;
  if (lane == 0) norms[r * ld_norms + blk] = __float2half_rn(nrm);
}

// Quantized embedding lookup: row ids[t] of the table is dequantised on the fly.
// One warp per (token, 128-block): centroid gather, inverse rotation (the rotation is its
// own inverse), block norm, cast.
__global__ void __launch_bounds__(256) embed_kernel(const uint8_t* codes, int packed, int64_t ld_codes, const __half* norms,
                                                    int64_t ld_norms, const float* ct, int n_levels, const int64_t* ids,
                                                    int64_t vocab, void* out, int out_dtype, int64_t ld_out, int tokens,
                                                    int hidden, int nb) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= (int64_t)tokens * nb) return;
  const int t = (int)(warp / nb), blk = (int)(warp - (int64_t)t * nb);
  int64_t row = ids[t];
  const bool ok = row >= 0 && row < vocab;  // out-of-range ids give a zero row
  if (!ok) row = 0;
  float v[4];
  if (packed) {
    // elements 4l..4l+3: low nibbles of bytes 4l.. for l < 16, high nibbles of bytes 4(l-16).. otherwise
    const uint32_t w = *reinterpret_cast<const uint32_t*>(codes + row * ld_codes + blk * 64 + (lane & 15) * 4);
    const uint32_t nib = (lane < 16 ? w : (w >> 4)) & 0x0f0f0f0fu;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (nib >> (8 * i)) & 0xff;
      v[i] = c < n_levels ? __ldg(ct + c) : 0.f;
    }
  } else {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(codes + row * ld_codes + blk * kBlock + lane * 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (w >> (8 * i)) & 0xff;
      v[i] = c < n_levels ? __ldg(ct + c) : 0.f;
    }
  }
  warp_fwht128(v, lane);
  const float nrm = ok ? __half2float(norms[row * ld_norms + blk]) : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int col = blk * kBlock + lane * 4 + i;
    if (col < hidden) store_from_float(out, out_dtype, (int64_t)t * ld_out + col, v[i] * nrm);
  }
}

}  // namespace pe

using namespace pe;

extern "C" int pe_embedding(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                            const float* ct_scaled, int n_levels, const int64_t* ids, int64_t vocab, void* out,
                            int out_dtype, int64_t ld_out, int tokens, int hidden, int hidden_padded, void* stream) {
  if (!codes || !norms || !ct_scaled || !ids || !out || tokens < 1 || hidden < 1 || vocab < 1) return PE_ERR_ARG;
  if (out_dtype < PE_F32 || out_dtype > PE_BF16 || n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (hidden_padded % kBlock || hidden > hidden_padded || hidden_padded - hidden >= kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 3) || (ld_codes & 3)) return PE_ERR_ALIGN;
  if (ld_out < hidden) return PE_ERR_ARG;
  const int nb = hidden_padded / kBlock;
  const int64_t warps = (int64_t)tokens * nb;
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  embed_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(codes), packed, ld_codes, static_cast<const __half*>(norms), ld_norms, ct_scaled, n_levels,
      ids, vocab, out, out_dtype, ld_out, tokens, hidden, nb);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_fwht128(const void* x, int x_dtype, int64_t ld_x, void* x_tf, int out_dtype, int64_t ld_out,
                          int batch, int in_f, int in_f_padded, void* stream) {
  if (!x || !x_tf || batch < 1 || in_f < 1) return PE_ERR_ARG;
  if (x_dtype < PE_F32 || x_dtype > PE_BF16 || out_dtype < PE_F32 || out_dtype > PE_BF16) return PE_ERR_ARG;
  if (in_f_padded % kBlock || in_f > in_f_padded || in_f_padded - in_f >= kBlock) return PE_ERR_SHAPE;
  if (ld_x < in_f || ld_out < in_f_padded) return PE_ERR_ARG;
  const int nb = in_f_padded / kBlock;
  const int64_t warps = (int64_t)batch * nb;
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  fwht128_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, x_dtype, ld_x, x_tf, out_dtype,
                                                                                 ld_out, batch, in_f, nb);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_pack_nibble(const int8_t* codes, uint8_t* packed, int64_t out_f, int64_t in_f_padded, void* stream) {
  if (!codes || !packed || out_f < 1 || in_f_padded < 1) return PE_ERR_ARG;
  if (in_f_padded % kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15)) return PE_ERR_ALIGN;
  const int64_t n_chunks = out_f * (in_f_padded / 32);
  const int64_t blocks = (n_chunks + 255) / 256;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  pack_nibble_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(codes, packed, n_chunks);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_quantize(const void* weight, int w_dtype, int64_t ld_w, int64_t out_f, int in_f, int in_f_padded,
                           const float* levels, int n_levels, int8_t* codes, int64_t ld_codes, void* norms, int64_t ld_norms,
                           void* stream) {
  if (!weight || !levels || !codes || !norms || out_f < 1 || in_f < 1 || in_f > in_f_padded) return PE_ERR_ARG;
  if (w_dtype < PE_F32 || w_dtype > PE_BF16 || n_levels < 2 || n_levels > 256) return PE_ERR_ARG;
  if (in_f_padded % kBlock) return PE_ERR_SHAPE;
  if (ld_w < in_f || ld_codes < in_f_padded || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 3) || (ld_codes & 3)) return PE_ERR_ALIGN;
  const int nb = in_f_padded / kBlock;
  const int64_t warps = out_f * nb;
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  quantize_kernel<<<(unsigned)blocks, 256, n_levels * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      weight, w_dtype, ld_w, out_f, in_f, nb, levels, n_levels, codes, ld_codes, static_cast<__half*>(norms), ld_norms);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}
