// Device helpers shared by the decode-size matmul kernels: asynchronous 16-byte copies,
// the lane-replicated shared-memory centroid table, the register-resident table for
// layers with at most eight levels, and the fp16x2 multiply-add primitives.
#pragma once
#include "pe_common.cuh"

namespace pe {

constexpr int kLutBytes = 32768;  // 256 entries x 32 lanes x 4 B (entry e of lane l at e*128 + l*4)

// low half of a, high half of b
__device__ __forceinline__ uint32_t lo_hi(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7610;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}


// table address of byte BYTE of a code word: table + byte * 128 + lane * 4
template <int BYTE>
__device__ __forceinline__ uint32_t lut_addr(uint32_t word, uint32_t lane_base) {
  uint32_t bt;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(bt) : "r"(word), "r"(0), "n"(0x4440 | BYTE));
  return bt * 128u + lane_base;
}
__device__ __forceinline__ uint32_t lut_ld(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Register-resident centroid table for layers with at most 8 levels (3-bit codes stored in
// nibbles): the low and the high byte of the eight fp16 centroids sit in two register
// pairs, and one byte-permute looks four codes up at once -- a nibble 0..7 IS a valid
// permute selector.  Two more permutes interleave low and high bytes into the fp16 pairs
// (ct[lo nibble], ct[hi nibble]) the MMA wants.  No shared-memory traffic at all, which is
// what bounds the table-lookup path.
struct RegTable { uint32_t lo0, lo1, hi0, hi1; };

// word (4 code bytes) -> the four A registers of its bytes 0..3
__device__ __forceinline__ void reg_decode(uint32_t w, const RegTable& tb, uint32_t out[4]) {
  uint32_t L, H, w2 = w >> 16;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(L) : "r"(tb.lo0), "r"(tb.lo1), "r"(w));
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(H) : "r"(tb.hi0), "r"(tb.hi1), "r"(w));
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(out[0]) : "r"(L), "r"(H));
  asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(out[1]) : "r"(L), "r"(H));
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(L) : "r"(tb.lo0), "r"(tb.lo1), "r"(w2));
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(H) : "r"(tb.hi0), "r"(tb.hi1), "r"(w2));
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(out[2]) : "r"(L), "r"(H));
  asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(out[3]) : "r"(L), "r"(H));
}

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float h2sum(uint32_t h) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
  return f.x + f.y;
}


__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// fp16 pairs of one code word, in the order the staged activations have them.
//  PACKED: the four bytes' pairs (ct[low nibble], ct[high nibble]) = weights (k, k+64)
//  !PACKED: two pairs (ct[c0], ct[c1]), (ct[c2], ct[c3]) = consecutive weights
template <bool PACKED, bool REGTAB>
__device__ __forceinline__ void decode_word(uint32_t w, uint32_t lane_base, const RegTable& tb, uint32_t a[4]) {
  if (PACKED && REGTAB) {
    reg_decode(w, tb, a);
  } else {
    const uint32_t ad0 = lut_addr<0>(w, lane_base), ad1 = lut_addr<1>(w, lane_base), ad2 = lut_addr<2>(w, lane_base),
                   ad3 = lut_addr<3>(w, lane_base);
    const uint32_t v0 = lut_ld(ad0), v1 = lut_ld(ad1), v2 = lut_ld(ad2), v3 = lut_ld(ad3);
    if (PACKED) {
      a[0] = v0; a[1] = v1; a[2] = v2; a[3] = v3;
    } else {
      a[0] = lo_hi(v0, v1);
      a[1] = lo_hi(v2, v3);
    }
  }
}

// dot product of one lane's 16 bytes of codes with its activation registers
template <bool PACKED, bool REGTAB, int NX>
__device__ __forceinline__ float reg_dot(const uint4& q, uint32_t lane_base, const RegTable& tb, const uint32_t (&x)[NX]) {
  uint32_t a[4][4];
  decode_word<PACKED, REGTAB>(q.x, lane_base, tb, a[0]);
  decode_word<PACKED, REGTAB>(q.y, lane_base, tb, a[1]);
  decode_word<PACKED, REGTAB>(q.z, lane_base, tb, a[2]);
  decode_word<PACKED, REGTAB>(q.w, lane_base, tb, a[3]);
  uint32_t c0, c1, c2, c3;
  if (PACKED) {
    c0 = hmul2_u(a[0][0], x[0]); c1 = hmul2_u(a[1][0], x[4]); c2 = hmul2_u(a[2][0], x[8]); c3 = hmul2_u(a[3][0], x[12]);
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      c0 = hfma2_u(a[0][i], x[i], c0); c1 = hfma2_u(a[1][i], x[4 + i], c1);
      c2 = hfma2_u(a[2][i], x[8 + i], c2); c3 = hfma2_u(a[3][i], x[12 + i], c3);
    }
  } else {
    c0 = hmul2_u(a[0][0], x[0]); c1 = hmul2_u(a[1][0], x[2]); c2 = hmul2_u(a[2][0], x[4]); c3 = hmul2_u(a[3][0], x[6]);
    c0 = hfma2_u(a[0][1], x[1], c0); c1 = hfma2_u(a[1][1], x[3], c1);
    c2 = hfma2_u(a[2][1], x[5], c2); c3 = hfma2_u(a[3][1], x[7], c3);
  }
  return h2sum(hadd2_u(hadd2_u(c0, c1), hadd2_u(c2, c3)));
}


// Decides whether the row-owner kernel (pe_gemv_rows.cu) takes a call and launches it.
// Returns PE_OK after a launch, 1 if the shape is not its kind (the caller goes on to the
// tile kernel), or a negative error code.
int gemv_rows_try(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                  const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f,
                  void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f, int in_f_padded,
                  int* status, cudaStream_t stream);

// The column-owner kernel for 3..8 activation rows (pe_gemv_cols8.cu), row-major layout only.  Returns PE_OK after a
// launch, 1 if the shape is not its kind, or a negative error code; gemv_cols8_takes answers the same question
// without launching.
int gemv_cols8_try(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, const float* ct_scaled,
                   int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f, void* y, int y_dtype,
                   int64_t ld_y, const void* bias, int batch, int out_f, int in_f_padded, cudaStream_t stream);
bool gemv_cols8_takes(int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, int out_f, int in_f_padded);

}  // namespace pe
