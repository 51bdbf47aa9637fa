// Row-owner matmul for one or two activation rows (the batch-1 / batch-2 decode step).
//
//   y[m, r] = sum_blk norm[r, blk] * sum_k ct[code[r, blk, k]] * xt[m, blk, k]   (+ bias[r])
//
// The tile kernel in pe_gemv.cu cuts a layer into equal byte ranges whatever its shape,
// which splits weight rows between CTAs and ends every launch with a hand-off through
// global memory (partials, a release/acquire pair, a second pass by the reducing CTA).
// At 1..2 activation rows that tail is a fifth of the launch.  Here a CTA owns whole
// weight rows instead, so nothing ever crosses CTAs:
//
//  * CTA c owns rows [c N / G, (c+1) N / G): one contiguous region of the row-major code
//    array (the reference's layout, unchanged) and of the norm array.  No scratch memory.
//  * The region is a line of 512-byte "items" (one weight row x 8 nibble blocks or 4 byte
//    blocks); warp w of 16 takes a contiguous 1/16 of the line.  An item is one 16-byte
//    asynchronous copy per lane into a lane-private ring in shared memory (12 items per
//    warp in flight, ~100 KB per SM) plus one 16/8-byte copy of the item's block norms.
//  * The activations are rotated once per CTA (zero-pad, FWHT-128 in registers and
//    shuffles) and staged in shared memory as fp16, laid out so that the four 16-byte
//    pieces a lane needs for an item are conflict-free 128-bit loads.
//  * A lane multiplies its 32 (16) weights of the item with fp16x2 FMAs -- four short
//    chains, widened to fp32 and scaled by the block norm -- and keeps a per-row fp32
//    partial.  When a row ends the 32 lanes are summed by shuffles.  A row that lies
//    inside one warp is stored directly; a row shared by neighbouring warps leaves one
//    partial per warp in shared memory and is summed in warp order after the loop, so the
//    result is bit-identical from run to run.
//  * Centroid lookup as in the tile kernel: register table (byte permutes) for layers
//    with at most eight levels, lane-replicated shared-memory table otherwise.
#include "pe_gemv_decode.cuh"

namespace pe {

constexpr int kRowWarps = 16;
constexpr int kRowThreads = kRowWarps * 32;
constexpr int kItemBytes = 512;
constexpr int kRowStage = kItemBytes + 16;  // codes + the item's norms

struct RowArgs {
  const uint8_t* codes;  // rows of cpr * 512 bytes, contiguous
  const uint8_t* norms;  // fp16, rows of nb, contiguous
  const float* ct; int n_levels;
  const void* x; int x_kind; int x_dtype; int64_t ld_x; int in_f;
  void* y; int y_dtype; int64_t ld_y;
  const __half* bias;
  int batch, N, K, nb, cpr;
};

__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
// dot product of one lane's 16 bytes of codes with its slice of one activation row
template <bool PACKED, bool REGTAB>
__device__ __forceinline__ float item_dot(const uint32_t a[4][4], uint32_t xp) {
  if (PACKED) {
    const uint4 x0 = lds128(xp), x1 = lds128(xp + 512), x2 = lds128(xp + 1024), x3 = lds128(xp + 1536);
    uint32_t c0 = hmul2_u(a[0][0], x0.x), c1 = hmul2_u(a[1][0], x1.x), c2 = hmul2_u(a[2][0], x2.x), c3 = hmul2_u(a[3][0], x3.x);
    c0 = hfma2_u(a[0][1], x0.y, c0); c1 = hfma2_u(a[1][1], x1.y, c1); c2 = hfma2_u(a[2][1], x2.y, c2); c3 = hfma2_u(a[3][1], x3.y, c3);
    c0 = hfma2_u(a[0][2], x0.z, c0); c1 = hfma2_u(a[1][2], x1.z, c1); c2 = hfma2_u(a[2][2], x2.z, c2); c3 = hfma2_u(a[3][2], x3.z, c3);
    c0 = hfma2_u(a[0][3], x0.w, c0); c1 = hfma2_u(a[1][3], x1.w, c1); c2 = hfma2_u(a[2][3], x2.w, c2); c3 = hfma2_u(a[3][3], x3.w, c3);
    return h2sum(hadd2_u(c0, c1)) + h2sum(hadd2_u(c2, c3));
  } else {
    const uint4 x0 = lds128(xp), x1 = lds128(xp + 512);
    uint32_t c0 = hmul2_u(a[0][0], x0.x), c1 = hmul2_u(a[1][0], x0.z), c2 = hmul2_u(a[2][0], x1.x), c3 = hmul2_u(a[3][0], x1.z);
    c0 = hfma2_u(a[0][1], x0.y, c0); c1 = hfma2_u(a[1][1], x0.w, c1); c2 = hfma2_u(a[2][1], x1.y, c2); c3 = hfma2_u(a[3][1], x1.w, c3);
    return h2sum(hadd2_u(c0, c1)) + h2sum(hadd2_u(c2, c3));
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

__device__ __forceinline__ void emit_row(const RowArgs& p, int row, int m, float v) {
  if (p.bias) v += __half2float(p.bias[row]);
  store_from_float(p.y, p.y_dtype, (int64_t)m * p.ld_y + row, v);
}

// Where the rotated block `b` of an activation row goes: lane l holds elements 4l..4l+3.
template <bool PACKED>
__device__ __forceinline__ void place_row_block(uint8_t* xrow, int b, const float v[4], int lane) {
  if (PACKED) {  // pairs (k, k+64); reader lane (b%8)*4 + k/16 takes piece (k%16)/4 of its item
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[i], 16);
    if (lane < 16) {
      const uint4 u = make_uint4(pack_half2(v[0], o[0]), pack_half2(v[1], o[1]), pack_half2(v[2], o[2]), pack_half2(v[3], o[3]));
      *reinterpret_cast<uint4*>(xrow + (b >> 3) * 2048 + (lane & 3) * 512 + ((b & 7) * 4 + (lane >> 2)) * 16) = u;
    }
  } else {  // natural order; reader lane (b%4)*8 + k/16 takes piece (k%16)/8
    const uint2 u = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
    *reinterpret_cast<uint2*>(xrow + (b >> 2) * 1024 + ((lane & 3) >> 1) * 512 + ((b & 3) * 8 + (lane >> 2)) * 16 + (lane & 1) * 8) = u;
  }
}

template <bool PACKED, bool REGTAB, int NBATCH, int DEPTH>
__global__ void __launch_bounds__(kRowThreads, 1) gemv_rows_kernel(const RowArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int ent_row[2 * kRowWarps];
  __shared__ float ent_val[2 * kRowWarps][2];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int G = gridDim.x, cta = blockIdx.x;
  constexpr int kNormBytes = PACKED ? 16 : 8;   // norms of one item
  constexpr int kChunkX = PACKED ? 2048 : 1024;  // staged activation bytes one item reads from

  const int r_beg = (int)((long long)p.N * cta / G), r_end = (int)((long long)p.N * (cta + 1) / G);
  const int items = (r_end - r_beg) * p.cpr;
  const int i0 = (int)((long long)items * w / kRowWarps), i1 = (int)((long long)items * (w + 1) / kRowWarps);

  // Programmatic dependent launch: codes, norms and centroids never change, so they are
  // requested before the previous kernel in the stream has finished; activations and the
  // output belong to it until griddepcontrol.wait returns.
  asm volatile("griddepcontrol.launch_dependents;");
  float ct_mine = 0.f;
  {
    const int e = PACKED ? (lane & 15) : (w + 16 * (lane & 15));
    if (e < p.n_levels) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(ct_mine) : "l"(p.ct + e));
  }

  // shared memory: [table 32 KB unless REGTAB][activations NBATCH x K fp16][ring]
  uint8_t* lut_g = smem;
  uint8_t* xs = smem + (REGTAB ? 0 : kLutBytes);
  const int x_row_bytes = p.K * 2;
  uint8_t* ring_g = xs + (size_t)NBATCH * x_row_bytes + (size_t)w * (DEPTH * kRowStage);
  const uint32_t st_base = smem_u32(ring_g), st_end = st_base + DEPTH * kRowStage;

  const int64_t gi0 = (int64_t)r_beg * p.cpr + i0;  // first item of this warp on the layer's item line
  const uint8_t* cptr = p.codes + gi0 * kItemBytes + lane * 16;
  const uint8_t* nptr = p.norms + gi0 * kNormBytes;
  int n_fetch = i0;
  {
    uint32_t st = st_base;
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (n_fetch < i1) {
        cp_async16(st + lane * 16, cptr);
        if (lane == 0) {
          if (PACKED) cp_async16(st + kItemBytes, nptr);
          else cp_async8(st + kItemBytes, nptr);
        }
        cptr += kItemBytes;
        nptr += kNormBytes;
        ++n_fetch;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      st += kRowStage;
    }
  }

  // ---- centroid table
  RegTable tb = {0, 0, 0, 0};
  if (PACKED && REGTAB) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hb = __half_as_ushort(__float2half_rn(__shfl_sync(0xffffffffu, ct_mine, i)));
      if (i < 4) { tb.lo0 |= (hb & 0xff) << (8 * i); tb.hi0 |= (hb >> 8) << (8 * i); }
      else { tb.lo1 |= (hb & 0xff) << (8 * (i - 4)); tb.hi1 |= (hb >> 8) << (8 * (i - 4)); }
    }
  } else if (PACKED) {
    const float lo = __shfl_sync(0xffffffffu, ct_mine, w);  // entry w + 16 i: low nibble w, high nibble i
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float hi = __shfl_sync(0xffffffffu, ct_mine, i);
      *reinterpret_cast<uint32_t*>(lut_g + (w + 16 * i) * 128 + lane * 4) = pack_half2(lo, hi);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float c = __shfl_sync(0xffffffffu, ct_mine, i);
      if (w + 16 * i < p.n_levels) *reinterpret_cast<uint32_t*>(lut_g + (w + 16 * i) * 128 + lane * 4) = pack_half2(c, c);
    }
  }
  const uint32_t lane_base = smem_u32(lut_g) + lane * 4;
  if (lane == 0) { ent_row[2 * w] = -1; ent_row[2 * w + 1] = -1; }

  // ---- activations: every (row, block) pair is one warp job; loads of a group go out
  // together so that a warp pays one memory latency per group
  asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    const bool raw = p.x_kind == PE_X_RAW;
    const bool vec_ok = (p.ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
    const int limit = raw ? p.in_f : p.K;
    const int jobs = p.nb * NBATCH;
    constexpr int U = 6;
    for (int base = w; base < jobs; base += kRowWarps * U) {
      float v[U][4];
      Raw4 raw4[U];  // loads first, conversions after: one memory round trip per group
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int job = base + u * kRowWarps;
        const bool on = job < jobs;
        const int m = (NBATCH > 1 && job >= p.nb) ? 1 : 0;
        const int b = job - m * p.nb;
        raw4[u] = load4_raw(p.x, p.x_dtype, (int64_t)m * p.ld_x, (on ? b : 0) * kBlock + lane * 4, on ? limit : 0, vec_ok);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) cvt4(raw4[u], p.x_dtype, v[u]);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int job = base + u * kRowWarps;
        if (job < jobs) {  // warp-uniform
          const int m = (NBATCH > 1 && job >= p.nb) ? 1 : 0;
          if (raw) warp_fwht128(v[u], lane);
          place_row_block<PACKED>(xs + m * x_row_bytes, job - m * p.nb, v[u], lane);
        }
      }
    }
  }
  __syncthreads();

  // ---- the item line
  int ch = i0 % p.cpr;
  int row = r_beg + i0 / p.cpr;
  bool started_here = ch == 0;
  int n_ent = 0;
  float acc0 = 0.f, acc1 = 0.f;
  const uint32_t xs_s = smem_u32(xs) + lane * 16;
  uint32_t xp = xs_s + ch * kChunkX;
  uint32_t st = st_base;
  const uint32_t norm_off = kItemBytes + (PACKED ? (lane >> 2) : (lane >> 3)) * 2;
  for (int i = i0; i < i1; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
    const uint4 q = lds128(st + lane * 16);
    unsigned short nh;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(nh) : "r"(st + norm_off));
    const float nrm = __half2float(__ushort_as_half(nh));
    uint32_t a[4][4];
    decode_word<PACKED, REGTAB>(q.x, lane_base, tb, a[0]);
    decode_word<PACKED, REGTAB>(q.y, lane_base, tb, a[1]);
    decode_word<PACKED, REGTAB>(q.z, lane_base, tb, a[2]);
    decode_word<PACKED, REGTAB>(q.w, lane_base, tb, a[3]);
    acc0 = fmaf(nrm, item_dot<PACKED, REGTAB>(a, xp), acc0);
    if (NBATCH > 1) acc1 = fmaf(nrm, item_dot<PACKED, REGTAB>(a, xp + x_row_bytes), acc1);
    __syncwarp();  // every lane has read the stage (codes and norms) before it is refilled
    if (n_fetch < i1) {
      cp_async16(st + lane * 16, cptr);
      if (lane == 0) {
        if (PACKED) cp_async16(st + kItemBytes, nptr);
        else cp_async8(st + kItemBytes, nptr);
      }
      cptr += kItemBytes;
      nptr += kNormBytes;
      ++n_fetch;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    st += kRowStage;
    if (st == st_end) st = st_base;
    xp += kChunkX;
    ++ch;
    if (ch == p.cpr || i == i1 - 1) {  // the row ends, or this warp's share of it does
      const float t0 = warp_sum(acc0);
      const float t1 = NBATCH > 1 ? warp_sum(acc1) : 0.f;
      if (started_here && ch == p.cpr) {
        if (lane == 0) {
          emit_row(p, row, 0, t0);
          if (NBATCH > 1) emit_row(p, row, 1, t1);
        }
      } else {
        if (lane == 0) {
          ent_row[2 * w + n_ent] = row;
          ent_val[2 * w + n_ent][0] = t0;
          ent_val[2 * w + n_ent][1] = t1;
        }
        ++n_ent;
      }
      acc0 = acc1 = 0.f;
      ch = 0;
      xp = xs_s;
      ++row;
      started_here = true;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- rows shared by neighbouring warps: the first entry of a row sums the row's
  // entries in warp order (entries are in row order; unused slots hold -1)
  __syncthreads();
  if (tid < 2 * kRowWarps) {
    const int r = ent_row[tid];
    if (r >= 0) {
      int prev = tid - 1;
      while (prev >= 0 && ent_row[prev] < 0) --prev;
      if (prev < 0 || ent_row[prev] != r) {
        float s0 = 0.f, s1 = 0.f;
        for (int f = tid; f < 2 * kRowWarps; ++f) {
          const int rr = ent_row[f];
          if (rr == r) { s0 += ent_val[f][0]; s1 += ent_val[f][1]; }
          else if (rr >= 0) break;
        }
        emit_row(p, r, 0, s0);
        if (NBATCH > 1) emit_row(p, r, 1, s1);
      }
    }
  }
}

// ---- one activation row: activations in registers -----------------------------------
//
// With a single activation row the loop above is bound by shared-memory bandwidth: every
// 512 bytes of codes drag 2 KB of staged activations through the same port as the ring
// and the table.  Here an item is 8 or 16 weight rows x 128 bytes (8 lanes x 16 B per row,
// two or four rows per lane) and warp w owns the 128-byte column chunks w, w+16, ... of the
// CTA's rows, so a lane meets the same few activation slices over and over and keeps them in
// registers (16 fp16 pairs per chunk, at most CPW chunks), and the rows of a lane give the
// scheduler independent dependency chains.  The price is a reduction per row
// group -- three shuffles over the 8 lanes of a row -- and a sum over the 16 warps' column
// partials through shared memory, in warp order (bit-reproducible), after every pass of
// 256 rows.  Each warp rotates only the blocks it owns.
constexpr int kPassRows = 256;
constexpr int kPartStride = kRowWarps + 1;  // floats per row in the partial array (bank spread)

struct ColArgs {
  const uint8_t* codes; int64_t ld_codes;  // bytes
  const uint8_t* norms; int64_t ld_norms;  // bytes between rows of fp16 norms
  const float* ct; int n_levels;
  const void* x; int x_kind; int x_dtype; int in_f;
  void* y; int y_dtype;
  const __half* bias;
  int N, K, n_chunks;
  // activation prologue (PE_PRO_*): what turns `x` into the matmul input
  int pro;
  const void* delta; int delta_dtype;  // PE_PRO_ADD_RMSNORM: optional addend of the residual x (fp16 / fp32)
  const __half* norm_w;                // PE_PRO_ADD_RMSNORM: norm weight
  __half* resid_out;                   // PE_PRO_ADD_RMSNORM: the updated residual (written by CTA 0), may be null
  float eps;
};

// ---- activation prologues: the glue op in front of a projection, computed while its input is staged ----
// PE_PRO_ADD_RMSNORM  input = half(r * rsqrt(mean(r^2) + eps)) * w   with r = half(x + half(delta)), the rounding
//                     steps of pe_add_rmsnorm;  PE_PRO_SILU_MUL  input = half(silu(gate)) * up, those of pe_silu_mul.
// 4 consecutive elements starting at `col` (a multiple of 4), zero beyond in_f.
__device__ __forceinline__ void resid4(const ColArgs& p, int col, float r[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.x) + col);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  r[0] = a.x; r[1] = a.y; r[2] = b.x; r[3] = b.y;
  if (p.delta) {
    float d[4];
    if (p.delta_dtype == PE_F32) {
      const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(p.delta) + col);
      d[0] = f.x; d[1] = f.y; d[2] = f.z; d[3] = f.w;
    } else {
      const uint2 du = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.delta) + col);
      const float2 da = __half22float2(*reinterpret_cast<const __half2*>(&du.x)), db = __half22float2(*reinterpret_cast<const __half2*>(&du.y));
      d[0] = da.x; d[1] = da.y; d[2] = db.x; d[3] = db.y;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = __half2float(__float2half_rn(r[i] + __half2float(__float2half_rn(d[i]))));
  }
}

__device__ __forceinline__ void pro_load4(const ColArgs& p, int col, bool on, float scale, float v[4]) {
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (!on || col >= p.in_f) return;  // in_f is a multiple of 4 on this path
  if (p.pro == PE_PRO_ADD_RMSNORM) {
    float r[4];
    resid4(p, col, r);
    const uint2 wu = *reinterpret_cast<const uint2*>(p.norm_w + col);
    const __half2 n0 = __hmul2(__floats2half2_rn(r[0] * scale, r[1] * scale), *reinterpret_cast<const __half2*>(&wu.x));
    const __half2 n1 = __hmul2(__floats2half2_rn(r[2] * scale, r[3] * scale), *reinterpret_cast<const __half2*>(&wu.y));
    const float2 a = __half22float2(n0), b = __half22float2(n1);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {  // PE_PRO_SILU_MUL: x = [gate (in_f) | up (in_f)]
    const uint2 g = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.x) + col);
    const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.x) + p.in_f + col);
    const float2 g0 = __half22float2(*reinterpret_cast<const __half2*>(&g.x)), g1 = __half22float2(*reinterpret_cast<const __half2*>(&g.y));
    const __half2 s0 = __floats2half2_rn(g0.x / (1.f + expf(-g0.x)), g0.y / (1.f + expf(-g0.y)));
    const __half2 s1 = __floats2half2_rn(g1.x / (1.f + expf(-g1.x)), g1.y / (1.f + expf(-g1.y)));
    const float2 a = __half22float2(__hmul2(s0, *reinterpret_cast<const __half2*>(&u.x)));
    const float2 b = __half22float2(__hmul2(s1, *reinterpret_cast<const __half2*>(&u.y)));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// ring slot of one item: SUB sub-items of 4 rows x 128 bytes, then 4 bytes of norms per row, rounded to whole 128-byte lines
__host__ __device__ constexpr int col_stage_bytes(int sub) { return (sub * kItemBytes + sub * 16 + 127) & ~127; }

template <bool PACKED, bool REGTAB, int CPW, int DEPTH, int SUB>
__global__ void __launch_bounds__(kRowThreads, 1) gemv_cols_kernel(const ColArgs p) {
  constexpr int kColStage = col_stage_bytes(SUB);
  constexpr int kGroupRows = 4 * SUB;  // weight rows of one item
  static_assert(DEPTH % CPW == 0, "the ring holds whole row groups");
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ float pro_red[kRowWarps];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int rs = lane >> 3, pc = lane & 7;  // row of the sub-item, 16-byte piece of the chunk
  const int G = gridDim.x, cta = blockIdx.x;
  constexpr int kXPerChunk = PACKED ? 16 : 8;  // fp16 pairs a lane keeps per chunk
  constexpr int kRgDepth = DEPTH / CPW;        // row groups in flight per warp
  constexpr int kNormStep = PACKED ? 64 : 32;  // norm bytes between this warp's chunks

  const int r_beg = (int)((long long)p.N * cta / G), r_end = (int)((long long)p.N * (cta + 1) / G);
  const int n_rg = (r_end - r_beg + kGroupRows - 1) / kGroupRows;
  int cnt = (p.n_chunks - w + kRowWarps - 1) / kRowWarps;  // chunks w, w+16, ... of this warp
  cnt = cnt < 0 ? 0 : (cnt > CPW ? CPW : cnt);

  asm volatile("griddepcontrol.launch_dependents;");
  float ct_mine = 0.f;
  {
    const int e = PACKED ? (lane & 15) : (w + 16 * (lane & 15));
    if (e < p.n_levels) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(ct_mine) : "l"(p.ct + e));
  }

  // shared memory: [table 32 KB unless REGTAB][rotation scratch][partials][ring]
  uint8_t* lut_g = smem;
  uint8_t* xw = smem + (REGTAB ? 0 : kLutBytes) + (size_t)w * (CPW * 512);
  float* part = reinterpret_cast<float*>(smem + (REGTAB ? 0 : kLutBytes) + (size_t)kRowWarps * CPW * 512);
  uint8_t* ring_g = reinterpret_cast<uint8_t*>(part) + kPassRows * kPartStride * 4 + (size_t)w * (DEPTH * kColStage);
  const uint32_t st_base = smem_u32(ring_g), st_end = st_base + DEPTH * kColStage;

  // ---- code stream.  An item is 4 SUB weight rows x 128 bytes: lane (rs, pc) copies its 16
  // bytes of rows rs, rs + 4, ... of the group.  The ring slot of item (row group rg, chunk
  // slot j) is (rg % kRgDepth) * CPW + j, so the refill issued after item (rg, j) is item
  // (rg + kRgDepth, j): same slot, same j, and the source is a running pointer plus a
  // compile-time offset.  One copy group per slot, empty for slots the warp does not
  // have, so the group count the math waits on is a constant.  Rows past the end of the
  // matrix are not fetched (their sums are never stored).
  const uint8_t* cptr_f = p.codes + (int64_t)(r_beg + rs) * p.ld_codes + (size_t)w * 128 + pc * 16;
  const uint8_t* nptr_f = p.norms + (int64_t)(r_beg + (lane & (kGroupRows - 1))) * p.ld_norms + (PACKED ? (size_t)w * 4 : (size_t)(w & ~1) * 2);
  const int64_t csub = 4 * p.ld_codes, cstep = kGroupRows * p.ld_codes, nstep = kGroupRows * p.ld_norms;
  int rg_f = 0;
  // sub-item s of the group being fetched covers rows r_beg + kGroupRows rg_f + 4 s .. + 3: skipped
  // as a whole beyond the CTA's rows, per row beyond the matrix
  int row_f = r_beg + rs;  // this lane's row in sub-item 0
  const uint32_t q_off = lane * 16;
  auto fetch_item = [&](uint32_t st, int j) {
    if (j < cnt && rg_f < n_rg) {
#pragma unroll
      for (int sb = 0; sb < SUB; ++sb)
        if (row_f + 4 * sb - rs < r_end && row_f + 4 * sb < p.N) cp_async16(st + sb * kItemBytes + q_off, cptr_f + sb * csub + j * 2048);
      if (lane < kGroupRows && row_f - rs + lane < p.N) cp_async4(st + SUB * kItemBytes + lane * 4, nptr_f + j * kNormStep);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto advance_fetch = [&]() {
    ++rg_f;
    cptr_f += cstep;
    nptr_f += nstep;
    row_f += kGroupRows;
  };
#pragma unroll
  for (int d = 0; d < kRgDepth; ++d) {
#pragma unroll
    for (int j = 0; j < CPW; ++j) fetch_item(st_base + (d * CPW + j) * kColStage, j);
    advance_fetch();
  }


  // ---- centroid table (built before the dependency wait: it needs nothing from the previous kernel)
  RegTable tb = {0, 0, 0, 0};
  if (PACKED && REGTAB) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hb = __half_as_ushort(__float2half_rn(__shfl_sync(0xffffffffu, ct_mine, i)));
      if (i < 4) { tb.lo0 |= (hb & 0xff) << (8 * i); tb.hi0 |= (hb >> 8) << (8 * i); }
      else { tb.lo1 |= (hb & 0xff) << (8 * (i - 4)); tb.hi1 |= (hb >> 8) << (8 * (i - 4)); }
    }
  } else if (PACKED) {
    const float lo = __shfl_sync(0xffffffffu, ct_mine, w);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float hi = __shfl_sync(0xffffffffu, ct_mine, i);
      *reinterpret_cast<uint32_t*>(lut_g + (w + 16 * i) * 128 + lane * 4) = pack_half2(lo, hi);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float c = __shfl_sync(0xffffffffu, ct_mine, i);
      if (w + 16 * i < p.n_levels) *reinterpret_cast<uint32_t*>(lut_g + (w + 16 * i) * 128 + lane * 4) = pack_half2(c, c);
    }
  }
  const uint32_t lane_base = smem_u32(lut_g) + lane * 4;

  // ---- this warp's activation slices: load, rotate, bounce through the warp's scratch
  // into the item layout, keep in registers
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t xr[CPW][kXPerChunk];
  {
    const bool raw = p.x_kind == PE_X_RAW;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;
    const int limit = raw ? p.in_f : p.K;
    constexpr int BPC = PACKED ? 2 : 1;  // quantization blocks per chunk
    float v[CPW * BPC][4];
    if (p.pro == PE_PRO_NONE) {
      // All loads are issued before any of them is used: the issue order is the program
      // order, so a conversion placed right behind its load would make every load wait for
      // the one before it (one memory round trip per block instead of one in total).
      Raw4 raw4[CPW * BPC];
#pragma unroll
      for (int u = 0; u < CPW * BPC; ++u) {
        const bool on = u / BPC < cnt;
        const int col = (on ? (w + 16 * (u / BPC)) * BPC + (u % BPC) : 0) * kBlock + lane * 4;
        raw4[u] = load4_raw(p.x, p.x_dtype, 0, col, on ? limit : 0, vec_ok);
      }
#pragma unroll
      for (int u = 0; u < CPW * BPC; ++u) cvt4(raw4[u], p.x_dtype, v[u]);
    } else {
      float scale = 1.f;
      if (p.pro == PE_PRO_ADD_RMSNORM) {
        // mean square of the updated residual over the whole row: every CTA computes it for itself (8 KB from
        // L2); CTA 0 also stores the updated residual for the launches that follow
        float ss = 0.f;
        for (int col = tid * 4; col < p.in_f; col += kRowThreads * 4) {
          float r[4];
          resid4(p, col, r);
          if (cta == 0 && p.resid_out)
            *reinterpret_cast<uint2*>(p.resid_out + col) = make_uint2(pack_half2(r[0], r[1]), pack_half2(r[2], r[3]));
          ss += r[0] * r[0] + r[1] * r[1] + r[2] * r[2] + r[3] * r[3];
        }
        ss = warp_sum(ss);
        if (lane == 0) pro_red[w] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < kRowWarps; ++i) tot += pro_red[i];
        scale = rsqrtf(tot / (float)p.in_f + p.eps);
      }
#pragma unroll
      for (int u = 0; u < CPW * BPC; ++u) {
        const bool on = u / BPC < cnt;
        const int col = (on ? (w + 16 * (u / BPC)) * BPC + (u % BPC) : 0) * kBlock + lane * 4;
        pro_load4(p, col, on, scale, v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < CPW * BPC; ++u) {
      if (u / BPC < cnt) {  // warp-uniform
        if (raw) warp_fwht128(v[u], lane);
        uint8_t* dst = xw + (u / BPC) * 512 + (u % BPC) * 256;
        if (PACKED) {  // pairs (k, k+64), in pair order
          float o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[u][i], 16);
          if (lane < 16)
            *reinterpret_cast<uint4*>(dst + lane * 16) = make_uint4(pack_half2(v[u][0], o[0]), pack_half2(v[u][1], o[1]),
                                                                    pack_half2(v[u][2], o[2]), pack_half2(v[u][3], o[3]));
        } else {
          *reinterpret_cast<uint2*>(dst + lane * 8) = make_uint2(pack_half2(v[u][0], v[u][1]), pack_half2(v[u][2], v[u][3]));
        }
      }
    }
    __syncwarp();
    const uint32_t xw_s = smem_u32(xw) + (PACKED ? (pc >> 2) * 256 + (pc & 3) * 64 : pc * 32);
#pragma unroll
    for (int j = 0; j < CPW; ++j) {
#pragma unroll
      for (int i = 0; i < kXPerChunk / 4; ++i) {
        uint4 t = make_uint4(0, 0, 0, 0);
        if (j < cnt) t = lds128(xw_s + j * 512 + i * 16);
        xr[j][4 * i + 0] = t.x; xr[j][4 * i + 1] = t.y; xr[j][4 * i + 2] = t.z; xr[j][4 * i + 3] = t.w;
      }
    }
  }
  if (!REGTAB) __syncthreads();  // the shared table has entries from every warp

  // ---- the item line, in passes of kPassRows rows
  const int n_warps_used = p.n_chunks < kRowWarps ? p.n_chunks : kRowWarps;
  const uint32_t norm_off = SUB * kItemBytes + rs * 4 + (PACKED ? (pc >> 2) * 2 : (w & 1) * 2);
  uint32_t st_rg = st_base;
  for (int rg0 = 0; rg0 < n_rg; rg0 += kPassRows / kGroupRows) {
    const int rg1 = n_rg < rg0 + kPassRows / kGroupRows ? n_rg : rg0 + kPassRows / kGroupRows;
    if (cnt > 0) {
      uint32_t part_s = smem_u32(part) + (rs * kPartStride + w) * 4;
      for (int rg = rg0; rg < rg1; ++rg) {
        const int rows_left = r_end - r_beg - kGroupRows * rg;  // sub-items beyond the CTA's rows were not fetched
        float acc[SUB];
#pragma unroll
        for (int sb = 0; sb < SUB; ++sb) acc[sb] = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
          asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
          const uint32_t st = st_rg + j * kColStage;
          if (j < cnt) {
#pragma unroll
            for (int sb = 0; sb < SUB; ++sb) {
              if (4 * sb < rows_left) {  // warp-uniform
                const uint4 q = lds128(st + sb * kItemBytes + q_off);
                unsigned short nh;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(nh) : "r"(st + norm_off + sb * 16));
                const float sdot = reg_dot<PACKED, REGTAB>(q, lane_base, tb, xr[j]);
                acc[sb] = fmaf(__half2float(__ushort_as_half(nh)), sdot, acc[sb]);
              }
            }
          }
          __syncwarp();  // every lane has read the slot before it is refilled
          fetch_item(st, j);
        }
        advance_fetch();
        st_rg += CPW * kColStage;
        if (st_rg == st_end) st_rg = st_base;
#pragma unroll
        for (int m = 1; m <= 4; m <<= 1) {
#pragma unroll
          for (int sb = 0; sb < SUB; ++sb) acc[sb] += __shfl_xor_sync(0xffffffffu, acc[sb], m);
        }
        if (pc == 0) {
#pragma unroll
          for (int sb = 0; sb < SUB; ++sb)
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(part_s + sb * (4 * kPartStride * 4)), "f"(acc[sb]) : "memory");
        }
        part_s += kGroupRows * kPartStride * 4;
      }
    }
    __syncthreads();
    for (int r = tid; r < kGroupRows * (rg1 - rg0); r += kRowThreads) {
      const int row = r_beg + kGroupRows * rg0 + r;
      if (row < r_end) {
        float s = 0.f;
        for (int ww = 0; ww < n_warps_used; ++ww) s += part[r * kPartStride + ww];
        if (p.bias) s += __half2float(p.bias[row]);
        store_from_float(p.y, p.y_dtype, row, s);
      }
    }
    if (rg1 < n_rg) __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <bool PACKED, bool REGTAB, int CPW>
static int launch_cols(const ColArgs& a, int G, cudaStream_t st) {
  // Sub-items (4 rows each) per step = independent decode-multiply chains per lane.  Byte codes, whose
  // every weight is a table lookup of its own, gain from four (measured 0.3 us per launch on the
  // 4096-wide layers); nibble codes are as fast or faster with two and need fewer registers.
  constexpr int SUB = (!PACKED && CPW <= 3) ? 4 : 2;
  // items in flight per warp: 6 to 8 KB of codes
  constexpr int DEPTH = SUB == 4 ? (CPW == 3 ? 3 : 4) : (CPW == 4 ? 8 : 6);
  const unsigned dyn_bytes = (REGTAB ? 0u : (unsigned)kLutBytes) + kRowWarps * CPW * 512u + kPassRows * kPartStride * 4u +
                             kRowWarps * DEPTH * (unsigned)col_stage_bytes(SUB);
  auto kfn = gemv_cols_kernel<PACKED, REGTAB, CPW, DEPTH, SUB>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_bytes));
    if (dev < 16) configured[dev] = true;
  }
  PE_CUDA_TRY(launch_pdl(kfn, dim3(G), dim3(kRowThreads), dyn_bytes, st, a));
  return PE_OK;
}

template <bool PACKED, bool REGTAB>
static int launch_cols_cpw(const ColArgs& a, int cpw, int G, cudaStream_t st) {
  switch (cpw) {
    case 1: return launch_cols<PACKED, REGTAB, 1>(a, G, st);
    case 2: return launch_cols<PACKED, REGTAB, 2>(a, G, st);
    case 3: return launch_cols<PACKED, REGTAB, 3>(a, G, st);
    case 4: return launch_cols<PACKED, REGTAB, 4>(a, G, st);
    default: return 1;
  }
}

struct ProArgs { int pro; const void* delta; int delta_dtype; const void* norm_w; void* resid_out; float eps; };

// batch 1: returns 1 if the shape is not this kernel's kind
static int gemv_cols_try(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                         const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int in_f, void* y,
                         int y_dtype, const void* bias, int out_f, int K, int sms, cudaStream_t stream,
                         const ProArgs* pro = nullptr) {
  const int64_t row_bytes = packed ? K / 2 : K;
  // norms are copied 4 bytes (two blocks) at a time: rows of norms must start 4-byte aligned and hold an even count
  if (row_bytes % 128 || (ld_norms & 1) || ((K / kBlock) & 1) || (reinterpret_cast<uintptr_t>(norms) & 3)) return 1;
  const int n_chunks = (int)(row_bytes / 128);
  const int cpw = (n_chunks + kRowWarps - 1) / kRowWarps;
  if (cpw > 4) return 1;
  // Small matrices (tensor-parallel shards) are latency bound: as many CTAs as there are groups of 8 rows, up to
  // one per SM.  Below 128 KB of codes the tile kernel's split along K spreads the few bytes better.
  const int G = out_f / 8 < sms ? out_f / 8 : sms;
  if (G < 1 || (long long)out_f * row_bytes < 131072) return 1;
  ColArgs a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const uint8_t*>(norms); a.ld_norms = ld_norms * 2;
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.x = x; a.x_kind = x_kind; a.x_dtype = x_dtype; a.in_f = in_f;
  a.y = y; a.y_dtype = y_dtype;
  a.bias = static_cast<const __half*>(bias);
  a.N = out_f; a.K = K; a.n_chunks = n_chunks;
  a.pro = pro ? pro->pro : PE_PRO_NONE;
  a.delta = pro ? pro->delta : nullptr; a.delta_dtype = pro ? pro->delta_dtype : PE_F16;
  a.norm_w = pro ? static_cast<const __half*>(pro->norm_w) : nullptr;
  a.resid_out = pro ? static_cast<__half*>(pro->resid_out) : nullptr;
  a.eps = pro ? pro->eps : 0.f;
  if (packed && n_levels <= 8) return launch_cols_cpw<true, true>(a, cpw, G, stream);
  if (packed) return launch_cols_cpw<true, false>(a, cpw, G, stream);
  return launch_cols_cpw<false, false>(a, cpw, G, stream);
}

template <bool PACKED, bool REGTAB, int NBATCH, int DEPTH>
static int launch_rows(const RowArgs& a, int G, unsigned dyn_bytes, cudaStream_t st) {
  auto kfn = gemv_rows_kernel<PACKED, REGTAB, NBATCH, DEPTH>;
  static thread_local unsigned configured[16] = {0};
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || configured[dev] < dyn_bytes) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_bytes));
    if (dev < 16) configured[dev] = dyn_bytes;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(kRowThreads);
  cfg.dynamicSmemBytes = dyn_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  PE_CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, a));
  return PE_OK;
}

template <bool PACKED, bool REGTAB, int NBATCH>
static int launch_rows_depth(const RowArgs& a, int G, unsigned fixed, cudaStream_t st) {
  const unsigned deep = fixed + kRowWarps * 12u * kRowStage, shallow = fixed + kRowWarps * 8u * kRowStage;
  if (deep <= 231424u) return launch_rows<PACKED, REGTAB, NBATCH, 12>(a, G, deep, st);
  if (shallow <= 231424u) return launch_rows<PACKED, REGTAB, NBATCH, 8>(a, G, shallow, st);
  return 1;
}

int gemv_rows_try(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                  const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f,
                  void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f, int in_f_padded,
                  int* status, cudaStream_t stream) {
  if (batch > 2 || !codes || !norms) return 1;
  const int K = in_f_padded, nb = K / kBlock;
  if (batch == 1) {
    const int n_sms = sm_count();
    if (n_sms <= 0) return PE_ERR_CUDA;
    const int r = gemv_cols_try(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, x_kind, x_dtype, in_f, y,
                                y_dtype, bias, out_f, K, n_sms, stream);
    if (r <= 0) return r;
  }
  const int64_t row_bytes = packed ? K / 2 : K;
  if (row_bytes % kItemBytes || ld_codes != row_bytes || ld_norms != nb) return 1;
  if (reinterpret_cast<uintptr_t>(norms) & 15) return 1;
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  const int cpr = (int)(row_bytes / kItemBytes);
  const int G = out_f < sms ? out_f : sms;
  if ((long long)out_f * cpr < (long long)G * kRowWarps * 4) return 1;  // too little work per warp: tile kernel
  if ((long long)out_f * cpr >= (1ll << 31)) return 1;

  RowArgs a;
  a.codes = static_cast<const uint8_t*>(codes);
  a.norms = static_cast<const uint8_t*>(norms);
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.x = x; a.x_kind = x_kind; a.x_dtype = x_dtype; a.ld_x = ld_x; a.in_f = in_f;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = static_cast<const __half*>(bias);
  a.batch = batch; a.N = out_f; a.K = K; a.nb = nb; a.cpr = cpr;
  const bool regtab = packed && n_levels <= 8;
  const unsigned fixed = (regtab ? 0u : (unsigned)kLutBytes) + (unsigned)batch * (unsigned)K * 2u;
  if (packed) {
    if (regtab) return batch == 1 ? launch_rows_depth<true, true, 1>(a, G, fixed, stream)
                                  : launch_rows_depth<true, true, 2>(a, G, fixed, stream);
    return batch == 1 ? launch_rows_depth<true, false, 1>(a, G, fixed, stream)
                      : launch_rows_depth<true, false, 2>(a, G, fixed, stream);
  }
  return batch == 1 ? launch_rows_depth<false, false, 1>(a, G, fixed, stream)
                    : launch_rows_depth<false, false, 2>(a, G, fixed, stream);
}

}  // namespace pe

// ---- batch-1 matmul with the glue op in front of it computed while the input is staged ----
extern "C" int pe_gemv_pro(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                           const float* ct_scaled, int n_levels, int prologue, const void* x, int in_f, const void* delta,
                           int delta_dtype, const void* norm_weight, void* resid_out, float eps, void* y, int y_dtype,
                           const void* bias, int out_f, int in_f_padded, void* stream) {
  using namespace pe;
  if (!codes || !norms || !ct_scaled || !x || !y) return PE_ERR_ARG;
  if (prologue != PE_PRO_ADD_RMSNORM && prologue != PE_PRO_SILU_MUL) return PE_ERR_ARG;
  if (prologue == PE_PRO_ADD_RMSNORM && (!norm_weight || (delta && delta_dtype != PE_F16 && delta_dtype != PE_F32))) return PE_ERR_ARG;
  if (out_f < 1 || in_f < 4 || in_f > in_f_padded || y_dtype < PE_F32 || y_dtype > PE_BF16) return PE_ERR_ARG;
  if (n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (in_f_padded % kBlock || in_f % 4) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15)) return PE_ERR_ALIGN;
  // the prologue reads its operands 8 or 16 bytes at a time
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(norm_weight) |
       reinterpret_cast<uintptr_t>(resid_out)) & 15)
    return PE_ERR_ALIGN;
  if (prologue == PE_PRO_SILU_MUL && (in_f % 8)) return PE_ERR_SHAPE;  // the `up` half starts in_f elements in: keep it 16-byte aligned
  if (ld_codes < (packed ? in_f_padded / 2 : in_f_padded) || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  ProArgs pro = {prologue, delta, delta_dtype, norm_weight, resid_out, eps};
  const int r = gemv_cols_try(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, PE_X_RAW, PE_F16, in_f, y, y_dtype,
                              bias, out_f, in_f_padded, sms, static_cast<cudaStream_t>(stream), &pro);
  return r == 1 ? PE_ERR_SHAPE : r;  // shapes the column-owner kernel does not take: the caller runs the separate launches
}

