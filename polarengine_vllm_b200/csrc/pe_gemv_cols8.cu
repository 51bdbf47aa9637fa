// Column-owner matmul for 3..8 activation rows (small decode batches) on the row-major layout.
//
//   y[m, r] = sum_blk norm[r, blk] * sum_k ct[code[r, blk, k]] * xt[m, blk, k]   (+ bias[r])
//
// Same ownership as the one-token kernel in pe_gemv_rows.cu: a CTA owns a contiguous range of weight rows,
// warp w of 16 owns the 128-byte column chunks w, w+16, ... of those rows and keeps the rotated activations of
// its chunks in registers, per-lane asynchronous copies fill a ring of items in shared memory, and the warps'
// column partials meet in shared memory and are summed in warp order (bit-reproducible).  What changes is the
// inner product: an item is 16 weight rows x 128 bytes and runs on the tensor cores as mma.sync m16n8k16 with
// the decoded WEIGHTS as the 16-row A operand and the (up to) 8 activation rows as the 8 columns of B, so a
// decoded weight is used for every token of the batch at once.  Lane (g, t) = (lane / 4, lane % 4) decodes rows
// g and g + 8 (A fragment) and holds, for token g, the activations of the k-slots t (B fragment); the product
// leaves rows g, g + 8 x tokens 2t, 2t+1 in its accumulator registers, which is exactly what the lane scales by
// the rows' block norms and adds up.  A k-slot of the instruction is only a label: the same (t, register)
// position means the same weight index in A and in B, whatever index that is, so nibble pairs (k, k + 64) and
// consecutive byte codes both map without any shuffling.
//
// Rows of an item are stored rotated by their parity (64 bytes for nibble codes, 16 for byte codes), so that the
// 16-byte pieces the lanes of a quarter warp load (two rows, four pieces each) fall into different banks.
#include "pe_gemv_decode.cuh"

namespace pe {

constexpr int kC8Warps = 16;
constexpr int kC8Threads = kC8Warps * 32;
constexpr int kC8Rows = 16;                        // weight rows of an item = rows of the MMA
constexpr int kC8Slot = kC8Rows * 128 + 128;       // codes, then 4 bytes of norms per row, rounded to a line
constexpr int kC8PartStride = kC8Warps + 1;
constexpr int kC8ScratchBytes = 2048;              // per warp: one rotated block of 8 tokens (fp16)
// Rows whose column partials are summed at a time.  Between two sums every warp must finish its items of the pass, so
// short passes turn the ring's run-ahead into waiting at the barrier (32-row passes: 26 us on a layer that takes 16
// for one token); the partial array [row][token][warp] is what limits them.
__host__ __device__ constexpr int c8_pass_rows(bool regtab) { return regtab ? 128 : 96; }
__host__ __device__ constexpr int c8_part_bytes(bool regtab) { return c8_pass_rows(regtab) * 8 * kC8PartStride * 4; }

struct Col8Args {
  const uint8_t* codes; int64_t ld_codes;  // bytes
  const uint8_t* norms; int64_t ld_norms;  // bytes between rows of fp16 norms
  const float* ct; int n_levels;
  const void* x; int x_kind; int x_dtype; int64_t ld_x; int in_f;
  void* y; int y_dtype; int64_t ld_y;
  const __half* bias;
  int batch, N, K, n_chunks;
};

__device__ __forceinline__ void c8_cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void c8_mma(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes of codes of rows g (q0) and g + 8 (q1) against the lane's matching activation registers.
//  nibble codes: a decoded byte is the A pair (w_i, w_i+64) of its row, x[i] the B pair of the same i: 8 products
//  byte codes:   a decoded word is two A pairs (w_k, w_k+1), (w_k+2, w_k+3): 4 products per 16 bytes
template <bool PACKED, bool REGTAB>
__device__ __forceinline__ void c8_piece(const uint4& q0, const uint4& q1, uint32_t lane_base, const RegTable& tb,
                                         const uint32_t* x, float d0[4], float d1[4]) {
  const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w}, w1[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t a[4], b[4];
    decode_word<PACKED, REGTAB>(w0[k], lane_base, tb, a);
    decode_word<PACKED, REGTAB>(w1[k], lane_base, tb, b);
    if (PACKED) {
      c8_mma(d0, a[0], b[0], a[1], b[1], x[4 * k], x[4 * k + 1]);
      c8_mma(d1, a[2], b[2], a[3], b[3], x[4 * k + 2], x[4 * k + 3]);
    } else {
      c8_mma((k & 1) ? d1 : d0, a[0], b[0], a[1], b[1], x[2 * k], x[2 * k + 1]);
    }
  }
}

template <bool PACKED, bool REGTAB, int CPW, int DEPTH>
__global__ void __launch_bounds__(kC8Threads, 1) gemv_cols8_kernel(const Col8Args p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int g = lane >> 2, t = lane & 3;     // MMA fragment coordinates
  const int rs = lane >> 3, pc = lane & 7;   // copy coordinates: row (mod 4) and 16-byte piece
  const int G = gridDim.x, cta = blockIdx.x;
  constexpr int kX = PACKED ? 32 : 16;       // activation registers per chunk
  constexpr int kPassRows = c8_pass_rows(REGTAB);
  constexpr int kRot = PACKED ? 4 : 1;       // pieces by which odd rows are rotated

  const int r_beg = (int)((long long)p.N * cta / G), r_end = (int)((long long)p.N * (cta + 1) / G);
  const int n_rg = (r_end - r_beg + kC8Rows - 1) / kC8Rows;
  int cnt = (p.n_chunks - w + kC8Warps - 1) / kC8Warps;  // chunks w, w+16, ... of this warp
  cnt = cnt < 0 ? 0 : (cnt > CPW ? CPW : cnt);

  asm volatile("griddepcontrol.launch_dependents;");

  // shared memory: [table 32 KB unless REGTAB][partials; the rotation scratch of the prologue lies inside][ring]
  static_assert(kC8Warps * kC8ScratchBytes <= c8_part_bytes(REGTAB), "the scratch fits the partial array");
  uint8_t* lut_g = smem;
  uint8_t* scratch = smem + (REGTAB ? 0 : kLutBytes) + (size_t)w * kC8ScratchBytes;
  float* part = reinterpret_cast<float*>(smem + (REGTAB ? 0 : kLutBytes));
  const uint32_t st_base = smem_u32(reinterpret_cast<uint8_t*>(part) + c8_part_bytes(REGTAB) + (size_t)w * (DEPTH * kC8Slot));

  // ---- code stream: items in the order the math takes them (row group, then chunk slot).  Running pointers: lane
  // (rs, pc) copies piece pc of rows rs, rs+4, rs+8, rs+12 of the item; the rotation of a row depends on rs only.
  const uint8_t* cptr_f = p.codes + (int64_t)(r_beg + rs) * p.ld_codes + (size_t)w * 128 + pc * 16;
  const uint8_t* nptr_f = p.norms + (int64_t)(r_beg + (lane & (kC8Rows - 1))) * p.ld_norms + (PACKED ? (size_t)w * 4 : (size_t)(w & ~1) * 2);
  const int64_t csub = 4 * p.ld_codes, cstep = kC8Rows * p.ld_codes, nstep = kC8Rows * p.ld_norms;
  const uint32_t dst_lane = rs * 128 + (((pc + (rs & 1) * kRot) & 7) << 4);
  constexpr int kNormStep = PACKED ? 64 : 32;  // norm bytes between this warp's chunks
  int rg_f = 0, row_f = r_beg + rs;            // row group being fetched; this lane's first row in it
  uint32_t st_f = st_base;
  const uint32_t st_end = st_base + DEPTH * kC8Slot;
  // one row group = CPW items, one copy group each (empty for slots the warp does not have or beyond the rows)
  auto fetch_group = [&]() {
#pragma unroll
    for (int j = 0; j < CPW; ++j) {
      if (j < cnt && rg_f < n_rg) {
#pragma unroll
        for (int sb = 0; sb < 4; ++sb)
          if (row_f + 4 * sb < r_end) cp_async16(st_f + dst_lane + sb * 512, cptr_f + sb * csub + j * 2048);
        if (lane < kC8Rows && row_f - rs + lane < r_end) c8_cp_async4(st_f + kC8Rows * 128 + lane * 4, nptr_f + j * kNormStep);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      st_f += kC8Slot;
      if (st_f == st_end) st_f = st_base;
    }
    ++rg_f;
    cptr_f += cstep;
    nptr_f += nstep;
    row_f += kC8Rows;
  };
  static_assert(DEPTH % CPW == 0 && CPW <= 2, "the ring holds whole row groups of one or two items");
#pragma unroll
  for (int d = 0; d < DEPTH / CPW; ++d) fetch_group();

  // ---- centroid table (needs nothing from the previous kernel)
  RegTable tb = {0, 0, 0, 0};
  if (PACKED && REGTAB) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hb = __half_as_ushort(__float2half_rn(i < p.n_levels ? p.ct[i] : 0.f));
      if (i < 4) { tb.lo0 |= (hb & 0xff) << (8 * i); tb.hi0 |= (hb >> 8) << (8 * i); }
      else { tb.lo1 |= (hb & 0xff) << (8 * (i - 4)); tb.hi1 |= (hb >> 8) << (8 * (i - 4)); }
    }
  } else {
    for (int e = w; e < (PACKED ? 256 : p.n_levels); e += kC8Warps) {
      uint32_t v;
      if (PACKED) {
        const int lo = e & 15, hi = e >> 4;
        v = pack_half2(lo < p.n_levels ? p.ct[lo] : 0.f, hi < p.n_levels ? p.ct[hi] : 0.f);
      } else {
        v = pack_half2(p.ct[e], p.ct[e]);
      }
      *reinterpret_cast<uint32_t*>(lut_g + e * 128 + lane * 4) = v;
    }
  }
  const uint32_t lane_base = smem_u32(lut_g) + lane * 4;

  // ---- activations of one chunk -> this lane's B registers: rotate block by block (8 tokens each), bounce
  // through the warp's scratch ([token][256 bytes]; nibble layers in (k, k+64) pair order)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const bool raw = p.x_kind == PE_X_RAW;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && (p.ld_x % 4 == 0);
  const int limit = raw ? p.in_f : p.K;
  uint32_t xr[CPW][kX];
  auto stage_x = [&](int j, uint32_t* dst) {
    constexpr int BPC = PACKED ? 2 : 1;
    const int chunk = w + kC8Warps * j;
#pragma unroll
    for (int b = 0; b < BPC; ++b) {
      const int col = (chunk * BPC + b) * kBlock + lane * 4;
      Raw4 r4[8];
#pragma unroll
      for (int tok = 0; tok < 8; ++tok) r4[tok] = load4_raw(p.x, p.x_dtype, (int64_t)tok * p.ld_x, col, tok < p.batch ? limit : 0, vec_ok);
#pragma unroll
      for (int tok = 0; tok < 8; ++tok) {
        float v[4];
        cvt4(r4[tok], p.x_dtype, v);
        if (raw) warp_fwht128(v, lane);
        if (PACKED) {
          float o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[i], 16);
          if (lane < 16)
            *reinterpret_cast<uint4*>(scratch + tok * 256 + lane * 16) =
                make_uint4(pack_half2(v[0], o[0]), pack_half2(v[1], o[1]), pack_half2(v[2], o[2]), pack_half2(v[3], o[3]));
        } else {
          *reinterpret_cast<uint2*>(scratch + tok * 256 + lane * 8) = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
        }
      }
      __syncwarp();
      const uint32_t src = smem_u32(scratch) + g * 256 + t * 64;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 u = lds128(src + i * 16);
        dst[b * 16 + 4 * i + 0] = u.x; dst[b * 16 + 4 * i + 1] = u.y; dst[b * 16 + 4 * i + 2] = u.z; dst[b * 16 + 4 * i + 3] = u.w;
      }
      __syncwarp();
    }
  };
#pragma unroll
  for (int j = 0; j < CPW; ++j) {
    if (j < cnt) stage_x(j, xr[j]);
    else {
#pragma unroll
      for (int i = 0; i < kX; ++i) xr[j][i] = 0;
    }
  }
  __syncthreads();  // the shared table has entries from every warp; the scratch becomes the partial array

  // ---- one item: 16 rows x this chunk -> acc (rows g, g+8 x tokens 2t, 2t+1)
  const int n_warps_used = p.n_chunks < kC8Warps ? p.n_chunks : kC8Warps;
  const uint32_t row_off = g * 128, rot = (g & 1) * kRot;
  auto do_item = [&](uint32_t st, const uint32_t* x, float acc[4]) {
    uint32_t n0, n1;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(n0) : "r"(st + kC8Rows * 128 + g * 4));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(n1) : "r"(st + kC8Rows * 128 + g * 4 + 32));
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&n0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&n1));
    if (PACKED) {
      const uint32_t a_off = st + row_off + (((t + rot) & 7) << 4), b_off = st + row_off + (((4 + t + rot) & 7) << 4);
      const uint4 qa0 = lds128(a_off), qa1 = lds128(a_off + 1024), qb0 = lds128(b_off), qb1 = lds128(b_off + 1024);
      float da0[4] = {0.f, 0.f, 0.f, 0.f}, da1[4] = {0.f, 0.f, 0.f, 0.f}, db0[4] = {0.f, 0.f, 0.f, 0.f}, db1[4] = {0.f, 0.f, 0.f, 0.f};
      c8_piece<true, REGTAB>(qa0, qa1, lane_base, tb, x, da0, da1);
      c8_piece<true, REGTAB>(qb0, qb1, lane_base, tb, x + 16, db0, db1);
      acc[0] = fmaf(f0.x, da0[0] + da1[0], fmaf(f0.y, db0[0] + db1[0], acc[0]));
      acc[1] = fmaf(f0.x, da0[1] + da1[1], fmaf(f0.y, db0[1] + db1[1], acc[1]));
      acc[2] = fmaf(f1.x, da0[2] + da1[2], fmaf(f1.y, db0[2] + db1[2], acc[2]));
      acc[3] = fmaf(f1.x, da0[3] + da1[3], fmaf(f1.y, db0[3] + db1[3], acc[3]));
    } else {
      const uint32_t a_off = st + row_off + (((2 * t + rot) & 7) << 4), b_off = st + row_off + (((2 * t + 1 + rot) & 7) << 4);
      const uint4 qa0 = lds128(a_off), qa1 = lds128(a_off + 1024), qb0 = lds128(b_off), qb1 = lds128(b_off + 1024);
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
      c8_piece<false, false>(qa0, qa1, lane_base, tb, x, d0, d1);
      c8_piece<false, false>(qb0, qb1, lane_base, tb, x + 8, d0, d1);
      const float ng = (w & 1) ? f0.y : f0.x, ng8 = (w & 1) ? f1.y : f1.x;  // chunk w + 16 j has the parity of w
      acc[0] = fmaf(ng, d0[0] + d1[0], acc[0]);
      acc[1] = fmaf(ng, d0[1] + d1[1], acc[1]);
      acc[2] = fmaf(ng8, d0[2] + d1[2], acc[2]);
      acc[3] = fmaf(ng8, d0[3] + d1[3], acc[3]);
    }
  };
  // rows g, g+8 of row group `rg_in_pass` x tokens 2t, 2t+1 -> the warp's column of the partial array
  auto put_part = [&](int rg_in_pass, const float acc[4]) {
    const int rl = rg_in_pass * kC8Rows + g;
    float* dst = part + ((rl * 8 + 2 * t) * kC8PartStride + w);
    dst[0] = acc[0];
    dst[kC8PartStride] = acc[1];
    dst[8 * 8 * kC8PartStride] = acc[2];
    dst[8 * 8 * kC8PartStride + kC8PartStride] = acc[3];
  };
  // sum of the warps' columns for the rows [row0, row0 + 32) of the CTA, bias, store
  auto reduce_pass = [&](int row0) {
    for (int i = tid; i < kPassRows * 8; i += kC8Threads) {
      const int tok = i / kPassRows, rl = i - tok * kPassRows;  // consecutive threads, consecutive rows of one token
      const int row = row0 + rl;
      if (row < r_end && tok < p.batch) {
        const float* src = part + (rl * 8 + tok) * kC8PartStride;
        float s = 0.f;
        for (int ww = 0; ww < n_warps_used; ++ww) s += src[ww];
        if (p.bias) s += __half2float(p.bias[row]);
        store_from_float(p.y, p.y_dtype, (int64_t)tok * p.ld_y + row, s);
      }
    }
  };

  uint32_t st_c = st_base;  // slot of the item being computed
  for (int rg0 = 0; rg0 < n_rg; rg0 += kPassRows / kC8Rows) {
#pragma unroll 1
    for (int rp = 0; rp < kPassRows / kC8Rows; ++rp) {
      if (rg0 + rp >= n_rg) break;  // CTA-uniform
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < CPW; ++j) {
        // the group's j-th item is the (j+1)-th oldest copy group in flight
        if (j == 0) asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
        else asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 2) : "memory");
        __syncwarp();
        if (j < cnt) do_item(st_c + j * kC8Slot, xr[j], acc);
      }
      __syncwarp();  // every lane has read the group's slots before they are refilled
      fetch_group();
      st_c += CPW * kC8Slot;
      if (st_c == st_end) st_c = st_base;
      if (cnt > 0) put_part(rp, acc);
    }
    __syncthreads();
    reduce_pass(r_beg + rg0 * kC8Rows);
    if (rg0 + kPassRows / kC8Rows < n_rg) __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <bool PACKED, bool REGTAB, int CPW>
static int launch_cols8(const Col8Args& a, int G, cudaStream_t st) {
  constexpr int DEPTH = 4;  // 8 KB of codes in flight per warp
  const unsigned dyn_bytes = (REGTAB ? 0u : (unsigned)kLutBytes) + (unsigned)c8_part_bytes(REGTAB) + kC8Warps * DEPTH * (unsigned)kC8Slot;
  auto kfn = gemv_cols8_kernel<PACKED, REGTAB, CPW, DEPTH>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_bytes));
    if (dev < 16) configured[dev] = true;
  }
  PE_CUDA_TRY(launch_pdl(kfn, dim3(G), dim3(kC8Threads), dyn_bytes, st, a));
  return PE_OK;
}

// Does the kernel take a layer?  Its chunks' activations for 8 tokens must fit the registers: one chunk of nibble
// codes (K <= 4096) or two of byte codes (K <= 4096) per warp.  (A form that walks the chunks one after the other
// for K = 12288 spent its time rotating activations -- 48 blocks per warp for 6 items -- and was no faster than the
// tile kernel.)
static int cols8_form(int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, int out_f, int K, int sms, int* cpw_out,
                      int* grid_out) {
  const int64_t row_bytes = packed ? K / 2 : K;
  if (row_bytes % 128 || ld_codes < row_bytes || (ld_norms & 1) || ((K / kBlock) & 1) || (reinterpret_cast<uintptr_t>(norms) & 3)) return 0;
  const int n_chunks = (int)(row_bytes / 128);
  const int cpw = (n_chunks + kC8Warps - 1) / kC8Warps;
  if (out_f < kC8Rows || (long long)out_f * row_bytes < 131072) return 0;
  const int G = out_f / kC8Rows < sms ? out_f / kC8Rows : sms;
  *cpw_out = cpw;
  *grid_out = G;
  return ((packed && cpw == 1) || (!packed && cpw <= 2)) ? 1 : 0;
}

// batch 3..8 on the row-major layout: returns 1 if the shape is not this kernel's kind
int gemv_cols8_try(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, const float* ct_scaled,
                   int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f, void* y, int y_dtype,
                   int64_t ld_y, const void* bias, int batch, int out_f, int in_f_padded, cudaStream_t stream) {
  if (batch < 3 || batch > 8 || !codes || !norms) return 1;
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  int cpw = 0, G = 0;
  const int form = cols8_form(packed, ld_codes, norms, ld_norms, out_f, in_f_padded, sms, &cpw, &G);
  if (form == 0) return 1;
  Col8Args a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const uint8_t*>(norms); a.ld_norms = ld_norms * 2;
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.x = x; a.x_kind = x_kind; a.x_dtype = x_dtype; a.ld_x = ld_x; a.in_f = in_f;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = static_cast<const __half*>(bias);
  a.batch = batch; a.N = out_f; a.K = in_f_padded;
  a.n_chunks = (int)((packed ? in_f_padded / 2 : in_f_padded) / 128);
  const bool regtab = packed && n_levels <= 8;
  if (packed) return regtab ? launch_cols8<true, true, 1>(a, G, stream) : launch_cols8<true, false, 1>(a, G, stream);
  return cpw == 1 ? launch_cols8<false, false, 1>(a, G, stream) : launch_cols8<false, false, 2>(a, G, stream);
}

bool gemv_cols8_takes(int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, int out_f, int in_f_padded) {
  const int sms = sm_count();
  if (sms <= 0) return false;
  int cpw = 0, G = 0;
  return cols8_form(packed, ld_codes, norms, ld_norms, out_f, in_f_padded, sms, &cpw, &G) != 0;
}

}  // namespace pe
