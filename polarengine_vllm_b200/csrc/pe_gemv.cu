// Decode-size quantized matmul (1..16 activation rows) for sm_100a: the tile kernel.
//
//   y[m, r] = sum_blk norm[r, blk] * sum_k ct[code[r, blk, k]] * xt[m, blk, k]   (+ bias[r])
//
// One and two activation rows over whole-row shapes go to the row-owner kernels in
// pe_gemv_rows.cu (gemv_run tries them first); everything else runs here.  The operand
// that costs anything is the code stream (0.5 or 1 byte per weight, read once from HBM):
//
//  * One persistent CTA per SM, 16 warps.  The unit of work is a "step": one 16-row
//    tile of the weight matrix times one 128-wide quantization block (1 KB of nibble
//    codes, 2 KB of byte codes).  Steps are numbered (row-tile-of-256, block, warp) and
//    the number line is cut into equal contiguous ranges, one per CTA, so every SM
//    streams the same number of bytes whatever the layer shape is.
//  * Codes travel by 16-byte asynchronous copies into a lane-private shared-memory ring
//    (8 KB per warp in flight), from the row-major arrays or from the tiled copy
//    (pe_retile: the step's codes followed by its 16 block norms, contiguous).
//  * Centroids are looked up in a shared-memory table that is replicated per lane
//    (entry e of lane l lives at table + e*128 + l*4), so 32 lanes with 32 different
//    codes never collide on a bank; the address is a byte extract and a multiply-add.
//    Nibble-packed layers use a 256-entry table indexed by the whole byte whose entry is
//    the fp16 pair (ct[lo], ct[hi]) = two weights per lookup; layers with at most eight
//    levels use a register table and byte permutes instead (no memory traffic).
//  * The dot products run on the tensor cores (mma.sync m16n8k16, fp16 in, fp32 out):
//    weights are the 16x16 A tile, up to 8 (or 2x8) activation rows are the B tile.
//    The k index of the MMA is a free permutation, so a lookup result is used as it
//    comes: for nibble layers the pair (k, k+64) of the half-block layout is one A
//    register and the activations are staged in shared memory in the same pairing.
//    One or two activation rows use fp16x2 FMAs instead (seven eighths of an MMA would be
//    padding).
//  * The block norm multiplies the 8-MMA partial sum of a block, not each weight.
//  * Activations are staged per CTA into shared memory once: either already rotated
//    (fp32, the reference's x_transformed) or raw fp16/bf16/fp32, in which case the
//    zero-pad and the FWHT-128 happen in the staging warps (one launch per layer).
//  * Split-K falls out of the range cut: a row tile whose blocks are spread over
//    several CTAs gets one fp32 partial per CTA in scratch memory; the CTA that owns the
//    tile's last step sums the partials in CTA order (bounded wait on a counter), adds
//    the bias, converts and stores.  No float atomics: results are bit-identical from
//    run to run.  The counters return to zero, so the scratch is reusable.
#include "pe_gemv_decode.cuh"

namespace pe {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kRowsPerCta = kWarps * 16;  // 256
constexpr int kXRowBytes = 320;           // 256 B of activations + 64 B pad (bank spread)

struct GemvArgs {
  const uint8_t* codes; int64_t ld_codes;   // row-major layout (the reference's)
  const __half* norms; int64_t ld_norms;
  const uint8_t* tiles;                     // tiled layout (pe_retile), used when TILED
  const float* ct; int n_levels;
  const void* x; int x_kind; int x_dtype; int64_t ld_x; int in_f;
  void* y; int y_dtype; int64_t ld_y;
  const __half* bias;
  int batch, N, K, nb;
  int n_rt16, n_rt256;
  int S;             // total steps = n_rt256 * nb * 16 (S * grid < 2^31)
  int cap;           // activation slots resident in shared memory per phase
  int max_slots;     // scratch partials per 16-row tile
  float* ws_part; unsigned* ws_cnt; int* ws_status;
  unsigned dyn_bytes;
  // grouped launch (blockIdx.y = problem): several matrices of one shape -- the experts of
  // a mixture layer -- each against its own few activation rows
  const int* x_rows;          // activation row m of the problem is row x_rows[m] of x (nullptr: row m)
  const int4* grp;            // per problem: (matrix index, first row of its rows in the row list / output, rows, -)
  int64_t grp_codes_stride, grp_norms_stride;  // bytes / halves between consecutive matrices
  size_t grp_ws_stride, grp_cnt_bytes;         // partial block and counter block per problem
};

__device__ __forceinline__ int64_t x_row_of(const GemvArgs& p, int m) { return p.x_rows ? (int64_t)p.x_rows[m] : (int64_t)m; }

__device__ __forceinline__ void mma16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Step-line arithmetic.  The host guarantees S * G < 2^31, so 32-bit division is exact.
__device__ __forceinline__ int range_start(int S, int G, int c) { return (int)((unsigned)S * (unsigned)c / (unsigned)G); }
__device__ __forceinline__ int owner_of(int S, int G, int idx) { return (int)(((unsigned)(idx + 1) * (unsigned)G - 1u) / (unsigned)S); }
__device__ __forceinline__ int ceil_div16(int v) { return v <= 0 ? 0 : (v + 15) >> 4; }

// block-step range [q_lo, q_hi) of warp w inside the CTA range [s, e), clipped to [cl, ch)
__device__ __forceinline__ void warp_q_range(int s, int e, int w, int cl, int ch, int& q_lo, int& q_hi) {
  q_lo = ceil_div16(s - w);
  q_hi = ceil_div16(e - w);
  if (q_lo < cl) q_lo = cl;
  if (q_hi > ch) q_hi = ch;
  if (q_hi < q_lo) q_hi = q_lo;
}

template <bool PACKED>
struct CodeRegs {
  uint4 a0, b0;  // rows g and g+8
  uint4 a1, b1;  // second 16 B (byte codes only)
};

// Tiled layout (pe_retile): the codes of one step -- 16 rows x one 128-block -- are 1 KB
// (2 KB for byte codes) of contiguous memory followed by the 16 fp16 block norms, and the
// steps of a row tile follow each other, so a warp streams one contiguous region.
template <bool PACKED> struct TileGeom {
  static constexpr int kCodeBytes = PACKED ? 1024 : 2048;
  static constexpr int kTileBytes = kCodeBytes + 32;            // + 16 norms
  static constexpr int kStageBytes = (kTileBytes + 63) & ~63;   // ring stage stride
};

// Request one step's codes (rows g and g+8 of a 16-row tile, one 128-block) into this
// warp's ring stage: 16-byte asynchronous copies, no registers held while the data is in
// flight.  Row-major source: stage layout [piece 0..(1|3)][lane] x 16 B (lane (g,t) copies
// its own 16-byte pieces of rows g and g+8).  Tiled source: the stage is a copy of the tile.
template <bool PACKED, bool TILED>
__device__ __forceinline__ void fetch(uint32_t stage, const GemvArgs& p, int rt256, int b, int w, int g, int t, int lane) {
  if (TILED) {
    int rt16 = rt256 * 16 + w;
    rt16 = rt16 < p.n_rt16 ? rt16 : p.n_rt16 - 1;
    const uint8_t* src = p.tiles + ((int64_t)rt16 * p.nb + b) * TileGeom<PACKED>::kTileBytes + lane * 16;
    const uint32_t dst = stage + lane * 16;
#pragma unroll
    for (int i = 0; i < TileGeom<PACKED>::kCodeBytes / 512; ++i) cp_async16(dst + 512 * i, src + 512 * i);
    if (lane < 2) cp_async16(dst + TileGeom<PACKED>::kCodeBytes, src + TileGeom<PACKED>::kCodeBytes);  // norms
    return;
  }
  int rowA = rt256 * kRowsPerCta + w * 16 + g;
  int rowB = rowA + 8;
  rowA = rowA < p.N ? rowA : p.N - 1;
  rowB = rowB < p.N ? rowB : p.N - 1;
  const uint32_t dst = stage + lane * 16;
  if (PACKED) {
    cp_async16(dst, p.codes + (int64_t)rowA * p.ld_codes + b * 64 + t * 16);
    cp_async16(dst + 512, p.codes + (int64_t)rowB * p.ld_codes + b * 64 + t * 16);
  } else {
    const uint8_t* pa = p.codes + (int64_t)rowA * p.ld_codes + b * 128 + t * 32;
    const uint8_t* pb = p.codes + (int64_t)rowB * p.ld_codes + b * 128 + t * 32;
    cp_async16(dst, pa);
    cp_async16(dst + 512, pb);
    cp_async16(dst + 1024, pa + 16);
    cp_async16(dst + 1536, pb + 16);
  }
}

template <bool PACKED, bool TILED>
__device__ __forceinline__ void read_stage(CodeRegs<PACKED>& r, const uint8_t* stage, int lane, int g, int t) {
  if (TILED && !PACKED) {  // rows of 128 B: lane (g,t) owns bytes [32 t, 32 t + 32) of rows g and g+8
    const uint4* ra = reinterpret_cast<const uint4*>(stage + g * 128 + t * 32);
    const uint4* rb = reinterpret_cast<const uint4*>(stage + (g + 8) * 128 + t * 32);
    r.a0 = ra[0]; r.a1 = ra[1];
    r.b0 = rb[0]; r.b1 = rb[1];
    return;
  }
  const uint4* s4 = reinterpret_cast<const uint4*>(stage) + lane;  // tiled nibble rows are 64 B: same addresses
  r.a0 = s4[0];
  r.b0 = s4[32];
  if (!PACKED) { r.a1 = s4[64]; r.b1 = s4[96]; }
}

// Four MMAs (16 rows x 64 k) from two code words of row g (wa) and of row g+8 (wb).
// All 16 table addresses are formed first, then the 16 lookups are issued back to back,
// then the MMAs alternate between two accumulator sets so that none waits on its
// predecessor.
//  PACKED: word i holds bytes for MMAs 2i (bytes 0,1) and 2i+1 (bytes 2,3).
//  !PACKED: the caller passes four words per row; word i is MMA i (codes 0,1 | 2,3).
template <bool PACKED, int NB, bool REGTAB>
__device__ __forceinline__ void quad_mma(float d0[NB / 2], float d1[NB / 2], const uint32_t* wa, const uint32_t* wb,
                                         uint32_t lane_base, const RegTable& tb, const uint4& xa, const uint4& xb,
                                         const uint4& ya, const uint4& yb) {
  uint32_t ad[16], v[16];
  if (PACKED && REGTAB) {
    uint32_t a0[4], b0[4], a1[4], b1[4];  // bytes 0..3 of wa[0], wb[0], wa[1], wb[1]
    reg_decode(wa[0], tb, a0);
    reg_decode(wb[0], tb, b0);
    reg_decode(wa[1], tb, a1);
    reg_decode(wb[1], tb, b1);
    mma16816(d0, a0[0], b0[0], a0[1], b0[1], xa.x, xa.y);
    mma16816(d1, a0[2], b0[2], a0[3], b0[3], xa.z, xa.w);
    mma16816(d0, a1[0], b1[0], a1[1], b1[1], xb.x, xb.y);
    mma16816(d1, a1[2], b1[2], a1[3], b1[3], xb.z, xb.w);
    if (NB == 16) {
      mma16816(d0 + 4, a0[0], b0[0], a0[1], b0[1], ya.x, ya.y);
      mma16816(d1 + 4, a0[2], b0[2], a0[3], b0[3], ya.z, ya.w);
      mma16816(d0 + 4, a1[0], b1[0], a1[1], b1[1], yb.x, yb.y);
      mma16816(d1 + 4, a1[2], b1[2], a1[3], b1[3], yb.z, yb.w);
    }
  } else if (PACKED) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ad[8 * i + 0] = lut_addr<0>(wa[i], lane_base);
      ad[8 * i + 1] = lut_addr<0>(wb[i], lane_base);
      ad[8 * i + 2] = lut_addr<1>(wa[i], lane_base);
      ad[8 * i + 3] = lut_addr<1>(wb[i], lane_base);
      ad[8 * i + 4] = lut_addr<2>(wa[i], lane_base);
      ad[8 * i + 5] = lut_addr<2>(wb[i], lane_base);
      ad[8 * i + 6] = lut_addr<3>(wa[i], lane_base);
      ad[8 * i + 7] = lut_addr<3>(wb[i], lane_base);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = lut_ld(ad[i]);
    mma16816(d0, v[0], v[1], v[2], v[3], xa.x, xa.y);
    mma16816(d1, v[4], v[5], v[6], v[7], xa.z, xa.w);
    mma16816(d0, v[8], v[9], v[10], v[11], xb.x, xb.y);
    mma16816(d1, v[12], v[13], v[14], v[15], xb.z, xb.w);
    if (NB == 16) {
      mma16816(d0 + 4, v[0], v[1], v[2], v[3], ya.x, ya.y);
      mma16816(d1 + 4, v[4], v[5], v[6], v[7], ya.z, ya.w);
      mma16816(d0 + 4, v[8], v[9], v[10], v[11], yb.x, yb.y);
      mma16816(d1 + 4, v[12], v[13], v[14], v[15], yb.z, yb.w);
    }
  } else {
    // two MMAs at a time (16 lookups): words 0,1 then words 2,3
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t a = wa[2 * h + i], b = wb[2 * h + i];
        ad[8 * i + 0] = lut_addr<0>(a, lane_base);
        ad[8 * i + 1] = lut_addr<1>(a, lane_base);
        ad[8 * i + 2] = lut_addr<0>(b, lane_base);
        ad[8 * i + 3] = lut_addr<1>(b, lane_base);
        ad[8 * i + 4] = lut_addr<2>(a, lane_base);
        ad[8 * i + 5] = lut_addr<3>(a, lane_base);
        ad[8 * i + 6] = lut_addr<2>(b, lane_base);
        ad[8 * i + 7] = lut_addr<3>(b, lane_base);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = lut_ld(ad[i]);
      const uint4& xx = h ? xb : xa;
      const uint4& yy = h ? yb : ya;
      const uint32_t p0 = lo_hi(v[0], v[1]), p1 = lo_hi(v[2], v[3]), p2 = lo_hi(v[4], v[5]), p3 = lo_hi(v[6], v[7]);
      const uint32_t r0 = lo_hi(v[8], v[9]), r1 = lo_hi(v[10], v[11]), r2 = lo_hi(v[12], v[13]), r3 = lo_hi(v[14], v[15]);
      mma16816(d0, p0, p1, p2, p3, xx.x, xx.y);
      mma16816(d1, r0, r1, r2, r3, xx.z, xx.w);
      if (NB == 16) {
        mma16816(d0 + 4, p0, p1, p2, p3, yy.x, yy.y);
        mma16816(d1 + 4, r0, r1, r2, r3, yy.z, yy.w);
      }
    }
  }
}

template <bool PACKED, int NB, bool REGTAB>
__device__ __forceinline__ void step_math(float acc[NB / 2], const CodeRegs<PACKED>& r, uint32_t lane_base,
                                          const RegTable& tb, const uint8_t* xslot, float nA, float nB, int g, int t,
                                          int batch) {
  // activation fragments of this block: 4 x 16 B per 8 rows of batch.  Lanes whose batch
  // row does not exist skip the load (their MMA columns are never read), which also
  // shrinks the shared-memory transaction to the quarter-warps that hold live rows.
  uint4 xf[4], yf[4];
  const uint8_t* xrow = xslot + g * kXRowBytes + t * 16;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    xf[j] = make_uint4(0, 0, 0, 0);
    yf[j] = make_uint4(0, 0, 0, 0);
  }
  if (g < batch) {
#pragma unroll
    for (int j = 0; j < 4; ++j) xf[j] = *reinterpret_cast<const uint4*>(xrow + j * 64);
  }
  if (NB == 16 && g + 8 < batch) {
#pragma unroll
    for (int j = 0; j < 4; ++j) yf[j] = *reinterpret_cast<const uint4*>(xrow + 8 * kXRowBytes + j * 64);
  }
  float d0[NB / 2], d1[NB / 2];
#pragma unroll
  for (int i = 0; i < NB / 2; ++i) d0[i] = d1[i] = 0.f;
  if (PACKED) {
    const uint32_t wa[4] = {r.a0.x, r.a0.y, r.a0.z, r.a0.w};
    const uint32_t wb[4] = {r.b0.x, r.b0.y, r.b0.z, r.b0.w};
    quad_mma<true, NB, REGTAB>(d0, d1, wa, wb, lane_base, tb, xf[0], xf[1], yf[0], yf[1]);
    quad_mma<true, NB, REGTAB>(d0, d1, wa + 2, wb + 2, lane_base, tb, xf[2], xf[3], yf[2], yf[3]);
  } else {
    const uint32_t wa[8] = {r.a0.x, r.a0.y, r.a0.z, r.a0.w, r.a1.x, r.a1.y, r.a1.z, r.a1.w};
    const uint32_t wb[8] = {r.b0.x, r.b0.y, r.b0.z, r.b0.w, r.b1.x, r.b1.y, r.b1.z, r.b1.w};
    quad_mma<false, NB, false>(d0, d1, wa, wb, lane_base, tb, xf[0], xf[1], yf[0], yf[1]);
    quad_mma<false, NB, false>(d0, d1, wa + 4, wb + 4, lane_base, tb, xf[2], xf[3], yf[2], yf[3]);
  }
  acc[0] = fmaf(nA, d0[0] + d1[0], acc[0]);
  acc[1] = fmaf(nA, d0[1] + d1[1], acc[1]);
  acc[2] = fmaf(nB, d0[2] + d1[2], acc[2]);
  acc[3] = fmaf(nB, d0[3] + d1[3], acc[3]);
  if (NB == 16) {
    acc[4] = fmaf(nA, d0[4] + d1[4], acc[4]);
    acc[5] = fmaf(nA, d0[5] + d1[5], acc[5]);
    acc[6] = fmaf(nB, d0[6] + d1[6], acc[6]);
    acc[7] = fmaf(nB, d0[7] + d1[7], acc[7]);
  }
}

// ---- one or two activation rows: no tensor cores --------------------------------
// With a single activation row seven eighths of every m16n8k16 MMA is padding, and the
// legacy mma.sync path retires only one such MMA per 8 cycles per scheduler: at eight
// MMAs per step it, not memory, bounds the stream.  For batch <= 2 the products go through
// the fp16x2 FMA pipe instead: a lane keeps the dot products of ITS 32 (64) weights of rows
// g and g+8 against its own slice of the activations -- two fp16x2 chains of 8 per row and
// block, widened to fp32 and scaled by the block norm -- and the four lanes of a row are
// summed once per tile, at hand-off time.
// A registers (fp16 pairs in activation order) of chunk j (16 bytes of activations) for rows g (a) and g+8 (b)
template <bool PACKED, bool REGTAB>
__device__ __forceinline__ void decode_chunk(const CodeRegs<PACKED>& r, int j, uint32_t lane_base, const RegTable& tb,
                                             uint32_t a[4], uint32_t b[4]) {
  if (PACKED) {
    const uint32_t wa = j == 0 ? r.a0.x : (j == 1 ? r.a0.y : (j == 2 ? r.a0.z : r.a0.w));
    const uint32_t wb = j == 0 ? r.b0.x : (j == 1 ? r.b0.y : (j == 2 ? r.b0.z : r.b0.w));
    if (REGTAB) {
      reg_decode(wa, tb, a);
      reg_decode(wb, tb, b);
    } else {
      const uint32_t ad[8] = {lut_addr<0>(wa, lane_base), lut_addr<1>(wa, lane_base), lut_addr<2>(wa, lane_base),
                              lut_addr<3>(wa, lane_base), lut_addr<0>(wb, lane_base), lut_addr<1>(wb, lane_base),
                              lut_addr<2>(wb, lane_base), lut_addr<3>(wb, lane_base)};
#pragma unroll
      for (int k = 0; k < 4; ++k) { a[k] = lut_ld(ad[k]); b[k] = lut_ld(ad[4 + k]); }
    }
  } else {
    const uint4 qa = j < 2 ? r.a0 : r.a1, qb = j < 2 ? r.b0 : r.b1;
    const uint32_t wa0 = (j & 1) ? qa.z : qa.x, wa1 = (j & 1) ? qa.w : qa.y;
    const uint32_t wb0 = (j & 1) ? qb.z : qb.x, wb1 = (j & 1) ? qb.w : qb.y;
    uint32_t ad[16], v[16];
    ad[0] = lut_addr<0>(wa0, lane_base); ad[1] = lut_addr<1>(wa0, lane_base);
    ad[2] = lut_addr<2>(wa0, lane_base); ad[3] = lut_addr<3>(wa0, lane_base);
    ad[4] = lut_addr<0>(wa1, lane_base); ad[5] = lut_addr<1>(wa1, lane_base);
    ad[6] = lut_addr<2>(wa1, lane_base); ad[7] = lut_addr<3>(wa1, lane_base);
    ad[8] = lut_addr<0>(wb0, lane_base); ad[9] = lut_addr<1>(wb0, lane_base);
    ad[10] = lut_addr<2>(wb0, lane_base); ad[11] = lut_addr<3>(wb0, lane_base);
    ad[12] = lut_addr<0>(wb1, lane_base); ad[13] = lut_addr<1>(wb1, lane_base);
    ad[14] = lut_addr<2>(wb1, lane_base); ad[15] = lut_addr<3>(wb1, lane_base);
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = lut_ld(ad[k]);
#pragma unroll
    for (int k = 0; k < 4; ++k) { a[k] = lo_hi(v[2 * k], v[2 * k + 1]); b[k] = lo_hi(v[8 + 2 * k], v[9 + 2 * k]); }
  }
}

// acc[0] row g batch 0, acc[1] row g batch 1, acc[2] row g+8 batch 0, acc[3] row g+8 batch 1: per-lane partials
template <bool PACKED, bool REGTAB>
__device__ __forceinline__ void step_fma(float acc[4], const CodeRegs<PACKED>& r, uint32_t lane_base, const RegTable& tb,
                                         const uint8_t* xslot, float nA, float nB, int t, int batch) {
  uint4 x0[4], x1[4];
  const uint8_t* xrow = xslot + t * 16;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x0[j] = *reinterpret_cast<const uint4*>(xrow + j * 64);
    x1[j] = make_uint4(0, 0, 0, 0);
  }
  if (batch > 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x1[j] = *reinterpret_cast<const uint4*>(xrow + kXRowBytes + j * 64);
  }
  uint32_t cA0[2] = {0, 0}, cB0[2] = {0, 0}, cA1[2] = {0, 0}, cB1[2] = {0, 0};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t a[4], b[4];
    decode_chunk<PACKED, REGTAB>(r, j, lane_base, tb, a, b);
    const uint32_t xx[4] = {x0[j].x, x0[j].y, x0[j].z, x0[j].w};
    const uint32_t yy[4] = {x1[j].x, x1[j].y, x1[j].z, x1[j].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      cA0[j & 1] = hfma2_u(a[k], xx[k], cA0[j & 1]);
      cB0[j & 1] = hfma2_u(b[k], xx[k], cB0[j & 1]);
    }
    if (batch > 1) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        cA1[j & 1] = hfma2_u(a[k], yy[k], cA1[j & 1]);
        cB1[j & 1] = hfma2_u(b[k], yy[k], cB1[j & 1]);
      }
    }
  }
  acc[0] = fmaf(nA, h2sum(cA0[0]) + h2sum(cA0[1]), acc[0]);
  acc[2] = fmaf(nB, h2sum(cB0[0]) + h2sum(cB0[1]), acc[2]);
  if (batch > 1) {
    acc[1] = fmaf(nA, h2sum(cA1[0]) + h2sum(cA1[1]), acc[1]);
    acc[3] = fmaf(nB, h2sum(cB1[0]) + h2sum(cB1[1]), acc[3]);
  }
}

// sum the four lanes (t = 0..3) that share a weight row; afterwards every lane holds the
// totals in the accumulator layout the hand-off expects from lanes with t == 0
__device__ __forceinline__ void quad_reduce(const float in[4], float out[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float v = in[i];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    out[i] = v;
  }
}

// Final store of one element of a 16-row tile.
__device__ __forceinline__ void emit(const GemvArgs& p, int row, int m, float v) {
  if (row < p.N && m < p.batch) {
    if (p.bias) v += __half2float(p.bias[row]);
    store_from_float(p.y, p.y_dtype, (int64_t)m * p.ld_y + row, v);
  }
}

// Hand-off of one 16-row tile at the end of this CTA's share of it.  Every CTA whose range
// touches the tile's row-tile-of-256 leaves exactly one fp32 partial per warp (zeros if none
// of the tile's steps fell to this warp) and bumps the tile's counter with a release --
// fire and forget, nobody waits here.  The CTA that owns the tile's LAST step is its
// reducer: at the very end of the kernel (reduce_tile) it waits, bounded, for the count,
// sums the partials in CTA order (fixed, whatever the arrival order: bit-reproducible),
// adds the bias, converts, stores, and returns the counter to zero.  A tile owned by a
// single CTA is stored directly.  Returns true if this warp must reduce the tile later.
template <int NB>
__device__ __noinline__ bool flush(const GemvArgs& p, const float* acc, int rt256, int w, int G, int cta, int lane,
                                   int g, int t) {
  const int rt16 = rt256 * 16 + w;
  const int row0 = rt16 * 16;
  if (rt16 >= p.n_rt16) return false;
  const int span_lo = rt256 * p.nb * 16;
  const int c_first = owner_of(p.S, G, span_lo);
  const int c_last = owner_of(p.S, G, span_lo + p.nb * 16 - 1);
  if (c_last == c_first) {
#pragma unroll
    for (int h = 0; h < NB / 8; ++h) {
      emit(p, row0 + g, 8 * h + 2 * t, acc[4 * h + 0]);
      emit(p, row0 + g, 8 * h + 2 * t + 1, acc[4 * h + 1]);
      emit(p, row0 + g + 8, 8 * h + 2 * t, acc[4 * h + 2]);
      emit(p, row0 + g + 8, 8 * h + 2 * t + 1, acc[4 * h + 3]);
    }
    return false;
  }
  const int tile_elems = 16 * p.batch;
  float* mine = p.ws_part + ((int64_t)rt16 * p.max_slots + (cta - c_first)) * tile_elems;
#pragma unroll
  for (int h = 0; h < NB / 8; ++h) {
    const int m0 = 8 * h + 2 * t;
    if (m0 < p.batch) { mine[m0 * 16 + g] = acc[4 * h + 0]; mine[m0 * 16 + g + 8] = acc[4 * h + 2]; }
    if (m0 + 1 < p.batch) { mine[(m0 + 1) * 16 + g] = acc[4 * h + 1]; mine[(m0 + 1) * 16 + g + 8] = acc[4 * h + 3]; }
  }
  __syncwarp();  // orders the lanes' stores before lane 0's release
  if (lane == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.ws_cnt + rt16) : "memory");
  return cta == c_last;
}

// The reducer's half of the hand-off (see flush).  The wait is bounded: if the count does
// not arrive the tile is left unwritten and the scratch's status word is set.
__device__ __noinline__ void reduce_tile(const GemvArgs& p, int rt256, int w, int G, int lane) {
  const int rt16 = rt256 * 16 + w;
  const int row0 = rt16 * 16;
  const int span_lo = rt256 * p.nb * 16;
  const int c_first = owner_of(p.S, G, span_lo);
  const int n_contrib = owner_of(p.S, G, span_lo + p.nb * 16 - 1) - c_first + 1;
  const int tile_elems = 16 * p.batch;
  const float* tile_ws = p.ws_part + (int64_t)rt16 * p.max_slots * tile_elems;
  int ok = 1;
  if (lane == 0) {
    unsigned seen = 0;
    const long long t0 = clock64();
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.ws_cnt + rt16) : "memory");
      if ((int)seen >= n_contrib) break;
      if (clock64() - t0 > (1ll << 30)) { ok = 0; break; }  // ~0.5 s: something is badly wrong
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) {
    if (lane == 0) atomicExch(p.ws_status, 1);
    return;
  }
  __syncwarp();  // lane 0's acquire happens before the other lanes' reads
  for (int e = lane; e < tile_elems; e += 32) {
    float s = 0.f;
    for (int c0 = 0; c0 < n_contrib; c0 += 8) {  // eight loads in flight, then eight adds in slot order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = c0 + u < n_contrib ? __ldcg(tile_ws + (c0 + u) * tile_elems + e) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    emit(p, row0 + (e & 15), e >> 4, s);
  }
  if (lane == 0) p.ws_cnt[rt16] = 0;
}

// Place one rotated 128-block (lane l holds elements 4l..4l+3) into its activation row.
template <bool PACKED>
__device__ __forceinline__ void place_block(uint8_t* row, const float v[4], int lane) {
  if (PACKED) {
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[i], 16);
    if (lane < 16) {  // pairs (k, k+64) for k = 4*lane..4*lane+3 = chunk `lane`
      const uint4 u = make_uint4(pack_half2(v[0], o[0]), pack_half2(v[1], o[1]), pack_half2(v[2], o[2]),
                                 pack_half2(v[3], o[3]));
      *reinterpret_cast<uint4*>(row + ((lane & 3) * 4 + (lane >> 2)) * 16) = u;
    }
  } else {  // halves 4*lane..4*lane+3 = half of chunk lane/2
    const int c = lane >> 1;
    const uint2 u = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
    *reinterpret_cast<uint2*>(row + ((c & 3) * 4 + (c >> 2)) * 16 + (lane & 1) * 8) = u;
  }
}

// Stage the activation slots of this phase into shared memory.  slot_blk[s] is the
// quantization block held by slot s.  Loads are issued in groups before any use so
// that a warp pays one memory latency per group, not one per item.
template <bool PACKED>
__device__ __noinline__ void stage_x(const GemvArgs& p, uint8_t* xs, const int* slot_blk, int cnt, int warp, int lane) {
  const int slot_bytes = p.batch * kXRowBytes;
  const bool vec_ok = (p.ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
  const int items = cnt * p.batch;
  if (p.x_kind == PE_X_RAW) {
    // one warp per (slot, activation row): load, pad, rotate, convert, place
    constexpr int U = 4;
    for (int base = warp; base < items; base += kWarps * U) {
      float v[U][4];
      Raw4 raw4[U];
      int sl[U], mm[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int item = base + u * kWarps;
        const bool on = item < items;
        sl[u] = on ? item / p.batch : 0;
        mm[u] = on ? item - sl[u] * p.batch : 0;
        raw4[u] = load4_raw(p.x, p.x_dtype, x_row_of(p, mm[u]) * p.ld_x, slot_blk[sl[u]] * kBlock + lane * 4, on ? p.in_f : 0, vec_ok);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) cvt4(raw4[u], p.x_dtype, v[u]);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (base + u * kWarps < items) {  // warp-uniform
          warp_fwht128(v[u], lane);
          place_block<PACKED>(xs + sl[u] * slot_bytes + mm[u] * kXRowBytes, v[u], lane);
        }
      }
    }
  } else {
    // already rotated: one thread per 16-byte chunk
    const int total = items * 16;
    constexpr int U = 2;
    for (int base = warp * 32 + lane; base < total; base += kThreads * U) {
      float a[U][4], b[U][4];
      Raw4 ra[U], rb[U];
      int dst[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int item = base + u * kThreads;
        const bool on = item < total;
        const int c = item & 15;
        const int sm = on ? item >> 4 : 0;
        const int sl = sm / p.batch, m = sm - sl * p.batch;
        const int col = slot_blk[sl] * kBlock;
        const int64_t row_off = x_row_of(p, m) * p.ld_x;
        const int lim = on ? p.K : 0;
        if (PACKED) {
          ra[u] = load4_raw(p.x, p.x_dtype, row_off, col + 4 * c, lim, vec_ok);
          rb[u] = load4_raw(p.x, p.x_dtype, row_off, col + 64 + 4 * c, lim, vec_ok);
        } else {
          ra[u] = load4_raw(p.x, p.x_dtype, row_off, col + 8 * c, lim, vec_ok);
          rb[u] = load4_raw(p.x, p.x_dtype, row_off, col + 8 * c + 4, lim, vec_ok);
        }
        dst[u] = on ? sl * slot_bytes + m * kXRowBytes + ((c & 3) * 4 + (c >> 2)) * 16 : -1;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        cvt4(ra[u], p.x_dtype, a[u]);
        cvt4(rb[u], p.x_dtype, b[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (dst[u] >= 0) {
          uint4 r;
          if (PACKED)
            r = make_uint4(pack_half2(a[u][0], b[u][0]), pack_half2(a[u][1], b[u][1]), pack_half2(a[u][2], b[u][2]),
                           pack_half2(a[u][3], b[u][3]));
          else
            r = make_uint4(pack_half2(a[u][0], a[u][1]), pack_half2(a[u][2], a[u][3]), pack_half2(b[u][0], b[u][1]),
                           pack_half2(b[u][2], b[u][3]));
          *reinterpret_cast<uint4*>(xs + dst[u]) = r;
        }
      }
    }
  }
}

// Stage the block norms of this phase: ns[row][slot], row stride nstr halves.  Thread
// (row = idx / 32, slot = idx % 32): lanes walk the blocks of one weight row (adjacent
// in memory); all 16 loads of a thread are in flight together.
__device__ __noinline__ void stage_norms(const GemvArgs& p, __half* ns, int nstr, const int* slot_rt, const int* slot_blk, int cnt,
                            int tid) {
  constexpr int U = kRowsPerCta * 32 / kThreads;  // 16
  const int s = tid & 31;
  const bool on = s < cnt;
  const int rt = on ? slot_rt[s] : 0, blk = on ? slot_blk[s] : 0;
  unsigned short v[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int row = (tid >> 5) + u * kWarps;
    const int grow = rt * kRowsPerCta + row;
    v[u] = (on && grow < p.N) ? __ldg(reinterpret_cast<const unsigned short*>(p.norms) + (int64_t)grow * p.ld_norms + blk)
                              : (unsigned short)0;
  }
  if (on) {
#pragma unroll
    for (int u = 0; u < U; ++u) reinterpret_cast<unsigned short*>(ns)[((tid >> 5) + u * kWarps) * nstr + s] = v[u];
  }
}

template <bool PACKED, int NB, int DEPTH, bool REGTAB, bool FMA, bool TILED, bool GROUPED = false>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvArgs pin) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int slot_rt[32], slot_blk[32];
  __shared__ GemvArgs grp_args;
  if (GROUPED) {
    // this CTA's problem: patch a copy of the arguments (matrix, rows, output, scratch).  The problem list
    // is written by the launch before this one (pe_moe_plan), so it is read only after the dependency wait;
    // a grouped launch therefore overlaps nothing with its predecessor but its own start-up.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int4 d = pin.grp[blockIdx.y];
    if (d.z <= 0) return;  // unused problem slot
    if (threadIdx.x == 0) {
      GemvArgs t = pin;
      t.codes += (int64_t)d.x * pin.grp_codes_stride;
      t.norms += (int64_t)d.x * pin.grp_norms_stride;
      t.batch = d.z < NB ? d.z : NB;
      if (pin.x_rows) t.x_rows = pin.x_rows + d.y;
      else t.x = static_cast<const uint8_t*>(pin.x) + (int64_t)d.y * pin.ld_x * (pin.x_dtype == PE_F32 ? 4 : 2);
      t.y = static_cast<uint8_t*>(pin.y) + (int64_t)d.y * pin.ld_y * (pin.y_dtype == PE_F32 ? 4 : 2);
      // scratch: [counter zone: one counter block per problem][partials, one block per problem]
      uint8_t* cnt = reinterpret_cast<uint8_t*>(pin.ws_cnt) + (size_t)blockIdx.y * pin.grp_cnt_bytes;
      t.ws_cnt = reinterpret_cast<unsigned*>(cnt);
      t.ws_status = reinterpret_cast<int*>(cnt + pin.grp_cnt_bytes - 4);
      t.ws_part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(pin.ws_part) + (size_t)blockIdx.y * pin.grp_ws_stride);
      grp_args = t;
    }
    __syncthreads();
  }
  const GemvArgs& p = GROUPED ? grp_args : pin;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int G = gridDim.x, cta = blockIdx.x;

  // ---- this CTA's and this warp's share of the step line
  const int s_beg = range_start(p.S, G, cta), s_end = range_start(p.S, G, cta + 1);
  const int Q0 = s_beg >> 4, Q1 = (s_end + 15) >> 4;  // block-steps touched by the CTA
  int q_lo, q_hi;
  warp_q_range(s_beg, s_end, w, 0, p.n_rt256 * p.nb, q_lo, q_hi);

  // ---- everything the prologue needs from memory is requested here, before any of it
  // is used, so that the prologue costs one memory latency: codes, centroids, norms and
  // the first group of activations.
  int rt_c = q_lo / p.nb, b_c = q_lo - rt_c * p.nb;  // compute cursor
  int rt_f = rt_c, b_f = b_c, q_f = q_lo;            // fetch cursor (runs kDepth-1 steps ahead)
  // Programmatic dependent launch: this grid may have been started while the previous
  // kernel in the stream was still draining.  Weights, norms and centroids never change,
  // so they are requested right away; the activations and the scratch buffer belong to
  // the previous kernel until griddepcontrol.wait returns.
  asm volatile("griddepcontrol.launch_dependents;");
  // (volatile asm loads: the compiler must not sink them to their first use, which is
  // after the dependency wait)
  float ct_mine = 0.f;
  {
    const int e = PACKED ? (lane & 15) : (w + 16 * (lane & 15));
    if (e < p.n_levels) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(ct_mine) : "l"(p.ct + e));
  }

  const int cnt0 = (Q1 - Q0) < p.cap ? (Q1 - Q0) : p.cap;
  // slot `lane` of the first phase
  const int my_q = Q0 + lane;
  const int my_rt = my_q / p.nb, my_blk = my_q - my_rt * p.nb;
  constexpr int NU = kRowsPerCta * 32 / kThreads;  // norm loads per thread (16)
  unsigned short nv[NU];
#pragma unroll
  for (int u = 0; u < NU; ++u) {
    const int grow = my_rt * kRowsPerCta + w + u * kWarps;
    nv[u] = 0;
    if (!TILED && lane < cnt0 && grow < p.N)
      asm volatile("ld.global.nc.u16 %0, [%1];"
                   : "=h"(nv[u])
                   : "l"(reinterpret_cast<const unsigned short*>(p.norms) + (int64_t)grow * p.ld_norms + my_blk));
  }
  // first activation item of this warp (raw input): slot = item / batch, row = item % batch
  const int slot_bytes = p.batch * kXRowBytes;
  const bool vec_ok = (p.ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
  const int items0 = cnt0 * p.batch;
  float xv[4];
  Raw4 xraw = {{0u, 0u, 0u, 0u}};
  int x_sl = 0, x_m = 0;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (p.x_kind == PE_X_RAW) {
    const bool on = w < items0;
    x_sl = on ? w / p.batch : 0;
    x_m = on ? w - x_sl * p.batch : 0;
    const int qq = Q0 + x_sl;
    xraw = load4_raw(p.x, p.x_dtype, x_row_of(p, x_m) * p.ld_x, (qq % p.nb) * kBlock + lane * 4, on ? p.in_f : 0, vec_ok);
  }

  // ---- shared memory: [table 32 KB][activation slots][norms][code ring 16 x 8 KB]
  uint8_t* lut_g = smem;
  const uint32_t lut_s = smem_u32(smem);
  uint8_t* xs = lut_g + kLutBytes;
  const int nstr = p.cap + 2;
  __half* ns = reinterpret_cast<__half*>(xs + (size_t)p.cap * slot_bytes);
  constexpr int kCodeBytes = PACKED ? 1024 : 2048;  // bytes of one step's codes per warp
  constexpr int kStage = TILED ? TileGeom<PACKED>::kStageBytes : kCodeBytes;
  constexpr int kDepth = DEPTH;                     // ring stages per warp
  uint8_t* ring_g = reinterpret_cast<uint8_t*>(ns) + (TILED ? 0 : ((kRowsPerCta * nstr * 2 + 15) & ~15)) + w * (kDepth * kStage);
  const uint32_t ring_s = smem_u32(ring_g);
  int i_f = 0;  // steps requested so far
  // the code stream goes last: it is the bulk, and whatever is requested after it
  // would queue behind megabytes of it in the memory system.  The ring is filled and
  // refilled kBatch steps at a time: consecutive steps of a warp are consecutive 64-byte
  // (128-byte) pieces of the same 16 rows, so requesting them together gives the DRAM
  // controller 256 contiguous bytes per row instead of one burst per row activation.
  constexpr int kBatch = 1;  // steps per refill (larger batches measured slower: fewer bytes in flight)
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    if (q_f < q_hi) {
      fetch<PACKED, TILED>(ring_s + (i_f % kDepth) * kStage, p, rt_f, b_f, w, g, t, lane);
      if (++b_f == p.nb) { b_f = 0; ++rt_f; }
      ++q_f;
      ++i_f;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  if (lane < cnt0 && w == 0) { slot_rt[lane] = my_rt; slot_blk[lane] = my_blk; }

  // ---- centroid table, replicated per lane.  Warp w writes entries w, w+16, ...; the
  // levels came with one load per lane and travel by shuffle.
  if (PACKED && REGTAB) {
    // no shared table: the centroids live in registers (below)
  } else if (PACKED) {
    const float lo = __shfl_sync(0xffffffffu, ct_mine, w);  // entry e = w + 16 i: low nibble w, high nibble i
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
  const uint32_t lane_base = lut_s + lane * 4;
  RegTable tb = {0, 0, 0, 0};
  if (PACKED && REGTAB) {  // fp16 bits of ct[0..7], split into low-byte and high-byte tables
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hb = __half_as_ushort(__float2half_rn(__shfl_sync(0xffffffffu, ct_mine, i)));
      if (i < 4) { tb.lo0 |= (hb & 0xff) << (8 * i); tb.hi0 |= (hb >> 8) << (8 * i); }
      else { tb.lo1 |= (hb & 0xff) << (8 * (i - 4)); tb.hi1 |= (hb >> 8) << (8 * (i - 4)); }
    }
  }
  if (!TILED && lane < cnt0) {
#pragma unroll
    for (int u = 0; u < NU; ++u) reinterpret_cast<unsigned short*>(ns)[(w + u * kWarps) * nstr + lane] = nv[u];
  }
  if (p.x_kind == PE_X_RAW) {
    if (w < items0) {
      cvt4(xraw, p.x_dtype, xv);
      warp_fwht128(xv, lane);
      place_block<PACKED>(xs + x_sl * slot_bytes + x_m * kXRowBytes, xv, lane);
    }
    if (items0 > kWarps) {  // more than one item per warp: the rest, in groups
      __syncthreads();      // slot table visible
      stage_x<PACKED>(p, xs, slot_blk, cnt0, w + kWarps, lane);
    }
  } else {
    __syncthreads();
    stage_x<PACKED>(p, xs, slot_blk, cnt0, w, lane);
  }

  float acc[NB / 2];
#pragma unroll
  for (int i = 0; i < NB / 2; ++i) acc[i] = 0.f;
  int run = 0;  // blocks accumulated for the current row tile
  float zeros[NB / 2];
#pragma unroll
  for (int i = 0; i < NB / 2; ++i) zeros[i] = 0.f;
  const int span = p.nb * 16;
  int pending = -1;                                                   // tile this warp must reduce at the end
  int next_flush = s_beg / span;                                      // first row-tile-of-256 the CTA touches
  const int last_tile = s_end > s_beg ? (s_end - 1) / span : next_flush - 1;  // last one

  int q = q_lo;
  bool first_phase = true;
  __syncwarp();
  for (int ph = Q0; ph < Q1; ph += p.cap) {
    const int cnt = (Q1 - ph) < p.cap ? (Q1 - ph) : p.cap;
    const int ph_end = ph + cnt;
    if (!first_phase) {
      __syncthreads();  // everyone done with the previous slots
      if (tid < cnt) {
        const int qq = ph + tid, r = qq / p.nb;
        slot_rt[tid] = r;
        slot_blk[tid] = qq - r * p.nb;
      }
      __syncthreads();
      if (!TILED) stage_norms(p, ns, nstr, slot_rt, slot_blk, cnt, tid);
      stage_x<PACKED>(p, xs, slot_blk, cnt, w, lane);
    }
    __syncthreads();
    first_phase = false;
    const int q_stop = q_hi < ph_end ? q_hi : ph_end;
    while (q < q_stop) {
      {
        {
          // Groups are committed one per step, kDepth up front and kBatch more after every
          // kBatch-th step, so step i's group is complete once at most
          // kDepth - 1 - (i % kBatch) younger groups are pending.
          const int i_step = q - q_lo;
          switch (i_step % kBatch) {
            case 0: asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory"); break;
            case 1: asm volatile("cp.async.wait_group %0;" ::"n"(kDepth > 2 ? kDepth - 2 : 0) : "memory"); break;
            case 2: asm volatile("cp.async.wait_group %0;" ::"n"(kDepth > 3 ? kDepth - 3 : 0) : "memory"); break;
            default: asm volatile("cp.async.wait_group %0;" ::"n"(kDepth > 4 ? kDepth - 4 : 0) : "memory"); break;
          }
          CodeRegs<PACKED> cur;
          const uint8_t* stage_g = ring_g + (i_step % kDepth) * kStage;
          read_stage<PACKED, TILED>(cur, stage_g, lane, g, t);
          float nA, nB;
          if (TILED) {  // the norms travelled with the codes
            nA = __half2float(*reinterpret_cast<const __half*>(stage_g + kCodeBytes + 2 * g));
            nB = __half2float(*reinterpret_cast<const __half*>(stage_g + kCodeBytes + 2 * g + 16));
          }
          const int slot = q - ph;
          if (!TILED) {
            nA = __half2float(ns[(w * 16 + g) * nstr + slot]);
            nB = __half2float(ns[(w * 16 + g + 8) * nstr + slot]);
          }
          if (FMA) step_fma<PACKED, REGTAB>(acc, cur, lane_base, tb, xs + slot * slot_bytes, nA, nB, t, p.batch);
          else step_math<PACKED, NB, REGTAB>(acc, cur, lane_base, tb, xs + slot * slot_bytes, nA, nB, g, t, p.batch);
          ++run;
          ++q;
          if (i_step % kBatch == kBatch - 1) {
            // the kBatch stages just consumed are free (their reads fed the math above)
#pragma unroll
            for (int d = 0; d < kBatch; ++d) {
              if (q_f < q_hi) {
                fetch<PACKED, TILED>(ring_s + (i_f % kDepth) * kStage, p, rt_f, b_f, w, g, t, lane);
                if (++b_f == p.nb) { b_f = 0; ++rt_f; }
                ++q_f;
                ++i_f;
              }
              asm volatile("cp.async.commit_group;" ::: "memory");
            }
          }
          if (++b_c == p.nb) {  // row tile finished on our side
            for (; next_flush < rt_c; ++next_flush)
              if (flush<NB>(p, zeros, next_flush, w, G, cta, lane, g, t)) pending = next_flush;
            if (FMA) {
              float red[NB / 2];
              quad_reduce(acc, red);
              if (flush<NB>(p, red, rt_c, w, G, cta, lane, g, t)) pending = rt_c;
            } else if (flush<NB>(p, acc, rt_c, w, G, cta, lane, g, t)) {
              pending = rt_c;
            }
            next_flush = rt_c + 1;
#pragma unroll
            for (int i = 0; i < NB / 2; ++i) acc[i] = 0.f;
            run = 0;
            b_c = 0;
            ++rt_c;
          }
        }
      }
    }
  }
  // every row-tile-of-256 this CTA's range touches gets a hand-off from every warp
  if (run > 0) {
    for (; next_flush < rt_c; ++next_flush)
      if (flush<NB>(p, zeros, next_flush, w, G, cta, lane, g, t)) pending = next_flush;
    if (FMA) {
      float red[NB / 2];
      quad_reduce(acc, red);
      if (flush<NB>(p, red, rt_c, w, G, cta, lane, g, t)) pending = rt_c;
    } else if (flush<NB>(p, acc, rt_c, w, G, cta, lane, g, t)) {
      pending = rt_c;
    }
    next_flush = rt_c + 1;
  }
  for (; next_flush <= last_tile; ++next_flush)
    if (flush<NB>(p, zeros, next_flush, w, G, cta, lane, g, t)) pending = next_flush;
  // A CTA owns the last step of at most one shared tile (only the first tile of its range
  // can have started in an earlier CTA and end here; later shared tiles end further on).
  if (pending >= 0) reduce_tile(p, pending, w, G, lane);
}

// ---- host side -----------------------------------------------------------------

static int pick_cap(int batch) { return batch <= 8 ? 32 : 16; }  // activation slots resident per phase (<= 80 KB)

// Scratch layout: [tile counters, fixed 256 KB][fp32 partials].  The counter region has
// the same size for every shape so that partials of one call can never land where a
// later call of another shape keeps its counters (counters must read zero on entry and
// are returned to zero; partials need no initial value).
constexpr size_t kCounterBytes = 262144;
constexpr int kMaxRowTiles = (int)(kCounterBytes / sizeof(unsigned)) - 1;  // last word: status (0 = ok)

struct Plan {
  int n_rt16, n_rt256, nb, G, cap, max_slots;
  long long S;
  size_t part_bytes, cnt_bytes;
  unsigned fixed_bytes;        // shared memory besides the code ring
  unsigned fixed_bytes_tiled;  // same without the norm staging area
};

static Plan make_plan(int batch, int N, int K, int sms) {
  Plan pl;
  pl.nb = K / kBlock;
  pl.n_rt16 = (N + 15) / 16;
  pl.n_rt256 = (pl.n_rt16 + 15) / 16;
  pl.S = (long long)pl.n_rt256 * pl.nb * 16;
  long long g = pl.S / 16;
  pl.G = (int)(g < sms ? (g < 1 ? 1 : g) : sms);
  pl.cap = pick_cap(batch);
  // CTAs that can share one row tile of 256: its nb*16 steps over ranges of S/G steps
  long long per = pl.S / pl.G;
  pl.max_slots = (int)(((long long)pl.nb * 16 + per - 1) / per) + 1;
  if (pl.max_slots > pl.G) pl.max_slots = pl.G;
  pl.part_bytes = (size_t)pl.n_rt16 * pl.max_slots * 16 * batch * sizeof(float);
  pl.cnt_bytes = kCounterBytes;
  const unsigned slot_bytes = batch * kXRowBytes;
  pl.fixed_bytes = kLutBytes + pl.cap * slot_bytes + ((kRowsPerCta * (pl.cap + 2) * 2 + 15) & ~15) + 64;
  pl.fixed_bytes_tiled = kLutBytes + pl.cap * slot_bytes + 64;
  return pl;
}

// The scratch size is computed for the largest SM count this library supports so that
// it does not depend on the device.
static constexpr int kMaxSms = 256;

}  // namespace pe

using namespace pe;

extern "C" size_t pe_gemv_workspace_bytes(int batch, int out_f, int in_f_padded) {
  if (batch < 1 || batch > 16 || out_f < 1 || in_f_padded < kBlock || in_f_padded % kBlock) return 0;
  if ((out_f + 15) / 16 > kMaxRowTiles) return 0;
  size_t best = 0;
  // max_slots grows with the CTA count; take the bound at kMaxSms
  Plan pl = make_plan(batch, out_f, in_f_padded, kMaxSms);
  best = pl.cnt_bytes + pl.part_bytes;
  return best;
}

template <bool PACKED, int NB, int DEPTH, bool REGTAB, bool FMA, bool TILED, bool GROUPED = false>
static int launch_t(GemvArgs a, const Plan& pl, cudaStream_t st, int n_problems = 1) {
  const int G = pl.G;
  a.dyn_bytes = (TILED ? pl.fixed_bytes_tiled : pl.fixed_bytes) +
                kWarps * DEPTH * (TILED ? TileGeom<PACKED>::kStageBytes : (PACKED ? 1024 : 2048));
  if (a.dyn_bytes > 231424u) return PE_ERR_LIMIT;  // 227 KB minus the 1 KB of static shared memory
  auto kfn = gemv_kernel<PACKED, NB, DEPTH, REGTAB, FMA, TILED, GROUPED>;
  static thread_local unsigned configured[16] = {0};
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 16 && configured[dev] < a.dyn_bytes) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.dyn_bytes));
    configured[dev] = a.dyn_bytes;
  } else if (dev >= 16) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.dyn_bytes));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G, n_problems);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = a.dyn_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  PE_CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, a));
  return PE_OK;
}

template <bool PACKED, int NB, int DEPTH, bool REGTAB, bool FMA = false>
static int launch(const GemvArgs& a, const Plan& pl, cudaStream_t st) {
  return a.tiles ? launch_t<PACKED, NB, DEPTH, REGTAB, FMA, true>(a, pl, st)
                 : launch_t<PACKED, NB, DEPTH, REGTAB, FMA, false>(a, pl, st);
}

// Argument checks shared by every decode-size entry point.
static int gemv_check(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, const void* tiles,
                      const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f,
                      void* y, int y_dtype, int64_t ld_y, int batch, int out_f, int in_f_padded) {
  if (!ct_scaled || !x || !y) return PE_ERR_ARG;
  if (!tiles && (!codes || !norms)) return PE_ERR_ARG;
  if (batch < 1 || out_f < 1 || in_f < 1 || in_f > in_f_padded) return PE_ERR_ARG;
  if (x_kind != PE_X_ROTATED && x_kind != PE_X_RAW) return PE_ERR_ARG;
  if (x_dtype < PE_F32 || x_dtype > PE_BF16 || y_dtype < PE_F32 || y_dtype > PE_BF16) return PE_ERR_ARG;
  if (n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (batch > 16 || in_f_padded % kBlock) return PE_ERR_SHAPE;
  if (tiles) {
    if (reinterpret_cast<uintptr_t>(tiles) & 15) return PE_ERR_ALIGN;
  } else {
    if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15)) return PE_ERR_ALIGN;
    if (ld_codes < (packed ? in_f_padded / 2 : in_f_padded) || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  }
  if (ld_x < (x_kind == PE_X_RAW ? in_f : in_f_padded) || ld_y < out_f) return PE_ERR_ARG;
  return PE_OK;
}

// One or two activation rows over the row-major arrays: kernels that own whole weight rows and use no scratch
// (only the status word, when a workspace is given).  PE_OK after a launch, 1 if the shape is not theirs.
static int gemv_scratch_free(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                             const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
                             int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
                             int in_f_padded, void* workspace, void* stream) {
  int* status = workspace ? reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kCounterBytes - 4) : nullptr;
  return gemv_rows_try(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y, y_dtype,
                       ld_y, bias, batch, out_f, in_f_padded, status, static_cast<cudaStream_t>(stream));
}

// The tile kernel (any batch up to 16, either layout); arguments already checked.
static int gemv_tile_run(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                         const void* tiles, const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype,
                         int64_t ld_x, int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
                         int in_f_padded, void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return PE_ERR_ARG;
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  if (sms > kMaxSms || (out_f + 15) / 16 > kMaxRowTiles) return PE_ERR_LIMIT;
  if ((long long)((out_f + 255) / 256) * (in_f_padded / kBlock) * 16 >= (1ll << 31) / kMaxSms) return PE_ERR_LIMIT;
  Plan pl = make_plan(batch, out_f, in_f_padded, sms);
  if (workspace_bytes < pl.cnt_bytes + pl.part_bytes) return PE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return PE_ERR_ALIGN;

  GemvArgs a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const __half*>(norms); a.ld_norms = ld_norms;
  a.tiles = static_cast<const uint8_t*>(tiles);
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.x = x; a.x_kind = x_kind; a.x_dtype = x_dtype; a.ld_x = ld_x; a.in_f = in_f;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = static_cast<const __half*>(bias);
  a.batch = batch; a.N = out_f; a.K = in_f_padded; a.nb = pl.nb;
  a.n_rt16 = pl.n_rt16; a.n_rt256 = pl.n_rt256; a.S = (int)pl.S; a.cap = pl.cap; a.max_slots = pl.max_slots;
  a.ws_cnt = static_cast<unsigned*>(workspace);
  a.ws_status = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kCounterBytes - 4);
  a.ws_part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.cnt_bytes);
  // the deepest code ring that fits beside table, activation slots and norms
  const unsigned ring_need = kWarps * 8u * (tiles ? (unsigned)TileGeom<true>::kStageBytes : 1024u);
  const bool deep = (tiles ? pl.fixed_bytes_tiled : pl.fixed_bytes) + ring_need <= 231424u;
  a.x_rows = nullptr; a.grp = nullptr; a.grp_codes_stride = a.grp_norms_stride = 0; a.grp_ws_stride = a.grp_cnt_bytes = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // DEPTH = ring stages per warp (1 KB nibble / 2 KB byte stages): 8 KB per warp when it fits, else 6 / 4 KB
  if (batch <= 2) {  // one or two activation rows: fp16x2 FMA path, no tensor cores (always fits the deep ring)
    if (packed && n_levels <= 8) return launch<true, 8, 8, true, true>(a, pl, st);
    if (packed) return launch<true, 8, 8, false, true>(a, pl, st);
    return launch<false, 8, 4, false, true>(a, pl, st);
  }
  if (packed && n_levels <= 8) {  // 2- and 3-bit layers: centroid table in registers
    if (batch <= 8) return deep ? launch<true, 8, 8, true>(a, pl, st) : launch<true, 8, 6, true>(a, pl, st);
    return launch<true, 16, 6, true>(a, pl, st);
  }
  if (packed) {
    if (batch <= 8) return deep ? launch<true, 8, 8, false>(a, pl, st) : launch<true, 8, 6, false>(a, pl, st);
    return launch<true, 16, 6, false>(a, pl, st);
  }
  if (batch <= 8) return deep ? launch<false, 8, 4, false>(a, pl, st) : launch<false, 8, 2, false>(a, pl, st);
  return launch<false, 16, 2, false>(a, pl, st);
}

// Shared by pe_gemv (row-major codes + norms) and pe_gemv_tiled (tiles != nullptr).
static int gemv_run(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                    const void* tiles, const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype,
                    int64_t ld_x, int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
                    int in_f_padded, void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return PE_ERR_ARG;
  const int c = gemv_check(codes, packed, ld_codes, norms, ld_norms, tiles, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y,
                           y_dtype, ld_y, batch, out_f, in_f_padded);
  if (c != PE_OK) return c;
  if (!tiles && batch <= 2) {
    const int r = gemv_scratch_free(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f,
                                    y, y_dtype, ld_y, bias, batch, out_f, in_f_padded,
                                    workspace_bytes >= kCounterBytes ? workspace : nullptr, stream);
    if (r <= 0) return r;
  }
  if (!tiles && batch >= 3 && batch <= 8) {  // small batches on the row-major layout: column-owner kernel, no scratch
    const int r = gemv_cols8_try(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y,
                                 y_dtype, ld_y, bias, batch, out_f, in_f_padded, static_cast<cudaStream_t>(stream));
    if (r <= 0) return r;
  }
  return gemv_tile_run(codes, packed, ld_codes, norms, ld_norms, tiles, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y,
                       y_dtype, ld_y, bias, batch, out_f, in_f_padded, workspace, workspace_bytes, stream);
}

extern "C" int pe_gemv_small_batch_takes(int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, int out_f,
                                         int in_f_padded) {
  return gemv_cols8_takes(packed, ld_codes, norms, ld_norms, out_f, in_f_padded) ? 1 : 0;
}

extern "C" int pe_gemv(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                       const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
                       int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
                       int in_f_padded, void* workspace, size_t workspace_bytes, void* stream) {
  return gemv_run(codes, packed, ld_codes, norms, ld_norms, nullptr, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y,
                  y_dtype, ld_y, bias, batch, out_f, in_f_padded, workspace, workspace_bytes, stream);
}

// Reads a status word back (and optionally clears it): waits for the stream, no allocation.
static int read_status_word(int* word, int clear, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0;
  PE_CUDA_TRY(cudaMemcpyAsync(&v, word, sizeof(int), cudaMemcpyDeviceToHost, st));
  PE_CUDA_TRY(cudaStreamSynchronize(st));
  if (clear && v != 0) PE_CUDA_TRY(cudaMemsetAsync(word, 0, sizeof(int), st));
  return v < 0 ? 0 : v;
}

extern "C" int pe_gemv_status(void* workspace, size_t workspace_bytes, int clear, void* stream) {
  if (!workspace || workspace_bytes < kCounterBytes) return PE_ERR_ARG;
  return read_status_word(reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kCounterBytes - 4), clear, stream);
}

// ---- grouped launch: the experts of a mixture layer ------------------------------------
//
// `max_problems` problems of one shape share a launch (grid y).  Problem i is described on
// the device by (matrix index, first row, rows <= 16, 0): rows first .. first + rows - 1 of
// the row list `x_rows` (or of x itself when x_rows is NULL) times matrix `index` of a
// stack of matrices, written to the same rows of y.  Slots with rows <= 0 return at once,
// so the caller can size the launch for the worst case without knowing the routing.
namespace pe {
// The scratch starts with a counter zone of fixed size, whatever the shapes, so that the
// partials of one call can never land where a later call keeps counters (which must read
// zero on entry and are returned to zero).
constexpr size_t kGroupedCounterZone = 4u << 20;
static size_t grouped_cnt_bytes(int n_rt16) { return ((size_t)(n_rt16 + 1) * 4 + 255) & ~(size_t)255; }
static int grouped_ctas(int max_problems, long long S, int sms) {
  // one CTA per SM over all problems when there are few of them (a CTA fills an SM: a second wave of CTAs only
  // repeats the per-CTA set-up on half the bytes), about two per SM-slot otherwise (problems differ in size)
  long long g = (max_problems * 8 <= sms ? 1ll * sms : 2ll * sms) / max_problems;
  if (g < 1) g = 1;
  if (g > sms) g = sms;
  if (g > S / 16) g = S / 16 < 1 ? 1 : S / 16;
  return (int)g;
}
}  // namespace pe

extern "C" size_t pe_gemv_grouped_workspace_bytes(int max_problems, int out_f, int in_f_padded) {
  if (max_problems < 1 || out_f < 1 || in_f_padded < kBlock || in_f_padded % kBlock) return 0;
  const long long S = (long long)((out_f + 255) / 256) * (in_f_padded / kBlock) * 16;
  const Plan pl = make_plan(16, out_f, in_f_padded, grouped_ctas(max_problems, S, kMaxSms));
  if ((size_t)max_problems * grouped_cnt_bytes(pl.n_rt16) > kGroupedCounterZone) return 0;
  return kGroupedCounterZone + (size_t)max_problems * pl.part_bytes;
}

extern "C" int pe_gemv_grouped(const void* codes, int packed, int64_t ld_codes, int64_t codes_stride, const void* norms,
                               int64_t ld_norms, int64_t norms_stride, const float* ct_scaled, int n_levels, const void* x,
                               int x_kind, int x_dtype, int64_t ld_x, int in_f, const int32_t* x_rows, void* y, int y_dtype,
                               int64_t ld_y, const int32_t* problems, int max_problems, int max_rows, int out_f,
                               int in_f_padded, void* workspace, size_t workspace_bytes, void* stream) {
  if (!codes || !norms || !ct_scaled || !x || !y || !problems || !workspace) return PE_ERR_ARG;
  if (max_rows < 1 || max_rows > 16) return PE_ERR_ARG;
  if (max_problems < 1 || max_problems > 65535 || out_f < 1 || in_f < 1 || in_f > in_f_padded) return PE_ERR_ARG;
  if (x_kind != PE_X_ROTATED && x_kind != PE_X_RAW) return PE_ERR_ARG;
  if (x_dtype < PE_F32 || x_dtype > PE_BF16 || y_dtype < PE_F32 || y_dtype > PE_BF16) return PE_ERR_ARG;
  if (n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (in_f_padded % kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15) || (codes_stride & 15) ||
      (reinterpret_cast<uintptr_t>(problems) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return PE_ERR_ALIGN;
  if (ld_codes < (packed ? in_f_padded / 2 : in_f_padded) || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  if (ld_x < (x_kind == PE_X_RAW ? in_f : in_f_padded) || ld_y < out_f) return PE_ERR_ARG;
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  if (sms > kMaxSms || (out_f + 15) / 16 > kMaxRowTiles) return PE_ERR_LIMIT;
  const long long S = (long long)((out_f + 255) / 256) * (in_f_padded / kBlock) * 16;
  if (S >= (1ll << 31) / kMaxSms) return PE_ERR_LIMIT;
  Plan pl = make_plan(16, out_f, in_f_padded, grouped_ctas(max_problems, S, sms));
  const size_t cnt_bytes = grouped_cnt_bytes(pl.n_rt16);
  // sized like pe_gemv_grouped_workspace_bytes (its CTA count per problem is an upper bound of this one)
  const size_t need = pe_gemv_grouped_workspace_bytes(max_problems, out_f, in_f_padded);
  if (need == 0) return PE_ERR_LIMIT;
  if (workspace_bytes < need) return PE_ERR_WORKSPACE;
  const Plan pl_max = make_plan(16, out_f, in_f_padded, grouped_ctas(max_problems, S, kMaxSms));

  GemvArgs a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const __half*>(norms); a.ld_norms = ld_norms;
  a.tiles = nullptr;
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.x = x; a.x_kind = x_kind; a.x_dtype = x_dtype; a.ld_x = ld_x; a.in_f = in_f;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = nullptr;
  a.batch = 16; a.N = out_f; a.K = in_f_padded; a.nb = pl.nb;
  a.n_rt16 = pl.n_rt16; a.n_rt256 = pl.n_rt256; a.S = (int)pl.S; a.cap = pl.cap; a.max_slots = pl.max_slots;
  a.ws_cnt = static_cast<unsigned*>(workspace);
  a.ws_status = nullptr;  // per problem, set in the kernel
  a.ws_part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kGroupedCounterZone);
  a.x_rows = x_rows;
  a.grp = reinterpret_cast<const int4*>(problems);
  a.grp_codes_stride = codes_stride; a.grp_norms_stride = norms_stride;
  a.grp_cnt_bytes = cnt_bytes;
  a.grp_ws_stride = pl_max.part_bytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (max_rows <= 8) {  // every problem fits one 8-row activation tile: half the tensor work per step
    if (packed && n_levels <= 8) return launch_t<true, 8, 6, true, false, false, true>(a, pl, st, max_problems);
    if (packed) return launch_t<true, 8, 6, false, false, false, true>(a, pl, st, max_problems);
    return launch_t<false, 8, 2, false, false, false, true>(a, pl, st, max_problems);
  }
  if (packed && n_levels <= 8) return launch_t<true, 16, 6, true, false, false, true>(a, pl, st, max_problems);
  if (packed) return launch_t<true, 16, 6, false, false, false, true>(a, pl, st, max_problems);
  return launch_t<false, 16, 2, false, false, false, true>(a, pl, st, max_problems);
}

// ---- tiled weight layout ---------------------------------------------------------
namespace pe {
// one thread per 16-byte piece of the output
template <bool PACKED>
__global__ void __launch_bounds__(256) retile_kernel(const uint8_t* codes, int64_t ld_codes, const __half* norms,
                                                     int64_t ld_norms, uint8_t* out, int N, int nb, int64_t n_pieces) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pieces) return;
  constexpr int kPieces = TileGeom<PACKED>::kTileBytes / 16;   // 66 or 130
  constexpr int kRowBytes = PACKED ? 64 : 128;
  const int64_t tile = i / kPieces;
  const int piece = (int)(i - tile * kPieces);
  const int rt16 = (int)(tile / nb), b = (int)(tile - (int64_t)rt16 * nb);
  uint4 v = make_uint4(0, 0, 0, 0);
  if (piece < TileGeom<PACKED>::kCodeBytes / 16) {
    const int r = piece / (kRowBytes / 16), c = piece % (kRowBytes / 16);
    const int row = rt16 * 16 + r;
    if (row < N) v = *reinterpret_cast<const uint4*>(codes + (int64_t)row * ld_codes + b * kRowBytes + c * 16);
  } else {  // norms: rows 0..7 in the first piece, 8..15 in the second
    const int r0 = (piece - TileGeom<PACKED>::kCodeBytes / 16) * 8;
    unsigned short h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int row = rt16 * 16 + r0 + k;
      h[k] = row < N ? __half_as_ushort(norms[(int64_t)row * ld_norms + b]) : (unsigned short)0;
    }
    v = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
  }
  *reinterpret_cast<uint4*>(out + i * 16) = v;
}
}  // namespace pe

extern "C" size_t pe_retile_bytes(int packed, int64_t out_f, int64_t in_f_padded) {
  if (out_f < 1 || in_f_padded < kBlock || in_f_padded % kBlock) return 0;
  const size_t tile = packed ? TileGeom<true>::kTileBytes : TileGeom<false>::kTileBytes;
  return (size_t)((out_f + 15) / 16) * (size_t)(in_f_padded / kBlock) * tile;
}

extern "C" int pe_retile(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, void* tiles,
                         int64_t out_f, int64_t in_f_padded, void* stream) {
  if (!codes || !norms || !tiles || out_f < 1 || out_f > 0x7fffffff) return PE_ERR_ARG;
  if (in_f_padded < kBlock || in_f_padded % kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15) || (reinterpret_cast<uintptr_t>(tiles) & 15)) return PE_ERR_ALIGN;
  const int nb = (int)(in_f_padded / kBlock);
  const int64_t n_pieces = (int64_t)pe_retile_bytes(packed, out_f, in_f_padded) / 16;
  const int64_t blocks = (n_pieces + 255) / 256;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (packed)
    retile_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(codes), ld_codes,
                                                         static_cast<const __half*>(norms), ld_norms,
                                                         static_cast<uint8_t*>(tiles), (int)out_f, nb, n_pieces);
  else
    retile_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(codes), ld_codes,
                                                          static_cast<const __half*>(norms), ld_norms,
                                                          static_cast<uint8_t*>(tiles), (int)out_f, nb, n_pieces);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_gemv_tiled(const void* tiles, int packed, const float* ct_scaled, int n_levels, const void* x, int x_kind,
                             int x_dtype, int64_t ld_x, int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias,
                             int batch, int out_f, int in_f_padded, void* workspace, size_t workspace_bytes, void* stream) {
  if (!tiles) return PE_ERR_ARG;
  return gemv_run(nullptr, packed, 0, nullptr, 0, tiles, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y, y_dtype, ld_y,
                  bias, batch, out_f, in_f_padded, workspace, workspace_bytes, stream);
}

// ---- entry point for callers that cannot allocate device memory -------------------
//
// Some hosts of this library hand every byte of device memory to their own pool at
// start-up (an inference server sizes its KV cache from "whatever is free" and keeps
// it), so a cudaMalloc made later on behalf of one linear layer can fail, and the code
// that calls into the layer has no allocator of its own to ask.  For them the split-K
// scratch lives inside the library image: a fixed array in device global memory that
// exists on every GPU that loads the library, from load until exit.
constexpr size_t kNoAllocScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// In host code the array's name only stands for the symbol; the device address has to
// be asked for, once per device, with that device current.
static void* g_noalloc_ptr[64] = {nullptr};

extern "C" size_t pe_gemv_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

// Device address of the array on the current device (looked up once per device).
static int noalloc_scratch(void** out) {
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PE_ERR_LIMIT;
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    PE_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return PE_OK;
}

extern "C" int pe_gemv_noalloc(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                               const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype,
                               int64_t ld_x, int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch,
                               int out_f, int in_f_padded, void* stream) {
  const int c = gemv_check(codes, packed, ld_codes, norms, ld_norms, nullptr, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f,
                           y, y_dtype, ld_y, batch, out_f, in_f_padded);
  if (c != PE_OK) return c;
  const size_t need = pe_gemv_workspace_bytes(batch, out_f, in_f_padded);
  if (need == 0 || need > kNoAllocScratchBytes) return PE_ERR_LIMIT;  // shape needs more scratch than the built-in array holds
  void* ws = nullptr;
  const int r = noalloc_scratch(&ws);
  if (r != PE_OK) return r;
  if (batch <= 2) {  // kernels that own whole weight rows touch nothing of the array but its status word
    const int rr = gemv_scratch_free(codes, packed, ld_codes, norms, ld_norms, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f,
                                     y, y_dtype, ld_y, bias, batch, out_f, in_f_padded, ws, stream);
    if (rr <= 0) return rr;
  }
  // The array keeps whatever the previous call left.  Only the tile counters have to
  // read zero on entry; clear the ones this shape uses, in stream order.
  const size_t counter_bytes = (size_t)((out_f + 15) / 16) * sizeof(unsigned);
  PE_CUDA_TRY(cudaMemsetAsync(ws, 0, counter_bytes, static_cast<cudaStream_t>(stream)));
  return gemv_tile_run(codes, packed, ld_codes, norms, ld_norms, nullptr, ct_scaled, n_levels, x, x_kind, x_dtype, ld_x, in_f, y,
                       y_dtype, ld_y, bias, batch, out_f, in_f_padded, ws, kNoAllocScratchBytes, stream);
}

extern "C" int pe_gemv_noalloc_status(int clear, void* stream) {
  void* ws = nullptr;
  const int r = noalloc_scratch(&ws);
  if (r != PE_OK) return r;
  return read_status_word(reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + kCounterBytes - 4), clear, stream);
}
