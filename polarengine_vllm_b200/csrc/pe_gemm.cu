// Prefill-size quantized matmul (many activation rows) on the 5th-generation tensor
// cores: tcgen05.mma with TMEM accumulators, TMA-staged activations, in-kernel dequant.
//
//   Y[m, n] = sum_k Xt[m, k] * (ct[code[n, k]] * norm[n, k / 128])        (+ bias[n])
//
// Two persistent kernels share the scheme; both walk K in steps of 64:
//   * one thread issues TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast) for the bf16
//     activation tiles and for the raw code rows of the step;
//   * 16 decode warps turn code rows into a bf16 weight stage in the swizzled K-major layout the tensor
//     core reads (table look-up or byte permutes, times the block norm) -- the decoded weights never
//     touch HBM or L2.  The warps form groups that take alternate K steps, because one warp's trip through
//     a step (barrier round trips, proxy fence) lasts longer than the step's MMAs;
//   * one thread issues tcgen05.mma (bf16 in, fp32 accumulate in TMEM: two accumulators of 256 columns
//     = all 512) and hands stages back with tcgen05.commit;
//   * after the last step the decode warps read the accumulators back (tcgen05.ld), add the bias,
//     convert and store.
// gemm_kernel: one CTA per 256 tokens x 256 weight rows (up to 256 tokens, and the grouped launches of a
// mixture-of-experts layer).  gemm_pair_kernel: a cluster of two CTAs per 512 tokens x 256 weight rows,
// one cta_group::2 MMA per pair, each CTA decoding half of the weight tile (more than 256 tokens).
// The activations are prepared by a small kernel (pad + FWHT-128 for raw input, bf16, and for nibble
// layers the (k, k+64) pairing of the half-block layout so that one code byte decodes to two adjacent
// K elements).
//
// Every wait is bounded: on time-out the kernel records a status code in the first word
// of the workspace, all roles leave their loops, TMEM is released and the grid returns.
#include <cuda.h>

#include "pe_common.cuh"
#include "pe_gemv_decode.cuh"

namespace pe {

constexpr int kTileM = 256;          // tokens per CTA tile (two UMMA M=128 halves)
constexpr int kTileN = 256;          // weight rows per CTA tile (UMMA N)
constexpr int kStepK = 64;           // K elements per pipeline stage (128 bytes of bf16)
constexpr int kXStages = 3;          // activation stages (two 128-token tiles each): deep, they come from L2/HBM
constexpr int kWStages = 2;          // decoded-weight stages: produced locally
constexpr int kXTileBytes = 128 * kStepK * 2;        // 16 KB
constexpr int kWTileBytes = kTileN * kStepK * 2;     // 32 KB
constexpr int kGemmThreads = 576;                    // 18 warps: TMA, MMA, 16 decode/epilogue
constexpr int kDecodeThreads = 512;
constexpr int kGroups = 2;                          // decode warp groups of the single-CTA kernel, one K step each
constexpr int kGroupWarps = kDecodeThreads / 32 / kGroups;
static_assert(kWStages == kGroups, "a decode group owns its weight stage");
constexpr long long kTimeoutCycles = 1ll << 31;

struct GemmArgs {
  const uint8_t* codes; int64_t ld_codes;
  const __half* norms; int64_t ld_norms;
  const float* ct; int n_levels;
  void* y; int y_dtype; int64_t ld_y;
  const __half* bias;
  int M, N, K;
  int tiles_m, tiles_n;
  int lut_bytes;  // n_levels (256 for nibble pairs) x 128 B
  int nc;         // code stages
  int ksplit;     // single-CTA kernel: K ranges per tile (1 = none); partial results in `part`
  float* part;    // [ksplit][M][N] fp32
  int y_tma;      // paired kernel: the output leaves through TMA stores (16-bit output, 16-byte aligned rows)
  int* status;
  // grouped launch over a stack of matrices (the experts of a mixture layer): tile list on the device
  const int4* gtiles;        // per tile: (first activation row, rows, first weight row inside the expert, expert)
  const int* n_gtiles;       // number of tiles in the list
  int64_t grp_norm_stride;   // halves between the norms of consecutive experts
};

// Activation rows [m0, m_end) and weight rows n0 .. n0 + 255 of an expert; crow0 = row of the code tensor.
struct TileCoord { int m0, m_end, n0, crow0, expert; };
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& p, int tile) {
  TileCoord t;
  if (p.gtiles) {
    const int4 d = p.gtiles[tile];
    t.m0 = d.x; t.m_end = d.x + d.y; t.n0 = d.z; t.expert = d.w; t.crow0 = d.w * p.N + d.z;
  } else {
    t.m0 = (tile % p.tiles_m) * kTileM; t.m_end = p.M; t.n0 = (tile / p.tiles_m) * kTileN; t.expert = 0; t.crow0 = t.n0;
  }
  return t;
}

// ---- PTX wrappers -----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if the CTA is aborting (somebody timed out, maybe us).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kTimeoutCycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (SBO), LBO field 1,
// descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&r);
}

// low half of a, high half of b
__device__ __forceinline__ uint32_t lo_hi16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7610;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// bf16 centroids of a layer with at most 8 levels as a register table for reg_decode (byte permutes instead of
// shared-memory look-ups: the look-ups are what fills the shared-memory pipe when a weight tile serves few tokens)
__device__ __forceinline__ RegTable bf16_reg_table(const float* ct, int n_levels) {
  RegTable tb = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t hb = pack_bf16(i < n_levels ? ct[i] : 0.f, 0.f) & 0xffffu;
    if (i < 4) { tb.lo0 |= (hb & 0xff) << (8 * i); tb.hi0 |= (hb >> 8) << (8 * i); }
    else { tb.lo1 |= (hb & 0xff) << (8 * (i - 4)); tb.hi1 |= (hb >> 8) << (8 * (i - 4)); }
  }
  return tb;
}

// table entry address: lut + byte * 128 + lane * 4
template <int BYTE>
__device__ __forceinline__ uint32_t glut(uint32_t word, uint32_t lane_base) {
  uint32_t b, v;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(b) : "r"(word), "r"(0), "n"(0x4440 | BYTE));
  const uint32_t addr = b * 128u + lane_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

template <bool PACKED>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const GemmArgs p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap cmap) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* sm = smem_raw + (base - raw);
  // [X stages 3 x 32 KB][W stages 2 x 32 KB][table][code stages nc x (256 rows x 32|64 B)][barriers]
  constexpr int kXStage = 2 * kXTileBytes;
  constexpr uint32_t kWOff = kXStages * kXStage;
  constexpr uint32_t kLutOff = kWOff + kWStages * kWTileBytes;
  constexpr int kCodeRow = PACKED ? 32 : 64;          // code bytes per weight row per K step
  constexpr int kCodeStage = kTileN * kCodeRow;
  const uint32_t c_off = kLutOff + p.lut_bytes;
  const uint32_t bar_off = c_off + p.nc * kCodeStage;
  const uint32_t lut_s = base + kLutOff;
  uint8_t* lut_g = sm + kLutOff;
  const uint32_t bars = base + bar_off;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + bar_off + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + bar_off + 196);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto full_x = [&](int s) { return bars + 8 * s; };         // 3
  auto empty_x = [&](int s) { return bars + 24 + 8 * s; };   // 3
  auto full_w = [&](int s) { return bars + 48 + 8 * s; };    // 2
  auto empty_w = [&](int s) { return bars + 64 + 8 * s; };   // 2
  auto full_c = [&](int s) { return bars + 80 + 8 * s; };    // up to 4
  auto empty_c = [&](int s) { return bars + 112 + 8 * s; };  // up to 4
  const uint32_t acc_full = bars + 144;
  const uint32_t acc_empty = bars + 152;  // every decode warp has read the accumulators of a tile

  if (tid == 0) {
    for (int s = 0; s < kXStages; ++s) { mbar_init(full_x(s), 1); mbar_init(empty_x(s), 1); }
    for (int s = 0; s < kWStages; ++s) { mbar_init(full_w(s), kGroupWarps); mbar_init(empty_w(s), 1); }
    for (int s = 0; s < p.nc; ++s) { mbar_init(full_c(s), 1); mbar_init(empty_c(s), kGroupWarps); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kDecodeThreads / 32);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // centroid table, one copy per lane (entry e of lane l at e * 128 + l * 4)
  if (warp >= 2) {
    const int d = tid - 64;
    for (int e = d >> 5; e < (PACKED ? 256 : p.n_levels); e += kDecodeThreads / 32) {
      uint32_t v;
      if (PACKED) {
        const int lo = e & 15, hi = e >> 4;
        v = pack_bf16(lo < p.n_levels ? p.ct[lo] : 0.f, hi < p.n_levels ? p.ct[hi] : 0.f);
      } else {
        v = pack_bf16(p.ct[e], p.ct[e]);
      }
      *reinterpret_cast<uint32_t*>(lut_g + e * 128 + lane * 4) = v;
    }
  }
  if (warp == 1) {  // TMEM: all 512 columns, allocated and later freed by this warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  const int ksteps = p.K / kStepK;
  // A unit of work is a tile, or -- for dense launches with few tiles -- one of `ksplit` K ranges of a tile, whose
  // fp32 partial goes to the workspace and is summed by a second kernel.
  const int n_tiles = (p.gtiles ? *p.n_gtiles : p.tiles_m * p.tiles_n) * p.ksplit;
  auto unit_of = [&](int unit, int& split, int& ks0, int& ks1) {
    const int tile = unit / p.ksplit;
    split = unit - tile * p.ksplit;
    ks0 = (int)((long long)split * ksteps / p.ksplit);
    ks1 = (int)((long long)(split + 1) * ksteps / p.ksplit);
    return tile;
  };

  if (warp == 0) {
    // ---------------- TMA producer: activations and codes ----------------
    if (lane == 0) {
      int it = 0;
      for (int unit = blockIdx.x; unit < n_tiles && !*abort_flag; unit += gridDim.x) {
        int split, ks0, ks1;
        const TileCoord tc = tile_coord(p, unit_of(unit, split, ks0, ks1));
        const int m0 = tc.m0;
        const bool two = m0 + 128 < tc.m_end;
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const int sc = it % p.nc;
          if (!mbar_wait(empty_c(sc), ((it / p.nc) & 1) ^ 1, abort_flag, p.status, 6)) goto done_producer;
          mbar_expect_tx(full_c(sc), kCodeStage);
          tma_load_2d(base + c_off + sc * kCodeStage, &cmap, ks * kCodeRow, tc.crow0, full_c(sc));
          const int sx = it % kXStages;
          if (!mbar_wait(empty_x(sx), ((it / kXStages) & 1) ^ 1, abort_flag, p.status, 1)) goto done_producer;
          mbar_expect_tx(full_x(sx), two ? 2 * kXTileBytes : kXTileBytes);
          tma_load_2d(base + sx * kXStage, &xmap, ks * kStepK, m0, full_x(sx));
          if (two) tma_load_2d(base + sx * kXStage + kXTileBytes, &xmap, ks * kStepK, m0 + 128, full_x(sx));
        }
      }
    done_producer:;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0, tcount = 0;
      for (int unit = blockIdx.x; unit < n_tiles && !*abort_flag; unit += gridDim.x, ++tcount) {
        int split, ks0, ks1;
        const TileCoord tc = tile_coord(p, unit_of(unit, split, ks0, ks1));
        const bool two = tc.m0 + 128 < tc.m_end;
        if (tcount > 0 && !mbar_wait(acc_empty, (tcount - 1) & 1, abort_flag, p.status, 9)) goto done_mma;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const int sx = it % kXStages, sw = it % kWStages;
          if (!mbar_wait(full_x(sx), (it / kXStages) & 1, abort_flag, p.status, 2)) goto done_mma;
          if (!mbar_wait(full_w(sw), (it / kWStages) & 1, abort_flag, p.status, 3)) goto done_mma;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t xa = base + sx * kXStage, wb = base + kWOff + sw * kWTileBytes;
#pragma unroll
          for (int kk = 0; kk < kStepK / 16; ++kk) {
            const uint64_t db = smem_desc_sw128(wb + kk * 32);
            const uint32_t acc = (ks > ks0 || kk > 0) ? 1u : 0u;
            umma_bf16(tmem, smem_desc_sw128(xa + kk * 32), db, kIdesc, acc);
            if (two) umma_bf16(tmem + 256, smem_desc_sw128(xa + kXTileBytes + kk * 32), db, kIdesc, acc);
          }
          umma_commit(empty_x(sx));  // both buffers are free once these MMAs have read them
          umma_commit(empty_w(sw));
        }
        umma_commit(acc_full);       // accumulators of this tile complete
      }
    done_mma:;
    }
  } else {
    // ---------------- decode + epilogue warps ----------------
    // A warp's trip through one K step is a chain of barrier round trips (codes full, weight stage empty, proxy
    // fence, arrival) that costs more than the step's MMAs however little it decodes.  So the 16 warps form two
    // groups; group g takes the steps with it % 2 == g, a whole 256-row stage each (thread = one weight row, all 64
    // K elements), and owns weight stage g and code stage g (a parity wait is only sound while the waiter is less
    // than two phases ahead of its barrier, which stages shared between groups would not guarantee).
    const int d = tid - 64;
    const int r = d & 255, g = d >> 8;
    const bool regtab = PACKED && p.n_levels <= 8;  // nibble codes below 8: a valid byte-permute selector
    const RegTable tb = regtab ? bf16_reg_table(p.ct, p.n_levels) : RegTable{0, 0, 0, 0};
    const uint32_t lane_base = lut_s + lane * 4;
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;        // 0..3
    const int half = grp & 1;               // accumulator (token half) this warp drains
    const int chalf = grp >> 1;             // which 128 of its 256 columns
    const uint32_t wrow = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
    const int sw7 = r & 7;
    int it = 0, tcount = 0;
    for (int unit = blockIdx.x; unit < n_tiles && !*abort_flag; unit += gridDim.x, ++tcount) {
      int split, ks0, ks1;
      const TileCoord tc = tile_coord(p, unit_of(unit, split, ks0, ks1));
      const int m0 = tc.m0, n0 = tc.n0;
      // where this unit's result goes: the output, or (K split) the fp32 partial of its K range
      void* const y_ptr = p.ksplit > 1 ? static_cast<void*>(p.part + (size_t)split * p.M * p.N) : p.y;
      const int y_dt = p.ksplit > 1 ? (int)PE_F32 : p.y_dtype;
      const int64_t y_ld = p.ksplit > 1 ? (int64_t)p.N : p.ld_y;
      const __half* const bias_ptr = p.ksplit > 1 ? nullptr : p.bias;
      const bool two = m0 + 128 < tc.m_end;
      int row = n0 + r;
      const bool row_ok = row < p.N;
      if (!row_ok) row = p.N - 1;
      const unsigned short* nrow =
          reinterpret_cast<const unsigned short*>(p.norms + (int64_t)tc.expert * p.grp_norm_stride + (int64_t)row * p.ld_norms);
      bool dead = false;
      for (int ks = ks0; ks < ks1; ++ks, ++it) {
        if ((it & (kGroups - 1)) != g) continue;  // warp-uniform
        const float nf = row_ok ? __half2float(__ushort_as_half(__ldg(nrow + (ks >> 1)))) : 0.f;  // in flight across the waits
        const int sc = it % p.nc;
        {
          const bool ok = mbar_wait(full_c(sc), (it / p.nc) & 1, abort_flag, p.status, 7);
          if (!__all_sync(0xffffffffu, ok)) { dead = true; break; }  // leave together or not at all
        }
        constexpr int CW = PACKED ? 2 : 4;  // 16-byte pieces of this row's codes
        uint4 c[CW];
        const uint8_t* csrc = sm + c_off + sc * kCodeStage + r * kCodeRow;
#pragma unroll
        for (int i = 0; i < CW; ++i) c[i] = *reinterpret_cast<const uint4*>(csrc + 16 * i);
        // the stage goes back only after the loads have delivered: an arrival issued straight behind
        // (bank-conflicted, multi-pass) loads can overtake them, and the refill then lands on unread rows
        {
          uint32_t seen = 0;
#pragma unroll
          for (int i = 0; i < CW; ++i) seen |= c[i].x | c[i].y | c[i].z | c[i].w;
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(bars + 224), "r"(seen) : "memory");
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_c(sc));
        const uint32_t n2 = pack_bf16(nf, nf);
        const int sw = it % kWStages;
        {
          const bool ok = mbar_wait(empty_w(sw), ((it / kWStages) & 1) ^ 1, abort_flag, p.status, 4);
          if (!__all_sync(0xffffffffu, ok)) { dead = true; break; }
        }
        uint8_t* wt = sm + kWOff + sw * kWTileBytes + wrow;
#pragma unroll
        for (int i = 0; i < CW; ++i) {
          const uint32_t wq[4] = {c[i].x, c[i].y, c[i].z, c[i].w};
          if (PACKED) {  // one code byte -> two adjacent K elements; word j of piece i -> chunk 4 i + j
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w = wq[j];
              uint4 o;
              if (regtab) {
                uint32_t a[4];
                reg_decode(w, tb, a);
                o.x = bf16x2_mul(a[0], n2); o.y = bf16x2_mul(a[1], n2); o.z = bf16x2_mul(a[2], n2); o.w = bf16x2_mul(a[3], n2);
              } else {
                o.x = bf16x2_mul(glut<0>(w, lane_base), n2);
                o.y = bf16x2_mul(glut<1>(w, lane_base), n2);
                o.z = bf16x2_mul(glut<2>(w, lane_base), n2);
                o.w = bf16x2_mul(glut<3>(w, lane_base), n2);
              }
              *reinterpret_cast<uint4*>(wt + (((4 * i + j) ^ sw7) << 4)) = o;
            }
          } else {       // one code byte -> one K element; words 2j, 2j+1 of piece i -> chunk 2 i + j
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t wa = wq[2 * j], wb = wq[2 * j + 1];
              uint4 o;
              o.x = bf16x2_mul(lo_hi16(glut<0>(wa, lane_base), glut<1>(wa, lane_base)), n2);
              o.y = bf16x2_mul(lo_hi16(glut<2>(wa, lane_base), glut<3>(wa, lane_base)), n2);
              o.z = bf16x2_mul(lo_hi16(glut<0>(wb, lane_base), glut<1>(wb, lane_base)), n2);
              o.w = bf16x2_mul(lo_hi16(glut<2>(wb, lane_base), glut<3>(wb, lane_base)), n2);
              *reinterpret_cast<uint4*>(wt + (((2 * i + j) ^ sw7) << 4)) = o;
            }
          }
        }
        // make the generic-proxy stores visible to the tensor core, then one arrive per warp
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_w(sw));
      }
      if (dead) break;
      // ---------------- epilogue: TMEM -> registers -> global ----------------
      {
        const bool ok = mbar_wait(acc_full, tcount & 1, abort_flag, p.status, 5);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (half == 0 || two) {
        const int m = m0 + half * 128 + q * 32 + lane;
        const uint32_t trow = tmem + half * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
        for (int cc = chalf * 4; cc < chalf * 4 + 4; ++cc) {
          uint32_t rr[32];
          tmem_ld32(trow + cc * 32, rr);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int nb0 = n0 + cc * 32;
          if (m < tc.m_end && nb0 < p.N) {
            const bool full = nb0 + 32 <= p.N && (y_ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(y_ptr) & 15) == 0);
            if (full && y_dt != PE_F32) {
              uint32_t o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float a = __uint_as_float(rr[2 * j]), b = __uint_as_float(rr[2 * j + 1]);
                if (bias_ptr) { a += __half2float(bias_ptr[nb0 + 2 * j]); b += __half2float(bias_ptr[nb0 + 2 * j + 1]); }
                o[j] = y_dt == PE_F16 ? pack_half2(a, b) : pack_bf16(a, b);
              }
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y_ptr) + (int64_t)m * y_ld + nb0);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            } else if (y_dt == PE_F32 && nb0 + 32 <= p.N && (y_ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(y_ptr) & 15) == 0)) {
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(y_ptr) + (int64_t)m * y_ld + nb0);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(rr[4 * j]), __uint_as_float(rr[4 * j + 1]), __uint_as_float(rr[4 * j + 2]),
                                       __uint_as_float(rr[4 * j + 3]));
                if (bias_ptr) {
                  v.x += __half2float(bias_ptr[nb0 + 4 * j]); v.y += __half2float(bias_ptr[nb0 + 4 * j + 1]);
                  v.z += __half2float(bias_ptr[nb0 + 4 * j + 2]); v.w += __half2float(bias_ptr[nb0 + 4 * j + 3]);
                }
                dst[j] = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (nb0 + j < p.N) {
                  float a = __uint_as_float(rr[j]);
                  if (bias_ptr) a += __half2float(bias_ptr[nb0 + j]);
                  store_from_float(y_ptr, y_dt, (int64_t)m * y_ld + nb0 + j, a);
                }
              }
            }
          }
        }
      }
      // the next tile's first MMA overwrites the accumulators: it waits for every decode warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
  }

  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag && tid == 0) {  // give copies that may still be in flight time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

// ---- paired form: two CTAs of a cluster share one tensor-core operation (cta_group::2) -----------------
// A pair owns 512 tokens x 256 weight rows.  Each CTA keeps ITS 128-token halves of the two 256-token
// accumulators in its own TMEM, stages its own activation tiles and decodes only 128 of the 256 weight
// rows: the tensor core of each SM reads that half from its own shared memory, so the decode work and the
// weight-operand traffic per SM are half of the single-CTA form (which is bound by them: with the decode
// and the activation copies switched off it still ran at three quarters of the dense-GEMM rate).
// The even CTA of the pair issues the MMAs.  It learns that the odd CTA's stages are full through
// arrivals on its own barriers (a relay thread for the TMA-filled activation stages, the decode warps
// directly for the weight stages) and hands stages back with one tcgen05.commit per CTA.
constexpr int kPairWStages = 4;                      // 16 KB each: this CTA's 128 weight rows; one per decode group
constexpr int kPairCodeStages = 4;                   // one per decode group
constexpr int kPairLutStride = 64;                   // nibble layers: 16 copies of the 256-entry pair table (16 KB)
constexpr int kPairWTileBytes = 128 * kStepK * 2;
constexpr int kPairTileM = 512;
constexpr int kPairThreads = kGemmThreads + 32;     // 19 warps: activation TMA, MMA, 16 decode/epilogue, code TMA
constexpr int kPairGroups = 4;                       // decode warp groups, one K step each.  A group owns weight stage g and
                                                     // code stage g: a parity wait is only sound while the waiter is
                                                     // less than two phases ahead of the barrier, which sharing a stage
                                                     // between groups does not guarantee
static_assert(kPairWStages == kPairGroups && kPairCodeStages == kPairGroups, "one stage of each ring per decode group");
constexpr int kPairGroupWarps = kDecodeThreads / 32 / kPairGroups;
constexpr uint32_t kIdescPair = (1u << 4) | (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | ((256u >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared-memory address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait on a barrier that CTAs of the cluster arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kTimeoutCycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
// TMA load of a CTA pair: the bytes land in THIS CTA's shared memory, the completion is counted on a barrier
// that may live in the other CTA of the pair (a mapped address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// arrival on ONE barrier (of this CTA or, with a mapped address, of the other) once the MMAs issued so far are done
__device__ __forceinline__ void umma_pair_commit(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

// table entry address: lut + byte * STRIDE + copy * 4
template <int BYTE, int STRIDE>
__device__ __forceinline__ uint32_t glut_s(uint32_t word, uint32_t lane_base) {
  uint32_t b, v;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(b) : "r"(word), "r"(0), "n"(0x4440 | BYTE));
  const uint32_t addr = b * (uint32_t)STRIDE + lane_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

template <bool PACKED>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const GemmArgs p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap cmap,
                 const __grid_constant__ CUtensorMap ymap) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  // [X stages 4|3 x 32 KB][W stages 4 x 16 KB][table][code stages 4 x (128 rows x 32|64 B)][barriers]
  constexpr int kPairXStages = PACKED ? 4 : 3;  // byte codes need twice the code stages' room
  constexpr int kLutStride = PACKED ? kPairLutStride : 128;
  constexpr int kXStage = 2 * kXTileBytes;
  constexpr uint32_t kWOff = kPairXStages * kXStage;
  constexpr uint32_t kLutOff = kWOff + kPairWStages * kPairWTileBytes;
  constexpr int kCodeRow = PACKED ? 32 : 64;
  constexpr int kCodeStage = 128 * kCodeRow;
  const uint32_t c_off = kLutOff + p.lut_bytes;
  const uint32_t bar_off = c_off + p.nc * kCodeStage;
  const uint32_t lut_s = base + kLutOff;
  uint8_t* lut_g = sm + kLutOff;
  const uint32_t bars = base + bar_off;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + bar_off + 216);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + bar_off + 220);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  auto full_x = [&](int s) { return bars + 8 * s; };          // up to 4
  auto empty_x = [&](int s) { return bars + 32 + 8 * s; };    // up to 4
  auto full_w = [&](int s) { return bars + 64 + 8 * s; };     // 4 (used in the even CTA)
  auto empty_w = [&](int s) { return bars + 96 + 8 * s; };    // 4
  auto full_c = [&](int s) { return bars + 128 + 8 * s; };    // 4
  auto empty_c = [&](int s) { return bars + 160 + 8 * s; };   // 4
  const uint32_t acc_full = bars + 192;
  const uint32_t acc_empty = bars + 200;  // used in the even CTA: both CTAs have read the accumulators of a tile
  const uint32_t stg_free = bars + 208;   // the output staging (inside the weight stages) has been read by the TMA stores

  if (tid == 0) {
    // activation stage: one barrier in the even CTA counts the bytes of both CTAs' copies
    for (int s = 0; s < kPairXStages; ++s) { mbar_init(full_x(s), 1); mbar_init(empty_x(s), 1); }
    // weight stage: the decode warps of both CTAs
    for (int s = 0; s < kPairWStages; ++s) { mbar_init(full_w(s), 2 * kPairGroupWarps); mbar_init(empty_w(s), 1); }
    for (int s = 0; s < p.nc; ++s) { mbar_init(full_c(s), 1); mbar_init(empty_c(s), kPairGroupWarps); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 2 * (kDecodeThreads / 32));  // every decode warp of both CTAs, once per tile
    mbar_init(stg_free, kDecodeThreads / 32);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp >= 2 && warp < 18) {
    const int d = tid - 64;
    for (int e = d >> 5; e < (PACKED ? 256 : p.n_levels); e += kDecodeThreads / 32) {
      uint32_t v;
      if (PACKED) {
        const int lo = e & 15, hi = e >> 4;
        v = pack_bf16(lo < p.n_levels ? p.ct[lo] : 0.f, hi < p.n_levels ? p.ct[hi] : 0.f);
      } else {
        v = pack_bf16(p.ct[e], p.ct[e]);
      }
      if (lane * 4 < kLutStride) *reinterpret_cast<uint32_t*>(lut_g + e * kLutStride + lane * 4) = v;
    }
  }
  if (warp == 1) {  // one warp of EACH CTA of the pair allocates (all 512 columns) and later frees
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs exist before anybody arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  const int ksteps = p.K / kStepK;
  // A unit of work is a tile or, when the launch has few tiles, one of `ksplit` K ranges of a tile (fp32 partials
  // in the workspace, summed by a second kernel).
  const int n_tiles = p.tiles_m * p.tiles_n * p.ksplit;
  auto unit_of = [&](int unit, int& split, int& ks0, int& ks1) {
    const int tile = unit / p.ksplit;
    split = unit - tile * p.ksplit;
    ks0 = (int)((long long)split * ksteps / p.ksplit);
    ks1 = (int)((long long)(split + 1) * ksteps / p.ksplit);
    return tile;
  };
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's activation tiles ----------------
    // Both CTAs' copies complete on the even CTA's barrier, which expects the bytes of both.
    if (lane == 0) {
      const uint32_t lead = map_to_cta(bars, 0) - bars;
      int it = 0;
      for (int unit = pair; unit < n_tiles && !*abort_flag; unit += n_pairs) {
        int split, ks0, ks1;
        const int tile = unit_of(unit, split, ks0, ks1);
        const int m0 = (tile % p.tiles_m) * kPairTileM;
        const bool two = m0 + 256 < p.M;
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const int sx = it % kPairXStages;
          if (!mbar_wait(empty_x(sx), ((it / kPairXStages) & 1) ^ 1, abort_flag, p.status, 1)) goto done_producer;
          if (leader) mbar_expect_tx(full_x(sx), 2 * (two ? 2 * kXTileBytes : kXTileBytes));
          tma_load_2d_pair(base + sx * kXStage, &xmap, ks * kStepK, m0 + (int)rank * 128, full_x(sx) + lead);
          if (two) tma_load_2d_pair(base + sx * kXStage + kXTileBytes, &xmap, ks * kStepK, m0 + 256 + (int)rank * 128, full_x(sx) + lead);
        }
      }
    done_producer:;
    }
  } else if (warp == 18) {
    // ---------------- TMA producer: this CTA's code rows (a thread of its own: it runs ahead of the activations) ----------------
    if (lane == 0) {
      int it = 0;
      for (int unit = pair; unit < n_tiles && !*abort_flag; unit += n_pairs) {
        int split, ks0, ks1;
        const int tile = unit_of(unit, split, ks0, ks1);
        const int n0 = (tile / p.tiles_m) * kTileN;
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const int sc = it % p.nc;
          if (!mbar_wait(empty_c(sc), ((it / p.nc) & 1) ^ 1, abort_flag, p.status, 6)) goto done_codes;
          mbar_expect_tx(full_c(sc), kCodeStage);
          tma_load_2d(base + c_off + sc * kCodeStage, &cmap, ks * kCodeRow, n0 + (int)rank * 128, full_c(sc));
        }
      }
    done_codes:;
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (even CTA) ----------------
      const uint32_t peer = map_to_cta(bars, 1) - bars;  // same barrier, odd CTA
      const uint32_t peer_acc_full = acc_full + peer;
      int it = 0, tcount = 0;
      for (int unit = pair; unit < n_tiles && !*abort_flag; unit += n_pairs, ++tcount) {
        int split, ks0, ks1;
        const int tile = unit_of(unit, split, ks0, ks1);
        const int m0 = (tile % p.tiles_m) * kPairTileM;
        const bool two = m0 + 256 < p.M;
        if (tcount > 0 && !mbar_wait_cluster(acc_empty, (tcount - 1) & 1, abort_flag, p.status, 9)) goto done_mma;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const int sx = it % kPairXStages, sw = it % kPairWStages;
          if (!mbar_wait_cluster(full_x(sx), (it / kPairXStages) & 1, abort_flag, p.status, 2)) goto done_mma;
          if (!mbar_wait_cluster(full_w(sw), (it / kPairWStages) & 1, abort_flag, p.status, 3)) goto done_mma;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t xa = base + sx * kXStage, wb = base + kWOff + sw * kPairWTileBytes;
#pragma unroll
          for (int kk = 0; kk < kStepK / 16; ++kk) {
            const uint64_t db = smem_desc_sw128(wb + kk * 32);
            const uint32_t acc = (ks > ks0 || kk > 0) ? 1u : 0u;
            umma_pair_bf16(tmem, smem_desc_sw128(xa + kk * 32), db, kIdescPair, acc);
            if (two) umma_pair_bf16(tmem + 256, smem_desc_sw128(xa + kXTileBytes + kk * 32), db, kIdescPair, acc);
          }
          umma_pair_commit(empty_x(sx));
          umma_pair_commit(empty_x(sx) + peer);
          umma_pair_commit(empty_w(sw));
          umma_pair_commit(empty_w(sw) + peer);
        }
        umma_pair_commit(acc_full);
        umma_pair_commit(peer_acc_full);
      }
    done_mma:;
    }
  } else {
    // ---------------- decode + epilogue warps ----------------
    // A warp's trip through one K step is a chain of barrier round trips (codes full, weight stage empty,
    // proxy fence, arrival) that costs more than the MMAs of the step, however little it decodes.  So the 16
    // warps form four groups and group g takes the steps with it % 4 == g, a whole 128-row stage each
    // (thread = one weight row, all 64 K elements): four steps are in the decode pipeline at a time.
    const int d = tid - 64;
    const int r = d & 127, g = d >> 7;
    const bool regtab = PACKED && p.n_levels <= 8;  // nibble codes below 8: a valid byte-permute selector
    const RegTable tb = regtab ? bf16_reg_table(p.ct, p.n_levels) : RegTable{0, 0, 0, 0};
    // nibble layers: lanes l and l + 16 share a copy of the table (a two-way bank conflict when their
    // entries differ but have the same parity; the decode warps have the time)
    const uint32_t lane_base = lut_s + (uint32_t)(lane * 4 & (kLutStride - 1));
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int half = grp & 1;
    const int chalf = grp >> 1;
    const uint32_t wrow = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
    const int sw7 = r & 7;
    const uint32_t lead = map_to_cta(bars, 0) - bars;
    int it = 0, tcount = 0;
    for (int unit = pair; unit < n_tiles && !*abort_flag; unit += n_pairs, ++tcount) {
      int split, ks0, ks1;
      const int tile = unit_of(unit, split, ks0, ks1);
      const int m0 = (tile % p.tiles_m) * kPairTileM, n0 = (tile / p.tiles_m) * kTileN;
      const bool two = m0 + 256 < p.M;
      // where this unit's result goes: the output, or (K split) the fp32 partial of its K range
      void* const y_ptr = p.ksplit > 1 ? static_cast<void*>(p.part + (size_t)split * p.M * p.N) : p.y;
      const int y_dt = p.ksplit > 1 ? (int)PE_F32 : p.y_dtype;
      const int64_t y_ld = p.ksplit > 1 ? (int64_t)p.N : p.ld_y;
      const __half* const bias_ptr = p.ksplit > 1 ? nullptr : p.bias;
      const bool tma_out = p.y_tma && p.ksplit == 1;
      int row = n0 + (int)rank * 128 + r;
      const bool row_ok = row < p.N;
      if (!row_ok) row = p.N - 1;
      const unsigned short* nrow = reinterpret_cast<const unsigned short*>(p.norms + (int64_t)row * p.ld_norms);
      bool dead = false;
      for (int ks = ks0; ks < ks1; ++ks, ++it) {
        if ((it & (kPairGroups - 1)) != g) continue;  // warp-uniform
        const float nf = row_ok ? __half2float(__ushort_as_half(__ldg(nrow + (ks >> 1)))) : 0.f;  // in flight across the waits
        const int sc = it % p.nc;
        {
          const bool ok = mbar_wait(full_c(sc), (it / p.nc) & 1, abort_flag, p.status, 7);
          if (!__all_sync(0xffffffffu, ok)) { dead = true; break; }
        }
        constexpr int CW = PACKED ? 2 : 4;  // 16-byte pieces of this row's codes
        uint4 c[CW];
        const uint8_t* csrc = sm + c_off + sc * kCodeStage + r * kCodeRow;
#pragma unroll
        for (int i = 0; i < CW; ++i) c[i] = *reinterpret_cast<const uint4*>(csrc + 16 * i);
        // The stage is handed back (and refilled at once by the code producer) only after the loads have
        // DELIVERED: a store that consumes every loaded register sits between them and the arrival.  Without
        // it rows of byte codes (64-byte row pitch, four-way bank conflicts) were overwritten before they were read.
        {
          uint32_t seen = 0;
#pragma unroll
          for (int i = 0; i < CW; ++i) seen |= c[i].x | c[i].y | c[i].z | c[i].w;
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(bars + 224), "r"(seen) : "memory");
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_c(sc));
        const uint32_t n2 = pack_bf16(nf, nf);
        const int sw = it % kPairWStages;
        {
          const bool ok = mbar_wait(empty_w(sw), ((it / kPairWStages) & 1) ^ 1, abort_flag, p.status, 4);
          if (!__all_sync(0xffffffffu, ok)) { dead = true; break; }
        }
        uint8_t* wt = sm + kWOff + sw * kPairWTileBytes + wrow;
#pragma unroll
        for (int i = 0; i < CW; ++i) {
          const uint32_t wq[4] = {c[i].x, c[i].y, c[i].z, c[i].w};
          if (PACKED) {  // one code byte -> two adjacent K elements; word j of piece i -> chunk 4 i + j
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w = wq[j];
              uint4 o;
              if (regtab) {
                uint32_t a[4];
                reg_decode(w, tb, a);
                o.x = bf16x2_mul(a[0], n2); o.y = bf16x2_mul(a[1], n2); o.z = bf16x2_mul(a[2], n2); o.w = bf16x2_mul(a[3], n2);
              } else {
                o.x = bf16x2_mul(glut_s<0, kLutStride>(w, lane_base), n2);
                o.y = bf16x2_mul(glut_s<1, kLutStride>(w, lane_base), n2);
                o.z = bf16x2_mul(glut_s<2, kLutStride>(w, lane_base), n2);
                o.w = bf16x2_mul(glut_s<3, kLutStride>(w, lane_base), n2);
              }
              *reinterpret_cast<uint4*>(wt + (((4 * i + j) ^ sw7) << 4)) = o;
            }
          } else {       // one code byte -> one K element; words 2j, 2j+1 of piece i -> chunk 2 i + j
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t wa = wq[2 * j], wb = wq[2 * j + 1];
              uint4 o;
              o.x = bf16x2_mul(lo_hi16(glut_s<0, kLutStride>(wa, lane_base), glut_s<1, kLutStride>(wa, lane_base)), n2);
              o.y = bf16x2_mul(lo_hi16(glut_s<2, kLutStride>(wa, lane_base), glut_s<3, kLutStride>(wa, lane_base)), n2);
              o.z = bf16x2_mul(lo_hi16(glut_s<0, kLutStride>(wb, lane_base), glut_s<1, kLutStride>(wb, lane_base)), n2);
              o.w = bf16x2_mul(lo_hi16(glut_s<2, kLutStride>(wb, lane_base), glut_s<3, kLutStride>(wb, lane_base)), n2);
              *reinterpret_cast<uint4*>(wt + (((2 * i + j) ^ sw7) << 4)) = o;
            }
          }
        }
        // visible to the tensor core of this SM, then one arrival per warp on the even CTA's barrier
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(full_w(sw));
          else mbar_arrive_remote(full_w(sw) + lead);
        }
      }
      if (dead) break;
      // ---------------- epilogue: this CTA's 128 token rows of both accumulators ----------------
      {
        const bool ok = mbar_wait_cluster(acc_full, tcount & 1, abort_flag, p.status, 5);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (tma_out) {
        // 16-bit output: every warp stages its 32 rows x 32 columns (2 KB, 64-byte swizzle) in its own piece of the
        // weight stages -- idle now: all MMAs are done and no warp decodes before the staging barrier below -- and one
        // lane sends it off as a TMA store, which writes whole 64-byte row pieces and clips at the matrix edges.
        // Per-lane 16-byte stores straight to global memory, 32 rows per instruction, took a quarter of the kernel.
        const uint32_t stg = base + kWOff + (uint32_t)(warp - 2) * 2048u + (uint32_t)lane * 64u;
        const int swz = (lane >> 1) & 3;
        if (half == 0 || two) {
          const int mrow0 = m0 + half * 256 + (int)rank * 128 + q * 32;
          const uint32_t trow = tmem + half * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
          for (int cc = chalf * 4; cc < chalf * 4 + 4; ++cc) {
            uint32_t rr[32];
            tmem_ld32(trow + cc * 32, rr);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int nb0 = n0 + cc * 32;
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float a = __uint_as_float(rr[2 * j]), b = __uint_as_float(rr[2 * j + 1]);
              if (p.bias) {
                if (nb0 + 2 * j < p.N) a += __half2float(p.bias[nb0 + 2 * j]);
                if (nb0 + 2 * j + 1 < p.N) b += __half2float(p.bias[nb0 + 2 * j + 1]);
              }
              o[j] = p.y_dtype == PE_F16 ? pack_half2(a, b) : pack_bf16(a, b);
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the previous store has read the buffer
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j)
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)((j ^ swz) << 4)), "r"(o[4 * j]),
                           "r"(o[4 * j + 1]), "r"(o[4 * j + 2]), "r"(o[4 * j + 3]) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && mrow0 < p.M && nb0 < p.N) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&ymap), "r"(stg), "r"(nb0), "r"(mrow0) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      } else {
      if (half == 0 || two) {
        const int m = m0 + half * 256 + (int)rank * 128 + q * 32 + lane;
        const uint32_t trow = tmem + half * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
        for (int cc = chalf * 4; cc < chalf * 4 + 4; ++cc) {
          uint32_t rr[32];
          tmem_ld32(trow + cc * 32, rr);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int nb0 = n0 + cc * 32;
          if (m < p.M && nb0 < p.N) {
            const bool full = nb0 + 32 <= p.N && (y_ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(y_ptr) & 15) == 0);
            if (full && y_dt != PE_F32) {
              uint32_t o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float a = __uint_as_float(rr[2 * j]), b = __uint_as_float(rr[2 * j + 1]);
                if (bias_ptr) { a += __half2float(bias_ptr[nb0 + 2 * j]); b += __half2float(bias_ptr[nb0 + 2 * j + 1]); }
                o[j] = y_dt == PE_F16 ? pack_half2(a, b) : pack_bf16(a, b);
              }
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y_ptr) + (int64_t)m * y_ld + nb0);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            } else if (y_dt == PE_F32 && nb0 + 32 <= p.N && (y_ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(y_ptr) & 15) == 0)) {
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(y_ptr) + (int64_t)m * y_ld + nb0);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(rr[4 * j]), __uint_as_float(rr[4 * j + 1]), __uint_as_float(rr[4 * j + 2]),
                                       __uint_as_float(rr[4 * j + 3]));
                if (bias_ptr) {
                  v.x += __half2float(bias_ptr[nb0 + 4 * j]); v.y += __half2float(bias_ptr[nb0 + 4 * j + 1]);
                  v.z += __half2float(bias_ptr[nb0 + 4 * j + 2]); v.w += __half2float(bias_ptr[nb0 + 4 * j + 3]);
                }
                dst[j] = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (nb0 + j < p.N) {
                  float a = __uint_as_float(rr[j]);
                  if (bias_ptr) a += __half2float(bias_ptr[nb0 + j]);
                  store_from_float(y_ptr, y_dt, (int64_t)m * y_ld + nb0 + j, a);
                }
              }
            }
          }
        }
      }
      }
      // the next tile's first MMA overwrites the accumulators: it waits for every decode warp of the pair
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(acc_empty);
        else mbar_arrive_remote(acc_empty + lead);
      }
      if (tma_out) {
        // no warp writes a weight stage of the next tile before every warp's staging has been read
        if (lane == 0) {
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          mbar_arrive(stg_free);
        }
        const bool ok = mbar_wait(stg_free, tcount & 1, abort_flag, p.status, 10);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores complete before the CTA leaves
  }

  // ---------------- common exit: nobody leaves while the other CTA may still signal or read here ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag && tid == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

// Activation preparation: (pad + FWHT for raw input), bf16, kernel K order.
// One warp per (row, 128-block).
// Grouped launches: row m of the prepared matrix is row x_rows[m] of x (a gather by token id), and only the first
// valid_rows[0] + valid_rows[1] rows exist (the rest of the list is undefined and is written as zeros).
__global__ void __launch_bounds__(256) gemm_prep_kernel(const void* x, int x_kind, int x_dtype, int64_t ld_x, int in_f,
                                                        __nv_bfloat16* xq, int M, int K, int pair_layout, const int* x_rows,
                                                        const int* valid_rows, int* status) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;  // the matmul's status word (it follows in stream order)
  // Grid-stride over the (row, block) items, four per trip with their loads issued together: one item is only 256
  // bytes in and 256 out, and a warp that handles one item per launch slot spends its life in launch and latency.
  constexpr int U = 4;
  const int lane = threadIdx.x & 31;
  const int nb = K / kBlock;
  const int64_t items = (int64_t)M * nb;
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const bool vin = (ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  const int n_live = valid_rows ? valid_rows[0] + valid_rows[1] : M;
  const int limit = x_kind == PE_X_RAW ? in_f : K;
  for (int64_t w0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w0 < items; w0 += n_warps * U) {
    Raw4 raw[U];
    int m[U], blk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t w = w0 + u * n_warps;
      const bool on = w < items;
      m[u] = on ? (int)(w / nb) : 0;
      blk[u] = on ? (int)(w - (int64_t)m[u] * nb) : 0;
      const bool live = on && m[u] < n_live;
      const int64_t src_row = (x_rows && live) ? x_rows[m[u]] : m[u];
      raw[u] = load4_raw(x, x_dtype, src_row * ld_x, blk[u] * kBlock + lane * 4, live ? limit : 0, vin);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (w0 + u * n_warps >= items) break;  // warp-uniform
      float v[4];
      cvt4(raw[u], x_dtype, v);
      if (x_kind == PE_X_RAW) warp_fwht128(v, lane);
      __nv_bfloat16* dst = xq + (int64_t)m[u] * K + blk[u] * kBlock;
      if (pair_layout) {
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[i], 16);
        if (lane < 16)  // positions 8*lane .. 8*lane+7 = pairs (k, k+64), k = 4*lane..4*lane+3
          *reinterpret_cast<uint4*>(dst + 8 * lane) = make_uint4(pack_bf16(v[0], o[0]), pack_bf16(v[1], o[1]),
                                                                 pack_bf16(v[2], o[2]), pack_bf16(v[3], o[3]));
      } else {
        *reinterpret_cast<uint2*>(dst + 4 * lane) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
      }
    }
  }
}

// Sum of the K-split partials of a dense launch, in split order (bit-reproducible), plus bias, to the output type.
__global__ void __launch_bounds__(256) gemm_splitk_reduce_kernel(const float* part, int ksplit, int M, int N, const __half* bias,
                                                                 void* y, int y_dtype, int64_t ld_y) {
  const int64_t total = (int64_t)M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i - (int64_t)m * N);
    float s = 0.f;
    for (int k = 0; k < ksplit; ++k) s += part[(size_t)k * total + i];
    if (bias) s += __half2float(bias[n]);
    store_from_float(y, y_dtype, (int64_t)m * ld_y + n, s);
  }
}

// Tile list of a grouped launch from the experts' row ranges (first, count): for every expert its
// ceil(count / 256) activation tiles x tiles_n weight tiles, weight tiles of one activation tile adjacent
// (CTAs that run side by side then share the activation tile in L2).  One thread scans, the block writes.
__global__ void __launch_bounds__(256) gemm_group_tiles_kernel(const int* expert_rows, int n_experts, int tiles_n, int max_tiles,
                                                               int4* tiles, int* n_tiles) {
  __shared__ int first_tile[1025];
  __shared__ int2 span[1024];  // (first row, rows) of every expert: read once, in parallel
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) span[e] = make_int2(expert_rows[2 * e], expert_rows[2 * e + 1]);
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < n_experts; ++e) {
      first_tile[e] = t;
      t += ((span[e].y + kTileM - 1) / kTileM) * tiles_n;
    }
    first_tile[n_experts] = t;
    *n_tiles = t < max_tiles ? t : max_tiles;
  }
  __syncthreads();
  // one warp per expert at a time
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int e = warp; e < n_experts; e += n_warps) {
    const int first = span[e].x, cnt = span[e].y;
    const int nt = first_tile[e + 1] - first_tile[e];
    for (int i = lane; i < nt; i += 32) {
      const int mt = i / tiles_n, ntile = i - mt * tiles_n;
      const int rows = cnt - mt * kTileM;
      if (first_tile[e] + i < max_tiles)
        tiles[first_tile[e] + i] = make_int4(first + mt * kTileM, rows < kTileM ? rows : kTileM, ntile * kTileN, e);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// CTAs of the preparation kernel: eight resident per SM, fewer for small inputs (a warp takes four items per trip)
static unsigned prep_grid(int64_t items, int sms) {
  const int64_t want = (items + 31) / 32;
  const int64_t cap = (int64_t)sms * 8;
  return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace pe

using namespace pe;

// K ranges per tile for a dense launch of up to 256 rows: with 16 tiles of a 4096-row layer on 148 SMs, each walking
// the whole K, nine tenths of the GPU idle; the K steps of a tile are spread over the SMs instead.
static int gemm_ksplit(int m, int out_f, int in_f_padded, int sms) {
  if (m > 256) return 1;
  const int tiles = ((m + kTileM - 1) / kTileM) * ((out_f + kTileN - 1) / kTileN);
  const int ksteps = in_f_padded / kStepK;
  int s = sms / tiles;
  if (s > ksteps / 4) s = ksteps / 4;  // at least four K steps per unit
  return s < 2 ? 1 : s;
}

// K ranges per 512-row pair tile: as many as there are idle pairs, at least eight K steps each; two ranges only for a
// long K (the fp32 partials and their sum cost about what halving a short tile saves).
static int pair_ksplit(int ptiles, int ksteps, int sms) {
  int ks = (sms / 2) / ptiles;
  if (ks > ksteps / 8) ks = ksteps / 8;
  if (ks == 2 && ksteps < 128) ks = 1;
  return ks < 2 ? 1 : ks;
}

// workspace: [status word, padded to 256 B][bf16 activations M x K]
extern "C" size_t pe_gemm_workspace_bytes(int m, int in_f_padded) {
  if (m < 1 || in_f_padded < kBlock || in_f_padded % kBlock) return 0;
  return 256 + (size_t)m * in_f_padded * 2;
}

// [the above][fp32 partials ksplit x M x N]: with this much room a launch of up to 256 rows on few tiles splits K
extern "C" size_t pe_gemm_workspace_bytes_splitk(int m, int out_f, int in_f_padded) {
  const size_t base = pe_gemm_workspace_bytes(m, in_f_padded);
  if (base == 0 || out_f < 1) return 0;
  const int sms = sm_count();
  int ks = sms > 0 ? gemm_ksplit(m, out_f, in_f_padded, sms) : 1;
  if (m > 256 && sms >= 2) {  // pairs of CTAs, 512-row tiles, at least eight K steps per unit
    const int ptiles = ((m + kPairTileM - 1) / kPairTileM) * ((out_f + kTileN - 1) / kTileN);
    ks = pair_ksplit(ptiles, in_f_padded / kStepK, sms);
  }
  return ks > 1 ? ((base + 255) & ~(size_t)255) + (size_t)ks * m * out_f * sizeof(float) : base;
}

extern "C" int pe_gemm(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                       const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
                       int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int m, int out_f, int in_f_padded,
                       void* workspace, size_t workspace_bytes, void* stream) {
  if (!codes || !norms || !ct_scaled || !x || !y || !workspace) return PE_ERR_ARG;
  if (m < 1 || out_f < 1 || in_f < 1 || in_f > in_f_padded) return PE_ERR_ARG;
  if (x_kind != PE_X_ROTATED && x_kind != PE_X_RAW) return PE_ERR_ARG;
  if (x_dtype < PE_F32 || x_dtype > PE_BF16 || y_dtype < PE_F32 || y_dtype > PE_BF16) return PE_ERR_ARG;
  if (n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (in_f_padded % kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15)) return PE_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return PE_ERR_ALIGN;
  if (workspace_bytes < pe_gemm_workspace_bytes(m, in_f_padded)) return PE_ERR_WORKSPACE;
  if (ld_codes < (packed ? in_f_padded / 2 : in_f_padded) || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  if (ld_x < (x_kind == PE_X_RAW ? in_f : in_f_padded) || ld_y < out_f) return PE_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return PE_ERR_CUDA;

  int* status = static_cast<int*>(workspace);
  __nv_bfloat16* xq = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(workspace) + 256);
  const int nb = in_f_padded / kBlock;
  const int64_t warps = (int64_t)m * nb;
  gemm_prep_kernel<<<prep_grid(warps, sms), 256, 0, st>>>(x, x_kind, x_dtype, ld_x, in_f, xq, m, in_f_padded,
                                                           packed ? 1 : 0, nullptr, nullptr, status);
  PE_CUDA_TRY(cudaGetLastError());

  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)in_f_padded, (cuuint64_t)m};
  const cuuint64_t strides[1] = {(cuuint64_t)in_f_padded * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStepK, 128};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xq, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PE_ERR_CUDA;

  GemmArgs a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const __half*>(norms); a.ld_norms = ld_norms;
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = static_cast<const __half*>(bias);
  a.M = m; a.N = out_f; a.K = in_f_padded;
  a.tiles_m = (m + kTileM - 1) / kTileM;
  a.tiles_n = (out_f + kTileN - 1) / kTileN;
  a.status = status;
  a.gtiles = nullptr; a.n_gtiles = nullptr; a.grp_norm_stride = 0; a.y_tma = 0; a.ksplit = 1; a.part = nullptr;
  a.lut_bytes = (packed ? 256 : n_levels) * 128;
  const int code_row = packed ? 32 : 64;
  const int code_stage = kTileN * code_row;
  const unsigned fixed = kXStages * 2 * kXTileBytes + kWStages * kWTileBytes + a.lut_bytes + 256 + 1024;
  a.nc = kGroups;  // a decode group owns its code stage
  const unsigned smem_bytes = fixed + a.nc * code_stage;

  // codes as a 2-D byte tensor (row stride ld_codes), boxes of 256 rows x one K step
  CUtensorMap cmap;
  const cuuint64_t cdims[2] = {(cuuint64_t)(packed ? in_f_padded / 2 : in_f_padded), (cuuint64_t)out_f};
  const cuuint64_t cstrides[1] = {(cuuint64_t)ld_codes};
  const cuuint32_t cbox[2] = {(cuuint32_t)code_row, (cuuint32_t)kTileN};
  if (enc(&cmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(codes), cdims, cstrides, cbox, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PE_ERR_CUDA;

  if (m > 256 && sms >= 2) {
    // more than one 256-token tile: pairs of CTAs, each decoding half of the weight tile
    a.tiles_m = (m + kPairTileM - 1) / kPairTileM;
    const int pair_code_stage = 128 * code_row;
    if (packed) a.lut_bytes = 256 * kPairLutStride;
    const unsigned pair_fixed = (packed ? 4 : 3) * 2 * kXTileBytes + kPairWStages * kPairWTileBytes + a.lut_bytes + 256 + 1024;
    a.nc = kPairCodeStages;
    const unsigned pair_smem = pair_fixed + a.nc * pair_code_stage;
    if (pair_smem <= 232448u) {
      CUtensorMap pmap;
      const cuuint32_t pbox[2] = {(cuuint32_t)code_row, 128};
      if (enc(&pmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(codes), cdims, cstrides, pbox, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return PE_ERR_CUDA;
      CUtensorMap ymap = pmap;  // a valid map also when the kernel does not use it
      a.y_tma = (y_dtype != PE_F32 && ld_y % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) ? 1 : 0;
      if (a.y_tma) {
        const cuuint64_t ydims[2] = {(cuuint64_t)out_f, (cuuint64_t)m};
        const cuuint64_t ystrides[1] = {(cuuint64_t)ld_y * 2};
        const cuuint32_t ybox[2] = {32, 32};
        if (enc(&ymap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, y, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
          return PE_ERR_CUDA;
      }
      // few pair tiles: split K when the workspace has room for the partials
      {
        const int ptiles = a.tiles_m * a.tiles_n, ksteps = in_f_padded / kStepK;
        a.ksplit = pair_ksplit(ptiles, ksteps, sms);
        const size_t part_off = (pe_gemm_workspace_bytes(m, in_f_padded) + 255) & ~(size_t)255;
        if (a.ksplit > 1 && workspace_bytes < part_off + (size_t)a.ksplit * m * out_f * sizeof(float)) a.ksplit = 1;
        a.part = a.ksplit > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + part_off) : nullptr;
      }
      const int pair_tiles = a.tiles_m * a.tiles_n * a.ksplit;
      const int pairs = pair_tiles < sms / 2 ? pair_tiles : sms / 2;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * pairs);
      cfg.blockDim = dim3(kPairThreads);
      cfg.dynamicSmemBytes = pair_smem;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (packed) {
        PE_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        PE_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<true>, a, map, pmap, ymap));
      } else {
        PE_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        PE_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<false>, a, map, pmap, ymap));
      }
      if (a.ksplit > 1) {
        const int64_t total = (int64_t)m * out_f;
        const unsigned rgrid = (unsigned)((total + 255) / 256 < (int64_t)sms * 8 ? (total + 255) / 256 : (int64_t)sms * 8);
        gemm_splitk_reduce_kernel<<<rgrid, 256, 0, st>>>(a.part, a.ksplit, m, out_f, a.bias, y, y_dtype, ld_y);
        PE_CUDA_TRY(cudaGetLastError());
      }
      return PE_OK;
    }
    a.tiles_m = (m + kTileM - 1) / kTileM;
    a.ksplit = 1; a.part = nullptr;
    a.nc = kGroups;
    a.lut_bytes = (packed ? 256 : n_levels) * 128;
  }
  // few tiles: split K when the caller's workspace has room for the partials
  a.ksplit = gemm_ksplit(m, out_f, in_f_padded, sms);
  const size_t part_off = (pe_gemm_workspace_bytes(m, in_f_padded) + 255) & ~(size_t)255;
  if (a.ksplit > 1 && workspace_bytes < part_off + (size_t)a.ksplit * m * out_f * sizeof(float)) a.ksplit = 1;
  a.part = a.ksplit > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + part_off) : nullptr;
  const int tiles = a.tiles_m * a.tiles_n * a.ksplit;
  const int grid = tiles < sms ? tiles : sms;
  if (packed) {
    PE_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    gemm_kernel<true><<<grid, kGemmThreads, smem_bytes, st>>>(a, map, cmap);
  } else {
    PE_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    gemm_kernel<false><<<grid, kGemmThreads, smem_bytes, st>>>(a, map, cmap);
  }
  PE_CUDA_TRY(cudaGetLastError());
  if (a.ksplit > 1) {
    const int64_t total = (int64_t)m * out_f;
    const unsigned rgrid = (unsigned)((total + 255) / 256 < (int64_t)sms * 8 ? (total + 255) / 256 : (int64_t)sms * 8);
    gemm_splitk_reduce_kernel<<<rgrid, 256, 0, st>>>(a.part, a.ksplit, m, out_f, a.bias, y, y_dtype, ld_y);
    PE_CUDA_TRY(cudaGetLastError());
  }
  return PE_OK;
}

// ---- grouped launch: the experts of a mixture layer, prefill-size batches ----------------------------
// workspace: [status, 256 B][tile count, 256 B][tile list][bf16 activations rows x K]
static int grouped_max_tiles(int n_experts, int rows, int out_f) {
  return (n_experts + rows / kTileM) * ((out_f + kTileN - 1) / kTileN);
}

extern "C" size_t pe_gemm_grouped_workspace_bytes(int n_experts, int rows, int out_f, int in_f_padded) {
  if (n_experts < 1 || n_experts > 1024 || rows < 1 || out_f < 1 || in_f_padded < kBlock || in_f_padded % kBlock) return 0;
  const size_t list = ((size_t)grouped_max_tiles(n_experts, rows, out_f) * 16 + 255) & ~(size_t)255;
  return 512 + list + (size_t)rows * in_f_padded * 2;
}

extern "C" int pe_gemm_grouped(const void* codes, int packed, int64_t ld_codes, int64_t codes_stride, const void* norms,
                               int64_t ld_norms, int64_t norms_stride, const float* ct_scaled, int n_levels, const void* x,
                               int x_kind, int x_dtype, int64_t ld_x, int in_f, const int32_t* x_rows, void* y, int y_dtype,
                               int64_t ld_y, const int32_t* expert_rows, int n_experts, int rows, int out_f, int in_f_padded,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (!codes || !norms || !ct_scaled || !x || !y || !expert_rows || !workspace) return PE_ERR_ARG;
  if (n_experts < 1 || rows < 1 || out_f < 1 || in_f < 1 || in_f > in_f_padded) return PE_ERR_ARG;
  if (n_experts > 1024) return PE_ERR_LIMIT;
  if (x_kind != PE_X_ROTATED && x_kind != PE_X_RAW) return PE_ERR_ARG;
  if (x_dtype < PE_F32 || x_dtype > PE_BF16 || y_dtype < PE_F32 || y_dtype > PE_BF16) return PE_ERR_ARG;
  if (n_levels < 2 || n_levels > 256 || (packed && n_levels > 16)) return PE_ERR_ARG;
  if (in_f_padded % kBlock) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (ld_codes & 15)) return PE_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return PE_ERR_ALIGN;
  // the experts' code matrices are addressed as one tall 2-D tensor: they must follow each other
  if (codes_stride != (int64_t)out_f * ld_codes) return PE_ERR_ARG;
  if (ld_codes < (packed ? in_f_padded / 2 : in_f_padded) || ld_norms < in_f_padded / kBlock) return PE_ERR_ARG;
  if (ld_x < (x_kind == PE_X_RAW ? in_f : in_f_padded) || ld_y < out_f) return PE_ERR_ARG;
  if ((int64_t)n_experts * out_f > 0x7fffffff) return PE_ERR_LIMIT;
  const size_t need = pe_gemm_grouped_workspace_bytes(n_experts, rows, out_f, in_f_padded);
  if (need == 0) return PE_ERR_SHAPE;
  if (workspace_bytes < need) return PE_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  if (sms <= 0) return PE_ERR_CUDA;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return PE_ERR_CUDA;

  const int max_tiles = grouped_max_tiles(n_experts, rows, out_f);
  const size_t list_bytes = ((size_t)max_tiles * 16 + 255) & ~(size_t)255;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  int* n_tiles = reinterpret_cast<int*>(ws + 256);
  int4* tiles = reinterpret_cast<int4*>(ws + 512);
  __nv_bfloat16* xq = reinterpret_cast<__nv_bfloat16*>(ws + 512 + list_bytes);
  const int tiles_n = (out_f + kTileN - 1) / kTileN;  // (the preparation kernel clears the status word)
  gemm_group_tiles_kernel<<<1, 256, 0, st>>>(expert_rows, n_experts, tiles_n, max_tiles, tiles, n_tiles);
  PE_CUDA_TRY(cudaGetLastError());
  const int nb = in_f_padded / kBlock;
  const int64_t warps = (int64_t)rows * nb;
  gemm_prep_kernel<<<prep_grid(warps, sms), 256, 0, st>>>(x, x_kind, x_dtype, ld_x, in_f, xq, rows, in_f_padded,
                                                           packed ? 1 : 0, x_rows, expert_rows + 2 * (n_experts - 1), status);
  PE_CUDA_TRY(cudaGetLastError());

  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)in_f_padded, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)in_f_padded * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStepK, 128};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xq, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PE_ERR_CUDA;

  GemmArgs a;
  a.codes = static_cast<const uint8_t*>(codes); a.ld_codes = ld_codes;
  a.norms = static_cast<const __half*>(norms); a.ld_norms = ld_norms;
  a.ct = ct_scaled; a.n_levels = n_levels;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.bias = nullptr;
  a.M = rows; a.N = out_f; a.K = in_f_padded;
  a.tiles_m = 1; a.tiles_n = tiles_n;
  a.status = status;
  a.gtiles = tiles; a.n_gtiles = n_tiles; a.grp_norm_stride = norms_stride; a.y_tma = 0; a.ksplit = 1; a.part = nullptr;
  a.lut_bytes = (packed ? 256 : n_levels) * 128;
  const int code_row = packed ? 32 : 64;
  const int code_stage = kTileN * code_row;
  const unsigned fixed = kXStages * 2 * kXTileBytes + kWStages * kWTileBytes + a.lut_bytes + 256 + 1024;
  a.nc = kGroups;  // a decode group owns its code stage
  const unsigned smem_bytes = fixed + a.nc * code_stage;

  CUtensorMap cmap;
  const cuuint64_t cdims[2] = {(cuuint64_t)(packed ? in_f_padded / 2 : in_f_padded), (cuuint64_t)n_experts * (cuuint64_t)out_f};
  const cuuint64_t cstrides[1] = {(cuuint64_t)ld_codes};
  const cuuint32_t cbox[2] = {(cuuint32_t)code_row, (cuuint32_t)kTileN};
  if (enc(&cmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(codes), cdims, cstrides, cbox, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PE_ERR_CUDA;

  const int grid = max_tiles < sms ? max_tiles : sms;
  if (packed) {
    PE_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    gemm_kernel<true><<<grid, kGemmThreads, smem_bytes, st>>>(a, map, cmap);
  } else {
    PE_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    gemm_kernel<false><<<grid, kGemmThreads, smem_bytes, st>>>(a, map, cmap);
  }
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}
