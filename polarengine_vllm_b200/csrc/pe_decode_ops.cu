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
  pdl_enter();
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
  pdl_enter();
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
  pdl_enter();
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


// Single-query attention over the KV cache for one decode step (grouped-query form), optionally with the
// rotary embedding and the KV-cache write of the new token folded in.
// CTA (kv head, sequence, split): the G = hq / hkv query heads of a kv head share every K and V row; the
// cache positions 0 .. L-1 are cut into `splits` equal ranges so that a one-sequence step still fills the SMs.
//  * A warp owns the positions p_lo + w, p_lo + w + 8, ... of the CTA's range.  Lane l holds elements
//    4l .. 4l+3 of a row: a K or V row is one coalesced 256-byte load per warp, the queries sit in registers.
//    Per position: G dot products (five shuffles each), an online-softmax update of (max, sum, weighted V
//    rows) per head; the rows of six positions are requested together.
//  * The 8 warps meet in shared memory, rescaled to the CTA's maximum.  One split: normalise and store.
//    Several: every CTA leaves (weighted rows, max, sum) in scratch and takes a ticket; the CTA that draws
//    the last ticket merges the splits in split order (bit-reproducible) and returns the ticket counter to
//    zero.  Nobody waits for anybody.
//  * Fused form (qkv != null): q, k, v are the raw rows of the fused q/k/v projection.  Every warp rotates
//    the G queries for itself (rotate-half pairs (j, j + 64) live in lanes l and l + 16); the CTA whose range
//    holds the current position rotates the new key, writes key and value into the caches and uses its
//    registers for that position instead of reading the row back.
constexpr int kAttThreads = 512;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kAttTargetCtas = 128;  // measured on a 640-token cache: 16 / 32 / 64 / 128 CTAs -> 17.6 / 13.2 / 11.4 / 11.0 us per launch
constexpr int kAttMaxGroup = 8;
constexpr int kAttMaxSplits = 16;
constexpr int kAttInFlight = 6;  // positions whose K and V rows a warp requests together

struct AttArgs {
  const __half* q;      // (batch, hq, D) rotated queries, or null in the fused form
  const __half* qkv; int64_t ld_qkv;  // fused form: rows of (hq + 2 hkv) * D raw projection outputs
  __half* k_cache; __half* v_cache;   // (batch, hkv, max_len, D); written at the current position in the fused form
  const int64_t* pos_dev; int64_t pos_host;
  __half* out;          // (batch, hq * D)
  int hq, hkv, max_len;
  float scale, theta;
  float* parts; unsigned* tickets;
};

__device__ __forceinline__ void half4_to_float(const uint2& u, float f[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// rotate-half rotary embedding of the 4 elements a lane holds (elements 4l..4l+3; the pair partner is 64 away,
// in lane l ^ 16), rounded to fp16 as pe_rope_cache stores them
__device__ __forceinline__ void rope4(float x[4], const float c[4], const float s[4], int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float o = __shfl_xor_sync(0xffffffffu, x[i], 16);
    const float r = lane < 16 ? x[i] * c[i] - o * s[i] : x[i] * c[i] + o * s[i];
    x[i] = __half2float(__float2half_rn(r));
  }
}

template <int D, int G>
__device__ __forceinline__ void attention_body(const AttArgs& p, float* att_smem) {
  static_assert(D == 128, "a row is 32 lanes x 4 elements");
  __shared__ unsigned my_ticket;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z, splits = gridDim.z;
  const int64_t pos = p.pos_dev ? *p.pos_dev : p.pos_host;
  const int64_t len64 = pos + 1;  // the current token counts
  const int L = (int)(len64 < 1 ? 1 : (len64 > p.max_len ? p.max_len : len64));
  const int chunk = (L + splits - 1) / splits;
  const int p_lo = sp * chunk, p_hi = p_lo + chunk < L ? p_lo + chunk : L;
  __half* kb = p.k_cache + ((int64_t)b * p.hkv + kvh) * (int64_t)p.max_len * D;
  __half* vb = p.v_cache + ((int64_t)b * p.hkv + kvh) * (int64_t)p.max_len * D;
  const bool fused = p.qkv != nullptr;
  const int cur = fused && pos >= 0 && pos < p.max_len ? (int)pos : -1;  // position whose K/V rows come from qkv

  // ---- queries (and, fused, the new key / value) in registers
  float q[G][4], knew[4] = {0.f, 0.f, 0.f, 0.f}, vnew[4] = {0.f, 0.f, 0.f, 0.f};
  if (fused) {
    __shared__ float rope_c[D / 2], rope_s[D / 2];  // computed once per CTA: large angles take the slow path of cosf / sinf
    if (tid < D / 2) {
      const float inv = 1.f / powf(p.theta, (float)(2 * tid) / (float)D);
      const float ang = (float)pos * inv;
      rope_c[tid] = cosf(ang);
      rope_s[tid] = sinf(ang);
    }
    __syncthreads();
    float c[4], s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c[i] = rope_c[(lane & 15) * 4 + i];
      s[i] = rope_s[(lane & 15) * 4 + i];
    }
    const __half* row = p.qkv + (int64_t)b * p.ld_qkv;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      half4_to_float(*reinterpret_cast<const uint2*>(row + ((int64_t)kvh * G + g) * D + lane * 4), q[g]);
      rope4(q[g], c, s, lane);
    }
    half4_to_float(*reinterpret_cast<const uint2*>(row + ((int64_t)p.hq + kvh) * D + lane * 4), knew);
    rope4(knew, c, s, lane);
    const uint2 vraw = *reinterpret_cast<const uint2*>(row + ((int64_t)p.hq + p.hkv + kvh) * D + lane * 4);
    half4_to_float(vraw, vnew);
    if (w == 0 && cur >= p_lo && cur < p_hi) {  // this CTA owns the current position: one warp fills the caches
      *reinterpret_cast<uint2*>(kb + (int64_t)cur * D + lane * 4) = make_uint2(pack_half2(knew[0], knew[1]), pack_half2(knew[2], knew[3]));
      *reinterpret_cast<uint2*>(vb + (int64_t)cur * D + lane * 4) = vraw;
    }
  } else {
#pragma unroll
    for (int g = 0; g < G; ++g)
      half4_to_float(*reinterpret_cast<const uint2*>(p.q + ((int64_t)b * p.hq + (int64_t)kvh * G + g) * D + lane * 4), q[g]);
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i) q[g][i] *= p.scale;

  // ---- this warp's positions, online softmax
  float m[G], l[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }
  // Rows of kAttInFlight positions are requested together, before any of them is used: a warp's share of a
  // 640-token cache (at most 5 positions with 16 ranges) costs one memory round trip, not one per position.
  constexpr int U = kAttInFlight;
  for (int p0 = p_lo + w; p0 < p_hi; p0 += kAttWarps * U) {
    uint2 kr[U], vr[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int pp = p0 + u * kAttWarps;
      kr[u] = vr[u] = make_uint2(0, 0);
      if (pp < p_hi && pp != cur) {
        kr[u] = *reinterpret_cast<const uint2*>(kb + (int64_t)pp * D + lane * 4);
        vr[u] = *reinterpret_cast<const uint2*>(vb + (int64_t)pp * D + lane * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int pp = p0 + u * kAttWarps;
      if (pp < p_hi) {  // warp-uniform
        float kf[4], vf[4];
        if (pp == cur) {
#pragma unroll
          for (int i = 0; i < 4; ++i) { kf[i] = knew[i]; vf[i] = vnew[i]; }
        } else {
          half4_to_float(kr[u], kf);
          half4_to_float(vr[u], vf);
        }
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = q[g][0] * kf[0] + q[g][1] * kf[1] + q[g][2] * kf[2] + q[g][3] * kf[3];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
#pragma unroll
          for (int g = 0; g < G; ++g) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], o);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float mn = fmaxf(m[g], sc[g]);
          const float corr = __expf(m[g] - mn), e = __expf(sc[g] - mn);
          m[g] = mn;
          l[g] = l[g] * corr + e;
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[g][i] = acc[g][i] * corr + e * vf[i];
        }
      }
    }
  }

  // ---- the warps meet: [warp][G][D] weighted rows, [warp][G] maxima and sums
  float* racc = att_smem;                            // kAttWarps * G * D
  float* rm = racc + kAttWarps * G * D;              // kAttWarps * G
  float* rl = rm + kAttWarps * kAttMaxGroup;         // kAttWarps * G
#pragma unroll
  for (int g = 0; g < G; ++g) {
    *reinterpret_cast<float4*>(racc + (w * G + g) * D + lane * 4) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    if (lane == 0) { rm[w * kAttMaxGroup + g] = m[g]; rl[w * kAttMaxGroup + g] = l[g]; }
  }
  __syncthreads();
  __half* op = p.out + ((int64_t)b * p.hq + (int64_t)kvh * G) * D;
  const size_t head = (size_t)b * p.hkv + kvh;
  float* part = p.parts ? p.parts + (head * splits + sp) * G * (D + 2) : nullptr;
  for (int i = tid; i < G * D; i += kAttThreads) {
    const int g = i / D, d = i % D;
    float mx = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < kAttWarps; ++ww) mx = fmaxf(mx, rm[ww * kAttMaxGroup + g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int ww = 0; ww < kAttWarps; ++ww) {
      const float lw = rl[ww * kAttMaxGroup + g];
      if (lw > 0.f) {  // a warp without positions has no maximum
        const float f = __expf(rm[ww * kAttMaxGroup + g] - mx);
        num += racc[(ww * G + g) * D + d] * f;
        den += lw * f;
      }
    }
    if (splits == 1) {
      op[i] = __float2half_rn(num / den);
    } else {  // this split's record: [G][D + 2] = weighted rows, maximum, sum
      part[g * (D + 2) + d] = num;
      if (d == 0) { part[g * (D + 2) + D] = mx; part[g * (D + 2) + D + 1] = den; }
    }
  }
  if (splits == 1) return;
  unsigned* ticket = p.tickets + head;
  __threadfence();
  __syncthreads();
  if (tid == 0) my_ticket = atomicAdd(ticket, 1u);
  __syncthreads();
  if (my_ticket != (unsigned)(splits - 1)) return;
  __threadfence();
  const float* all = part - (size_t)sp * G * (D + 2);  // record of split 0
  for (int i = tid; i < G * D; i += kAttThreads) {
    const int g = i / D, d = i % D;
    // all three values of every split are requested before any is used: one memory round trip, not one per split
    float mv[kAttMaxSplits], lv[kAttMaxSplits], nv[kAttMaxSplits];
#pragma unroll
    for (int s2 = 0; s2 < kAttMaxSplits; ++s2) {
      const float* rec = all + ((size_t)(s2 < splits ? s2 : 0) * G + g) * (D + 2);
      mv[s2] = __ldcg(rec + D);
      lv[s2] = s2 < splits ? __ldcg(rec + D + 1) : 0.f;
      nv[s2] = __ldcg(rec + d);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int s2 = 0; s2 < kAttMaxSplits; ++s2) mx = fmaxf(mx, lv[s2] > 0.f ? mv[s2] : -INFINITY);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kAttMaxSplits; ++s2) {
      const float f = lv[s2] > 0.f ? __expf(mv[s2] - mx) : 0.f;  // an empty split has no maximum
      num += (lv[s2] > 0.f ? nv[s2] : 0.f) * f;
      den += lv[s2] * f;
    }
    op[i] = __float2half_rn(num / den);
  }
  if (tid == 0) *ticket = 0u;
}

template <int D>
__global__ void __launch_bounds__(kAttThreads) decode_attention_kernel(const AttArgs p) {
  extern __shared__ __align__(16) float att_smem[];
  pdl_enter();
  switch (p.hq / p.hkv) {
    case 1: attention_body<D, 1>(p, att_smem); break;
    case 2: attention_body<D, 2>(p, att_smem); break;
    case 4: attention_body<D, 4>(p, att_smem); break;
    case 8: attention_body<D, 8>(p, att_smem); break;
    default: break;
  }
}

// ---- many sequences: thread per cache position -------------------------------------------------------
// With dozens of (sequence, kv head) pairs the launch fills the SMs without cutting the cache finely, and the
// warp-per-position form above pays five shuffles per dot product for nothing.  Here a thread owns a cache
// position for the scores (the 16 16-byte pieces of its K row requested together, the full 128-wide dot per
// query head with the queries broadcast from shared memory), one warp per query head does the softmax, and
// the V rows are summed with thread = (position stride 16, 16-byte piece), eight rows in flight per thread.
// Same split / ticket / merge scheme and the same scratch layout.
constexpr int kAttWideThreads = 256;
constexpr int kAttWideMaxSplits = 8;

template <int D, int G>
__device__ __forceinline__ void attention_wide_body(const __half* q, const __half* kb, const __half* vb, __half* out_row, float* att_smem,
                                               int p_lo, int p_hi, int chunk_cap, float scale, int splits, float* part,
                                               unsigned* ticket) {
  static_assert(D == 128, "pieces and thread mapping are laid out for 128-wide heads");
  __shared__ float head_max[kAttMaxGroup], head_sum[kAttMaxGroup];
  __shared__ unsigned my_ticket;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int n = p_hi > p_lo ? p_hi - p_lo : 0;
  float* qs = att_smem;                 // [G][D]
  float* sc = qs + kAttMaxGroup * D;    // [G][chunk_cap]
  float* red = sc + G * chunk_cap;      // [16 position groups][G][D]
  for (int i = tid; i < G * D; i += kAttWideThreads) qs[i] = __half2float(q[i]) * scale;
  __syncthreads();
  for (int i = tid; i < n; i += kAttWideThreads) {
    uint4 u[D / 8];
    const uint4* row = reinterpret_cast<const uint4*>(kb + (int64_t)(p_lo + i) * D);
#pragma unroll
    for (int c = 0; c < D / 8; ++c) u[c] = row[c];
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = 0.f;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&u[c]);
      float kf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        kf[2 * j] = f.x;
        kf[2 * j + 1] = f.y;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float4 qa = *reinterpret_cast<const float4*>(qs + g * D + c * 8);
        const float4 qb = *reinterpret_cast<const float4*>(qs + g * D + c * 8 + 4);
        acc[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) sc[g * chunk_cap + i] = acc[g];
  }
  __syncthreads();
  if (w < G) {  // head w: maximum, exponentials (kept unnormalised), sum
    float* sh = sc + w * chunk_cap;
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, sh[i]);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float e = __expf(sh[i] - m);
      sh[i] = e;
      sum += e;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) { head_max[w] = m; head_sum[w] = sum; }
  }
  __syncthreads();
  {
    const int ps = tid >> 4, piece = tid & 15;
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    constexpr int U = 8;
    for (int i0 = ps; i0 < n; i0 += 16 * U) {
      uint4 u[U];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int i = i0 + 16 * j;
        u[j] = i < n ? *reinterpret_cast<const uint4*>(vb + (int64_t)(p_lo + i) * D + piece * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int i = i0 + 16 * j;
        if (i < n) {
          const __half2* h2 = reinterpret_cast<const __half2*>(&u[j]);
          float vf[8];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 f = __half22float2(h2[c]);
            vf[2 * c] = f.x;
            vf[2 * c + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pr = sc[g * chunk_cap + i];
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[g][c] += pr * vf[c];
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dst = red + (ps * G + g) * D + piece * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
  }
  __syncthreads();
  if (splits == 1) {
    for (int i = tid; i < G * D; i += kAttWideThreads) {
      float v = 0.f;
#pragma unroll
      for (int gs = 0; gs < 16; ++gs) v += red[gs * G * D + i];
      out_row[i] = __float2half_rn(v / head_sum[i / D]);
    }
    return;
  }
  // this split's record: [G][D + 2] = weighted rows, maximum, sum
  for (int i = tid; i < G * D; i += kAttWideThreads) {
    float v = 0.f;
#pragma unroll
    for (int gs = 0; gs < 16; ++gs) v += red[gs * G * D + i];
    part[(i / D) * (D + 2) + (i % D)] = v;
  }
  if (tid < G) { part[tid * (D + 2) + D] = head_max[tid]; part[tid * (D + 2) + D + 1] = head_sum[tid]; }
  __threadfence();
  __syncthreads();
  if (tid == 0) my_ticket = atomicAdd(ticket, 1u);
  __syncthreads();
  if (my_ticket != (unsigned)(splits - 1)) return;
  __threadfence();
  const float* all = part - (size_t)blockIdx.z * G * (D + 2);  // record of split 0
  for (int i = tid; i < G * D; i += kAttWideThreads) {
    const int g = i / D, d = i % D;
    float mv[kAttWideMaxSplits], lv[kAttWideMaxSplits], nv[kAttWideMaxSplits];  // requested together: one memory round trip
#pragma unroll
    for (int s2 = 0; s2 < kAttWideMaxSplits; ++s2) {
      const float* rec = all + ((size_t)(s2 < splits ? s2 : 0) * G + g) * (D + 2);
      mv[s2] = __ldcg(rec + D);
      lv[s2] = s2 < splits ? __ldcg(rec + D + 1) : 0.f;
      nv[s2] = __ldcg(rec + d);
    }
    float m = -INFINITY;
#pragma unroll
    for (int s2 = 0; s2 < kAttWideMaxSplits; ++s2) m = fmaxf(m, lv[s2] > 0.f ? mv[s2] : -INFINITY);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kAttWideMaxSplits; ++s2) {
      const float f = lv[s2] > 0.f ? __expf(mv[s2] - m) : 0.f;  // an empty split has no maximum
      num += (lv[s2] > 0.f ? nv[s2] : 0.f) * f;
      den += lv[s2] * f;
    }
    out_row[i] = __float2half_rn(num / den);
  }
  if (tid == 0) *ticket = 0u;
}

template <int D>
__global__ void __launch_bounds__(kAttWideThreads) decode_attention_wide_kernel(const __half* q, const __half* k_cache, const __half* v_cache,
                                                                        const int64_t* pos_dev, int64_t pos_host, __half* out,
                                                                        int hq, int hkv, int max_len, float scale, float* parts,
                                                                        unsigned* tickets) {
  extern __shared__ __align__(16) float att_smem[];
  const int G = hq / hkv;
  const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z, splits = gridDim.z;
  pdl_enter();
  const int64_t len64 = (pos_dev ? *pos_dev : pos_host) + 1;  // the current token is already in the cache
  const int L = (int)(len64 < 1 ? 1 : (len64 > max_len ? max_len : len64));
  // chunk_cap sizes the score rows in shared memory; a multiple of 4 keeps the float4 area behind them aligned
  const int chunk = (L + splits - 1) / splits, chunk_cap = ((max_len + splits - 1) / splits + 3) & ~3;
  const int p_lo = sp * chunk, p_hi = p_lo + chunk < L ? p_lo + chunk : L;
  const __half* qp = q + ((int64_t)b * hq + (int64_t)kvh * G) * D;
  const __half* kb = k_cache + ((int64_t)b * hkv + kvh) * (int64_t)max_len * D;
  const __half* vb = v_cache + ((int64_t)b * hkv + kvh) * (int64_t)max_len * D;
  __half* op = out + ((int64_t)b * hq + (int64_t)kvh * G) * D;
  const size_t head = (size_t)b * hkv + kvh;
  float* part = parts ? parts + (head * splits + sp) * G * (D + 2) : nullptr;
  unsigned* ticket = tickets ? tickets + head : nullptr;
  switch (G) {
    case 1: attention_wide_body<D, 1>(qp, kb, vb, op, att_smem, p_lo, p_hi, chunk_cap, scale, splits, part, ticket); break;
    case 2: attention_wide_body<D, 2>(qp, kb, vb, op, att_smem, p_lo, p_hi, chunk_cap, scale, splits, part, ticket); break;
    case 4: attention_wide_body<D, 4>(qp, kb, vb, op, att_smem, p_lo, p_hi, chunk_cap, scale, splits, part, ticket); break;
    case 8: attention_wide_body<D, 8>(qp, kb, vb, op, att_smem, p_lo, p_hi, chunk_cap, scale, splits, part, ticket); break;
    default: break;
  }
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
  PE_CUDA_TRY(launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                         static_cast<__half*>(x), delta, delta_dtype, static_cast<const __half*>(weight), static_cast<__half*>(out),
                         hidden, eps));
  return PE_OK;
}

extern "C" int pe_rope_cache(const void* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, void* q_out,
                             void* k_cache, void* v_cache, int batch, int t, int hq, int hkv, int head_dim, int max_len,
                             float theta, void* stream) {
  if (!qkv || !q_out || !k_cache || !v_cache || batch < 1 || t < 1 || hq < 1 || hkv < 1 || max_len < 1) return PE_ERR_ARG;
  if (head_dim < 2 || head_dim > 2048 || (head_dim & 1)) return PE_ERR_SHAPE;
  if (ld_qkv < (int64_t)(hq + 2 * hkv) * head_dim) return PE_ERR_ARG;
  if ((int64_t)batch * t > 0x7fffffff || hq + 2 * hkv > 65535) return PE_ERR_LIMIT;
  PE_CUDA_TRY(launch_pdl(rope_cache_kernel, dim3((unsigned)(batch * t), (unsigned)(hq + 2 * hkv)), dim3(head_dim / 2), 0,
                         static_cast<cudaStream_t>(stream), static_cast<const __half*>(qkv), ld_qkv, pos_dev, pos_host,
                         static_cast<__half*>(q_out), static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), t, hq, hkv,
                         head_dim, max_len, theta));
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
  PE_CUDA_TRY(launch_pdl(silu_mul_kernel, dim3((unsigned)blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                         static_cast<const __half*>(gate_up), ld_gu, static_cast<__half*>(out), ld_out, inter, n_vec));
  return PE_OK;
}

// scratch of the split form: [tickets: one counter per (sequence, kv head), 4 KB, zero before the first
// call and left zero][one record per (sequence, kv head, split, query head of the group)]
extern "C" size_t pe_decode_attention_workspace_bytes(int batch, int hq, int hkv, int head_dim) {
  if (batch < 1 || hq < 1 || hkv < 1 || head_dim != 128 || hq % hkv || (size_t)batch * hkv * 4 > 4096) return 0;
  return 4096 + (size_t)batch * hkv * kAttMaxSplits * (hq / hkv) * (head_dim + 2) * sizeof(float);
}

static int attention_launch(AttArgs a, int batch, int head_dim, void* workspace, size_t workspace_bytes, void* stream) {
  if (!a.k_cache || !a.v_cache || !a.out || batch < 1 || a.hq < 1 || a.hkv < 1 || a.max_len < 1) return PE_ERR_ARG;
  if (head_dim != 128 || a.hq % a.hkv) return PE_ERR_SHAPE;
  const int G = a.hq / a.hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return PE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15) return PE_ERR_ALIGN;
  if (batch > 65535) return PE_ERR_LIMIT;
  // Cut the cache positions into so many ranges that the launch has about kAttTargetCtas CTAs of 16 warps (at
  // most 16 ranges of at least 32 positions of the longest possible sequence, none without a scratch buffer).
  // The cache of a one-sequence step is small; the launch is a chain of memory round trips, and a warp's share
  // of positions is what it adds to that chain, so more and smaller shares are faster.
  int splits = 1;
  const size_t need = pe_decode_attention_workspace_bytes(batch, a.hq, a.hkv, head_dim);
  if (workspace && need && workspace_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 15)) {
    splits = kAttTargetCtas / (a.hkv * batch);
    splits = splits < 1 ? 1 : (splits > kAttMaxSplits ? kAttMaxSplits : splits);
    if (a.max_len < 32 * splits) splits = a.max_len / 32 < 1 ? 1 : a.max_len / 32;
  }
  const size_t smem = ((size_t)kAttWarps * G * 128 + 2 * (size_t)kAttWarps * kAttMaxGroup) * sizeof(float);
  auto kfn = decode_attention_kernel<128>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  PE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(((size_t)kAttWarps * kAttMaxGroup * 128 + 2 * (size_t)kAttWarps * kAttMaxGroup) * sizeof(float))));
    if (dev < 16) configured[dev] = true;
  }
  a.parts = splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 4096) : nullptr;
  a.tickets = splits > 1 ? static_cast<unsigned*>(workspace) : nullptr;
  a.scale = 1.f / sqrtf((float)head_dim);
  PE_CUDA_TRY(launch_pdl(kfn, dim3((unsigned)a.hkv, (unsigned)batch, (unsigned)splits), dim3(kAttThreads), smem,
                         static_cast<cudaStream_t>(stream), a));
  return PE_OK;
}

extern "C" int pe_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos_dev,
                                   int64_t pos_host, void* out, int batch, int hq, int hkv, int head_dim, int max_len,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  if (!q) return PE_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(q) & 7) return PE_ERR_ALIGN;
  AttArgs a = {};
  a.q = static_cast<const __half*>(q);
  a.k_cache = static_cast<__half*>(const_cast<void*>(k_cache));
  a.v_cache = static_cast<__half*>(const_cast<void*>(v_cache));
  a.pos_dev = pos_dev; a.pos_host = pos_host;
  a.out = static_cast<__half*>(out);
  a.hq = hq; a.hkv = hkv; a.max_len = max_len;
  const int sms = sm_count();
  if (sms > 0 && batch >= 1 && hkv >= 1 && (int64_t)batch * hkv * 4 >= sms && head_dim == 128 && hq % hkv == 0 &&
      (hq / hkv == 1 || hq / hkv == 2 || hq / hkv == 4 || hq / hkv == 8) && k_cache && v_cache && out && max_len >= 1 &&
      batch <= 65535 && !((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15)) {
    // many (sequence, kv head) pairs: the thread-per-position kernel
    const int G = hq / hkv;
    int splits = 1;
    const size_t need = pe_decode_attention_workspace_bytes(batch, hq, hkv, head_dim);
    if (workspace && need && workspace_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 15)) {
      splits = sms / (hkv * batch);
      splits = splits < 1 ? 1 : (splits > kAttWideMaxSplits ? kAttWideMaxSplits : splits);
      if (max_len < 64 * splits) splits = max_len / 64 < 1 ? 1 : max_len / 64;
    }
    const int chunk_cap = ((max_len + splits - 1) / splits + 3) & ~3;  // as in the kernel
    const size_t smem = ((size_t)kAttMaxGroup * 128 + (size_t)G * chunk_cap + (size_t)16 * G * 128) * sizeof(float);
    if (smem <= 200 * 1024) {
      auto kfn = decode_attention_wide_kernel<128>;
      static thread_local size_t configured[16] = {0};
      int dev = 0;
      PE_CUDA_TRY(cudaGetDevice(&dev));
      if (smem > 48 * 1024 && (dev >= 16 || configured[dev] < smem)) {
        PE_CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev < 16) configured[dev] = smem;
      }
      float* parts = splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 4096) : nullptr;
      unsigned* tickets = splits > 1 ? static_cast<unsigned*>(workspace) : nullptr;
      PE_CUDA_TRY(launch_pdl(kfn, dim3((unsigned)hkv, (unsigned)batch, (unsigned)splits), dim3(kAttWideThreads), smem,
                             static_cast<cudaStream_t>(stream), static_cast<const __half*>(q), static_cast<const __half*>(k_cache),
                             static_cast<const __half*>(v_cache), pos_dev, pos_host, static_cast<__half*>(out), hq, hkv, max_len,
                             1.f / sqrtf((float)head_dim), parts, tickets));
      return PE_OK;
    }
  }
  return attention_launch(a, batch, head_dim, workspace, workspace_bytes, stream);
}

extern "C" int pe_rope_attention(const void* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, void* k_cache,
                                 void* v_cache, void* out, int batch, int hq, int hkv, int head_dim, int max_len, float theta,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!qkv) return PE_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(qkv) & 7) || (ld_qkv & 3)) return PE_ERR_ALIGN;
  if (hq >= 1 && hkv >= 1 && ld_qkv < (int64_t)(hq + 2 * hkv) * head_dim) return PE_ERR_ARG;
  AttArgs a = {};
  a.qkv = static_cast<const __half*>(qkv); a.ld_qkv = ld_qkv;
  a.k_cache = static_cast<__half*>(k_cache);
  a.v_cache = static_cast<__half*>(v_cache);
  a.pos_dev = pos_dev; a.pos_host = pos_host;
  a.out = static_cast<__half*>(out);
  a.hq = hq; a.hkv = hkv; a.max_len = max_len;
  a.theta = theta;
  return attention_launch(a, batch, head_dim, workspace, workspace_bytes, stream);
}
