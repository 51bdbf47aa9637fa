// Routing bookkeeping of a quantized mixture-of-experts layer, on the device:
//   pe_moe_plan    (token, slot) pairs -> rows grouped by expert + the problem list of
//                  pe_gemv_grouped, in one launch and without a host round trip;
//   pe_moe_combine weighted sum of the experts' outputs back into token order.
// The reference's layer does this with a Python loop over the selected experts
// (nemotron_offload.py:190-226).
#include "pe_common.cuh"

namespace pe {

constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxExperts = 1024;

// One CTA.  Pairs are bucketed by local expert with shared-memory counters; the order of
// the rows inside an expert depends on the arrival order of the atomics, which is harmless:
// every row of a grouped problem is computed independently of its neighbours, and the
// combine step finds a pair's row through `pos`.
__global__ void __launch_bounds__(kPlanThreads) moe_plan_kernel(const int64_t* ids, const int64_t* expert_map, int n_global,
                                                                int n_pairs, int top_k, int n_local, int rows_per_problem, int max_problems,
                                                                int32_t* row_token, int32_t* pos, int4* problems,
                                                                int32_t* expert_rows) {
  __shared__ int cnt[kPlanMaxExperts];     // pairs per expert, then a running cursor
  __shared__ int first[kPlanMaxExperts];   // first row of the expert in the grouped order
  __shared__ int pfirst[kPlanMaxExperts];  // first problem of the expert
  __shared__ int total_problems;
  const int tid = threadIdx.x;
  for (int e = tid; e < n_local; e += kPlanThreads) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < n_pairs; i += kPlanThreads) {
    int64_t e = ids[i];
    if (expert_map) e = (e >= 0 && e < n_global) ? expert_map[e] : -1;  // ids outside the map belong to nobody
    if (e >= 0 && e < n_local) atomicAdd(&cnt[(int)e], 1);
  }
  __syncthreads();
  if (tid == 0) {  // exclusive scans over at most 1024 experts
    int r = 0, pr = 0;
    for (int e = 0; e < n_local; ++e) {
      first[e] = r;
      pfirst[e] = pr;
      r += cnt[e];
      pr += (cnt[e] + rows_per_problem - 1) / rows_per_problem;
    }
    total_problems = pr;
  }
  __syncthreads();
  // problem list: expert e owns problems pfirst[e] .. ; unused slots get zero rows
  for (int e = tid; e < n_local; e += kPlanThreads) {
    const int c = cnt[e];
    if (expert_rows) { expert_rows[2 * e] = first[e]; expert_rows[2 * e + 1] = c; }
    for (int j = 0, p = pfirst[e]; j * rows_per_problem < c && p < max_problems; ++j, ++p) {
      const int rows = c - j * rows_per_problem;
      problems[p] = make_int4(e, first[e] + j * rows_per_problem, rows < rows_per_problem ? rows : rows_per_problem, 0);
    }
  }
  for (int p = total_problems + tid; p < max_problems; p += kPlanThreads) problems[p] = make_int4(0, 0, 0, 0);
  __syncthreads();
  for (int e = tid; e < n_local; e += kPlanThreads) cnt[e] = 0;  // now the cursor inside the expert
  __syncthreads();
  for (int i = tid; i < n_pairs; i += kPlanThreads) {
    int64_t e = ids[i];
    if (expert_map) e = (e >= 0 && e < n_global) ? expert_map[e] : -1;  // ids outside the map belong to nobody
    if (e >= 0 && e < n_local) {
      const int r = first[(int)e] + atomicAdd(&cnt[(int)e], 1);
      row_token[r] = i / top_k;
      pos[i] = r;
    } else {
      pos[i] = -1;  // routed to an expert of another rank
    }
  }
}

// out[t, :] = sum_j w[t, j] * y[pos[t * top_k + j], :] over the slots with pos >= 0, in slot
// order (bit-reproducible); 4 columns per thread.
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* y, int64_t ld_y, const int32_t* pos, const float* w, int top_k,
                                                          void* out, int out_dtype, int64_t ld_out, int hidden, int64_t n_vec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_vec) return;
  const int per_row = hidden >> 2;
  const int64_t t = idx / per_row;
  const int col = (int)(idx - t * per_row) * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < top_k; ++j) {
    const int r = pos[t * top_k + j];
    if (r >= 0) {
      const float wt = w[t * top_k + j];
      const float4 v = *reinterpret_cast<const float4*>(y + (int64_t)r * ld_y + col);
      acc.x += wt * v.x; acc.y += wt * v.y; acc.z += wt * v.z; acc.w += wt * v.w;
    }
  }
  store_from_float(out, out_dtype, t * ld_out + col, acc.x);
  store_from_float(out, out_dtype, t * ld_out + col + 1, acc.y);
  store_from_float(out, out_dtype, t * ld_out + col + 2, acc.z);
  store_from_float(out, out_dtype, t * ld_out + col + 3, acc.w);
}

// Routing of the reference's mixture layer (nemotron_offload.py:180-189) as one launch: fp32 softmax over the experts,
// the top_k largest (ties go to the lower expert id, as a stable descending sort would have them), optional
// renormalisation of the kept weights.  One warp per token; lane l holds experts l, l + 32, ...
constexpr int kRouteMaxPerLane = 32;  // up to 1024 experts
__global__ void __launch_bounds__(256) moe_route_kernel(const void* logits, int dtype, int64_t ld, int n_tokens, int n_experts, int top_k,
                                                        int renormalize, float* weights, int64_t* ids) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  float v[kRouteMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = -INFINITY;
    if (e < n_experts) {
      const int64_t at = (int64_t)tok * ld + e;
      v[i] = dtype == PE_F32 ? static_cast<const float*>(logits)[at]
             : dtype == PE_F16 ? __half2float(static_cast<const __half*>(logits)[at])
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(logits)[at]);
      mx = fmaxf(mx, v[i]);
    }
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    if (lane + 32 * i < n_experts) { v[i] = expf(v[i] - mx); sum += v[i]; }
    else v[i] = -1.f;  // never picked: probabilities are >= 0
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
  const float inv = 1.f / sum;
  float kept = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < top_k; ++k) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i)
      if (v[i] > best) { best = v[i]; best_e = lane + 32 * i; }  // lowest slot of this lane first
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, m);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, m);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i)
        if (i == (best_e >> 5)) v[i] = -1.f;
    }
    const float w = best * inv;
    kept += w;
    if (lane == k) { my_w = w; my_id = best_e; }  // top_k <= 32
  }
  if (lane < top_k) {
    weights[(int64_t)tok * top_k + lane] = renormalize ? my_w / kept : my_w;
    ids[(int64_t)tok * top_k + lane] = my_id;
  }
}

}  // namespace pe

using namespace pe;

extern "C" int pe_moe_plan(const int64_t* topk_ids, const int64_t* expert_map, int n_global_experts, int n_pairs, int top_k,
                           int n_local_experts,
                           int rows_per_problem, int max_problems, int32_t* row_token, int32_t* pos, int32_t* problems,
                           int32_t* expert_rows, void* stream) {
  if (!topk_ids || !row_token || !pos || !problems || n_pairs < 1 || top_k < 1 || max_problems < 1) return PE_ERR_ARG;
  if (rows_per_problem < 1 || rows_per_problem > 16) return PE_ERR_ARG;
  if (expert_map && n_global_experts < 1) return PE_ERR_ARG;
  if (n_local_experts < 1 || n_local_experts > kPlanMaxExperts) return PE_ERR_LIMIT;
  if (reinterpret_cast<uintptr_t>(problems) & 15) return PE_ERR_ALIGN;
  // every possible routing must fit: at most min(experts, pairs) partial problems plus pairs / rows full ones
  const int worst = (n_local_experts < n_pairs ? n_local_experts : n_pairs) + n_pairs / rows_per_problem;
  if (max_problems < worst) return PE_ERR_WORKSPACE;
  moe_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(topk_ids, expert_map, n_global_experts, n_pairs, top_k, n_local_experts,
                                                                             rows_per_problem, max_problems, row_token, pos,
                                                                             reinterpret_cast<int4*>(problems), expert_rows);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_moe_combine(const float* y, int64_t ld_y, const int32_t* pos, const float* topk_weights, int tokens, int top_k,
                              void* out, int out_dtype, int64_t ld_out, int hidden, void* stream) {
  if (!y || !pos || !topk_weights || !out || tokens < 1 || top_k < 1 || hidden < 4) return PE_ERR_ARG;
  if (out_dtype < PE_F32 || out_dtype > PE_BF16) return PE_ERR_ARG;
  if (hidden % 4 || ld_y % 4 || ld_y < hidden || ld_out < hidden) return PE_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(y) & 15) return PE_ERR_ALIGN;
  const int64_t n_vec = (int64_t)tokens * (hidden / 4);
  const int64_t blocks = (n_vec + 255) / 256;
  if (blocks > 0x7fffffff) return PE_ERR_LIMIT;
  moe_combine_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(y, ld_y, pos, topk_weights, top_k, out,
                                                                                    out_dtype, ld_out, hidden, n_vec);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}

extern "C" int pe_moe_route(const void* logits, int dtype, int64_t ld_logits, int n_tokens, int n_experts, int top_k, int renormalize,
                            float* weights, int64_t* ids, void* stream) {
  if (!logits || !weights || !ids || n_tokens < 1) return PE_ERR_ARG;
  if (dtype < PE_F32 || dtype > PE_BF16 || ld_logits < n_experts) return PE_ERR_ARG;
  if (n_experts < 1 || n_experts > 32 * kRouteMaxPerLane || top_k < 1 || top_k > 32 || top_k > n_experts) return PE_ERR_LIMIT;
  moe_route_kernel<<<(unsigned)((n_tokens + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, dtype, ld_logits, n_tokens,
                                                                                                 n_experts, top_k, renormalize, weights, ids);
  PE_CUDA_TRY(cudaGetLastError());
  return PE_OK;
}
