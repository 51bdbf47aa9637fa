/*
 * polar_b200.h -- C ABI of the B200 (sm_100a) PolarEngine quantized-linear kernels.
 *
 * Plain pointers and sizes only; no torch types.  Every function launches on the
 * stream it is given and returns immediately (asynchronous with respect to the
 * host), returning 0 on success or a negative PE_ERR_* code.  The caller owns all
 * buffers, including outputs and scratch; nothing here allocates device memory
 * unless its comment says so.  One caller thread per device.
 *
 * Reference interfaces these replace (paths inside caiovicentino/polarengine-vllm):
 *   polarengine_vllm/kernels/polar_gemm.py:425-437   polar_matmul (dispatcher)
 *   polarengine_vllm/kernels/polar_gemv.py:181-256   polar_gemv / polar_gemv_packed
 *   polarengine_vllm/kernels/polar_gemv_splitk.py:421-569  split-K variants
 *   polarengine_vllm/kernels/polar_gemm.py:312-418   polar_gemm / polar_gemm_packed
 *   polarengine_vllm/kernels/fwht.py:77-108          fwht_matmul
 *   polarengine_vllm/kernels/polar_gemv.py:263-283   pack_codes_int4
 *   polarengine_vllm/kernels/cuda/polar_gemv_cuda.cu:261-349, fwht_cuda.cu:93-141
 *                                                    (the optional pybind extension)
 */
#ifndef POLAR_B200_H
#define POLAR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / outputs */
enum { PE_F32 = 0, PE_F16 = 1, PE_BF16 = 2 };

/* what the activation pointer of pe_gemv / pe_gemm holds */
enum {
  PE_X_ROTATED = 0, /* already FWHT-128 rotated and zero padded to in_f_padded
                       (the reference's `x_transformed`, fwht.py:102-108)        */
  PE_X_RAW = 1      /* un-rotated activations with in_f valid columns; the kernel
                       pads and rotates while staging (linear_method.py:186-197) */
};

/* glue ops that pe_gemv_pro computes while it stages its input */
enum {
  PE_PRO_NONE = 0,
  PE_PRO_ADD_RMSNORM = 1, /* input = RMSNorm(x + delta) * norm_weight; the updated residual goes to resid_out */
  PE_PRO_SILU_MUL = 2     /* x = [gate | up] (2 * in_f fp16): input = silu(gate) * up                      */
};

/* error codes */
enum {
  PE_OK = 0,
  PE_ERR_ARG = -1,       /* null pointer, bad enum, non-positive size            */
  PE_ERR_SHAPE = -2,     /* in_f_padded not a multiple of 128, batch too large   */
  PE_ERR_ALIGN = -3,     /* pointer / leading dimension not 16-byte aligned      */
  PE_ERR_WORKSPACE = -4, /* scratch buffer too small                             */
  PE_ERR_CUDA = -5,      /* a CUDA runtime call failed; see pe_last_cuda_error() */
  PE_ERR_DEVICE = -6,    /* device is not sm_100                                  */
  PE_ERR_LIMIT = -7      /* size beyond a compiled-in maximum                    */
};

/* values a kernel leaves in a status word when a bounded device-side wait ran out */
enum {
  PE_STATUS_SPLITK_TIMEOUT = 1 /* pe_gemv tile kernel: a split-K partial never arrived */
};

int pe_version(void);
const char* pe_error_string(int code);
/* cudaError_t of the last failing runtime call made by this library on this thread */
int pe_last_cuda_error(void);

/* Kernels that wait on another party (a peer rank's flag in pe_allreduce_add_rmsnorm) give up after a limit, record a status value and return, so that a
 * missing peer costs a bounded time and never a hung GPU.  The default is about one second; this
 * sets it for launches made afterwards (process-wide).  No counterpart in the reference. */
int pe_set_wait_limit_us(int64_t microseconds);

/* One-time per-device set-up (opt-in shared-memory sizes, SM count).  Safe to call
 * repeatedly.  Makes `device` current.  No counterpart in the reference. */
int pe_init(int device);

/* ---- rotation ---------------------------------------------------------------
 * x (batch, in_f) -> x_tf (batch, in_f_padded): zero pad to a multiple of 128 and
 * rotate every 128-block by the normalised Hadamard matrix.
 * Replaces fwht_matmul + F.pad (fwht.py:77-108, linear_method.py:194-196) and
 * polarengine_cuda.fwht (fwht_cuda.cu:93-119).  ld_* are row strides in elements. */
int pe_fwht128(const void* x, int x_dtype, int64_t ld_x, void* x_tf, int out_dtype, int64_t ld_out,
               int batch, int in_f, int in_f_padded, void* stream);

/* ---- quantized embedding lookup ----------------------------------------------
 * out[t, :] = dequantised row ids[t] of a quantized (vocab, hidden) table:
 * FWHT-128(ct_scaled[codes[row, blk, :]]) * norm[row, blk] per block (the rotation is
 * its own inverse), i.e. row ids[t] of weight_converter._dequant_weight
 * (weight_converter.py:34-67) without materialising the table.  The reference keeps
 * embeddings unquantized at run time (config.py:188-193); its quantizer assigns them
 * 5 bits (utils.py:112-114).  ids are int64 on the device; out-of-range ids give zeros. */
int pe_embedding(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                 const float* ct_scaled, int n_levels, const int64_t* ids, int64_t vocab, void* out, int out_dtype,
                 int64_t ld_out, int tokens, int hidden, int hidden_padded, void* stream);

/* ---- decoder-layer glue ops (no reference counterpart) -----------------------
 * The reference leaves these to the serving framework (vLLM's fused RMSNorm, rotary and
 * activation ops); they are here so that an end-to-end decode step can be timed without
 * dozens of small framework kernels between the quantized projections.  fp16 tensors.
 *
 * pe_add_rmsnorm: x (rows, hidden) is the residual stream, updated in place with
 *   x += fp16(delta) when delta (fp16 or fp32, same shape, may be NULL) is given;
 *   out = fp16(x * rsqrt(mean(x^2) + eps)) * weight.  hidden % 8 == 0, hidden <= 16384.
 * pe_rope_cache: qkv (batch*t, (hq + 2 hkv) * head_dim), row stride ld_qkv.  Token i of a
 *   sequence sits at position base + i, base = *pos_dev if pos_dev is not NULL (a device
 *   scalar, for graph replay) else pos_host.  Rotate-half rotary embedding of the query and
 *   key heads (frequencies theta^(-2j/d)); queries go to q_out (batch, hq, t, head_dim),
 *   rotated keys and the values into the caches (batch, hkv, max_len, head_dim) at their
 *   positions (positions outside [0, max_len) are dropped).
 * pe_silu_mul: out[r, i] = fp16(silu(gate_up[r, i])) * gate_up[r, inter + i].
 * pe_decode_attention: one new token per sequence.  q (batch, hq, head_dim), caches as
 *   above holding positions 0 .. pos (pos = *pos_dev or pos_host, the token just written);
 *   out (batch, hq * head_dim) = softmax(q K^T / sqrt(head_dim)) V per query head, query head
 *   i reading kv head i / (hq / hkv).  head_dim = 128, hq / hkv in {1, 2, 4, 8}.  With a
 *   workspace (pe_decode_attention_workspace_bytes; its first 4 KB zero before the first call,
 *   left zero) the cache positions are split over up to 16 CTAs per kv head; NULL = one CTA.
 * pe_rope_attention: pe_rope_cache (t = 1) and pe_decode_attention as ONE launch: qkv (batch,
 *   (hq + 2 hkv) * head_dim) holds the raw fused projection of the new token; queries and the new
 *   key are rotated in registers, key and value are written into the caches at the position, and
 *   the attention uses them without reading them back.  Same output as the two calls. */
int pe_add_rmsnorm(void* x, const void* delta, int delta_dtype, const void* weight, void* out, int rows, int hidden,
                   float eps, void* stream);
int pe_rope_cache(const void* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, void* q_out, void* k_cache,
                  void* v_cache, int batch, int t, int hq, int hkv, int head_dim, int max_len, float theta, void* stream);
int pe_silu_mul(const void* gate_up, int64_t ld_gu, void* out, int64_t ld_out, int rows, int inter, void* stream);
size_t pe_decode_attention_workspace_bytes(int batch, int hq, int hkv, int head_dim);
int pe_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos_dev, int64_t pos_host,
                        void* out, int batch, int hq, int hkv, int head_dim, int max_len, void* workspace,
                        size_t workspace_bytes, void* stream);
int pe_rope_attention(const void* qkv, int64_t ld_qkv, const int64_t* pos_dev, int64_t pos_host, void* k_cache, void* v_cache,
                      void* out, int batch, int hq, int hkv, int head_dim, int max_len, float theta, void* workspace,
                      size_t workspace_bytes, void* stream);

/* ---- quantizer --------------------------------------------------------------
 * weight (out_f, in_f) fp32/fp16/bf16 -> codes int8 (out_f, in_f_padded), norms fp16 (out_f, in_f_padded/128):
 * per 128-block zero-pad, L2 norm (clamped at 1e-10), divide, rotate, scale by sqrt(128), index of the nearest of
 * `levels` (the UNscaled Lloyd-Max centroids; first minimum wins).  The arithmetic of
 * PolarQuantizer.quantize_tensor (quantizer.py:206-257) on the device; rotation and norm are summed in another
 * order than the reference's matrix product, so codes on a cell boundary may differ (a few per million).
 * Follow with pe_pack_nibble for widths <= 4 bits. */
int pe_quantize(const void* weight, int w_dtype, int64_t ld_w, int64_t out_f, int in_f, int in_f_padded,
                const float* levels, int n_levels, int8_t* codes, int64_t ld_codes, void* norms, int64_t ld_norms,
                void* stream);

/* ---- nibble packing ---------------------------------------------------------
 * int8 codes (out_f, in_f_padded) -> uint8 (out_f, in_f_padded/2), byte i of each
 * 128-block = code[64+i] << 4 | code[i].  Replaces pack_codes_int4
 * (polar_gemv.py:263-283) == pack_codes_half_block (packing.py:22-60). */
int pe_pack_nibble(const int8_t* codes, uint8_t* packed, int64_t out_f, int64_t in_f_padded, void* stream);

/* ---- decode-size matmul (batch <= 16) ----------------------------------------
 * y[m, r] = sum_blk norm[r, blk] * sum_k ct_scaled[code[r, blk, k]] * FWHT(x)[m, blk, k]
 * (+ bias[r]), fp32 accumulation, one launch, bit-reproducible from run to run.
 *
 *   codes   packed != 0: uint8 (out_f, in_f_padded/2) half-block nibbles
 *           packed == 0: int8/uint8 (out_f, in_f_padded), one code per byte
 *   ld_codes  row stride of codes in bytes (multiple of 16)
 *   norms   fp16 (out_f, n_blocks), ld_norms row stride in elements
 *   ct_scaled fp32 (n_levels), n_levels in 2..256 (<= 16 when packed)
 *   x       (batch, *) row-major with row stride ld_x elements; x_kind says whether
 *           it is rotated already (in_f_padded columns) or raw (in_f columns)
 *   y       (batch, out_f) row stride ld_y elements, dtype y_dtype
 *   bias    optional fp16 (out_f), may be NULL
 *   workspace / workspace_bytes  scratch of at least pe_gemv_workspace_bytes(...);
 *           its first 256 KB hold per-tile counters that must read zero on entry
 *           (zero-fill the buffer once after allocating it); every call returns
 *           them to zero, so the buffer can be reused by later calls of any shape
 *           on the same stream without refilling.  Calls that share a scratch
 *           buffer must not overlap on the device.  The last int32 of those 256 KB
 *           is a status word: a kernel whose bounded device-side wait ran out stores
 *           a PE_STATUS_* value there (the output is then undefined);
 *           pe_gemv_status() waits for the stream and returns the word (0 = ok),
 *           clearing it when `clear` is non-zero.
 *
 * Replaces polar_matmul's batch==1 branches and (for 2..16 rows) its GEMM branch
 * (polar_gemm.py:485-534), plus the cast/bias epilogue of linear_method.py:214-221. */
size_t pe_gemv_workspace_bytes(int batch, int out_f, int in_f_padded);
int pe_gemv_status(void* workspace, size_t workspace_bytes, int clear, void* stream);

/* 1 if pe_gemv runs batches of 3..8 rows of this layer on its row-major arrays with the column-owner
 * tensor-core kernel (weights decoded once per step and used for every row of the batch; no scratch
 * memory, no tiled copy of the layer needed), 0 if such batches go to the tile kernel, which streams the
 * tiled copy (pe_retile / pe_gemv_tiled) best.  No launch, no device access beyond the SM count. */
int pe_gemv_small_batch_takes(int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, int out_f,
                              int in_f_padded);
int pe_gemv(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
            const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
            int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
            int in_f_padded, void* workspace, size_t workspace_bytes, void* stream);

/* ---- grouped decode-size matmul: the experts of a mixture layer -----------------
 * One launch over a stack of matrices of one shape (expert e at codes + e * codes_stride
 * bytes, norms + e * norms_stride halves), each against its own 1..16 activation rows.
 * `problems` is a DEVICE array of max_problems int32 quadruples (expert, first, rows, 0):
 * problem i multiplies rows first .. first + rows - 1 of the row list -- row x_rows[j] of
 * x when x_rows is not NULL (a gather by token id), else row j of x -- with expert
 * `expert` and writes rows first .. of y.  Entries with rows <= 0 are skipped, so the host
 * sizes the launch for the worst case and never reads the routing back.  max_rows (<= 16)
 * bounds the rows of any problem (8 or less selects the lighter kernel); an expert with
 * more rows takes several problems.  No bias.  The scratch
 * (pe_gemv_grouped_workspace_bytes; 0 = too many problems) is its own buffer, not the one
 * of pe_gemv: its first 4 MiB must be zero before the first use and are left zero, so
 * calls of any shapes can share it in stream order.
 * Replaces the per-expert loop of the reference's MoE layer (nemotron_offload.py:190-226:
 * for each selected expert, gate/up projection, activation, down projection) with two
 * grouped launches; the reference's vLLM path has no quantized expert arithmetic
 * (moe_method.py:18-98). */
size_t pe_gemv_grouped_workspace_bytes(int max_problems, int out_f, int in_f_padded);
int pe_gemv_grouped(const void* codes, int packed, int64_t ld_codes, int64_t codes_stride, const void* norms,
                    int64_t ld_norms, int64_t norms_stride, const float* ct_scaled, int n_levels, const void* x,
                    int x_kind, int x_dtype, int64_t ld_x, int in_f, const int32_t* x_rows, void* y, int y_dtype,
                    int64_t ld_y, const int32_t* problems, int max_problems, int max_rows, int out_f,
                    int in_f_padded, void* workspace, size_t workspace_bytes, void* stream);

/* ---- grouped prefill-size matmul: the experts of a mixture layer on the tensor cores -----
 * pe_gemm over a stack of matrices (expert e's codes directly after expert e-1's:
 * codes_stride == out_f * ld_codes; norms + e * norms_stride halves).  expert_rows is a
 * DEVICE array of n_experts (first row, row count) pairs, ascending and contiguous (from
 * pe_moe_plan): rows first .. first + count - 1 of the row list -- row x_rows[j] of x when
 * x_rows is not NULL, else row j -- are multiplied with expert e and written to the same
 * rows of y.  `rows` = length of the row list (pairs); rows past the last expert's range
 * are ignored.  The tile list is built on the device, nothing is read back.  Replaces the
 * per-expert loop of nemotron_offload.py:190-226 for batches where every expert has many
 * rows; the reference's vLLM path runs vLLM's bf16 fused MoE here (moe_method.py:82-89). */
size_t pe_gemm_grouped_workspace_bytes(int n_experts, int rows, int out_f, int in_f_padded);
int pe_gemm_grouped(const void* codes, int packed, int64_t ld_codes, int64_t codes_stride, const void* norms,
                    int64_t ld_norms, int64_t norms_stride, const float* ct_scaled, int n_levels, const void* x,
                    int x_kind, int x_dtype, int64_t ld_x, int in_f, const int32_t* x_rows, void* y, int y_dtype,
                    int64_t ld_y, const int32_t* expert_rows, int n_experts, int rows, int out_f, int in_f_padded,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Routing of a mixture layer as one launch (nemotron_offload.py:180-189): fp32 softmax of the router logits over
 * the experts, the top_k largest in descending order (ties to the lower expert id), kept weights divided by
 * their sum when `renormalize`.  logits (n_tokens, n_experts) fp32 / fp16 / bf16 with row stride ld_logits;
 * weights (n_tokens, top_k) fp32 and ids (n_tokens, top_k) int64 out.  n_experts <= 1024, top_k <= 32. */
int pe_moe_route(const void* logits, int dtype, int64_t ld_logits, int n_tokens, int n_experts, int top_k, int renormalize,
                 float* weights, int64_t* ids, void* stream);

/* ---- mixture-of-experts bookkeeping on the device ----------------------------------
 * pe_moe_plan groups the (token, slot) pairs of a routing decision by local expert:
 *   topk_ids (n_pairs = tokens * top_k, int64, token-major); expert_map (optional, int64,
 *   global expert -> local index or -1, the expert-parallel placement, n_global_experts
 *   entries: ids outside [0, n_global_experts) are treated as -1);
 *   row_token[r] = token of grouped row r (the x_rows list of pe_gemv_grouped),
 *   pos[pair] = grouped row of the pair or -1 if its expert lives on another rank,
 *   problems = the problem list of pe_gemv_grouped with at most rows_per_problem rows each
 *   (max_problems >= min(experts, pairs) + pairs / rows_per_problem entries),
 *   expert_rows (optional) = (first grouped row, row count) per local expert, the input of
 *   pe_gemm_grouped.
 * pe_moe_combine: out[t, :] = sum_j topk_weights[t, j] * y[pos[t * top_k + j], :] (pairs
 *   with pos < 0 contribute nothing), y fp32 (rows, hidden), out fp32/fp16/bf16.
 * Together with pe_gemv_grouped they replace the per-expert Python loop of the reference's
 * MoE layer (nemotron_offload.py:190-226: index tokens, run the expert, index_add). */
int pe_moe_plan(const int64_t* topk_ids, const int64_t* expert_map, int n_global_experts, int n_pairs, int top_k, int n_local_experts,
                int rows_per_problem, int max_problems, int32_t* row_token, int32_t* pos, int32_t* problems,
                int32_t* expert_rows, void* stream);
int pe_moe_combine(const float* y, int64_t ld_y, const int32_t* pos, const float* topk_weights, int tokens, int top_k,
                   void* out, int out_dtype, int64_t ld_out, int hidden, void* stream);

/* ---- row-parallel epilogue across tensor-parallel ranks -----------------------------
 * One kernel per rank: all-reduce of the fp32 partial outputs of a row-parallel projection
 * (o_proj / down_proj shards, loader.py:558-638 slices them) over peer memory, then
 * x += fp16(sum), out = fp16(x * rsqrt(mean(x^2) + eps)) * weight (pe_add_rmsnorm).  It
 * stands where a vLLM deployment issues an NCCL all-reduce plus its add and norm kernels.
 *   peer_buffers: DEVICE array of `world` addresses, entry r = rank r's exchange buffer
 *     (pe_allreduce_buffer_bytes, zero before the first call) as mapped in THIS process
 *     (peer memory: CUDA IPC or symmetric-memory mappings; entry `rank` is the local one);
 *   every rank launches the same call (rows, hidden) in the same order;
 *   seq: device array of max_rows counters, zero at start, owned by the kernel;
 *   status: device word set to 1 if a peer did not arrive within about a second (the
 *     launch then completes with incomplete sums instead of hanging).
 * rows <= max_rows, hidden % 8 == 0, hidden <= 16384 and the same for every call on one
 * buffer, world <= 16.  Plain peer loads / stores only (no multicast). */
size_t pe_allreduce_buffer_bytes(int world, int max_rows, int hidden);
int pe_allreduce_add_rmsnorm(const float* partial, void* x, const void* weight, void* out, int rows, int hidden, float eps,
                             const uint64_t* peer_buffers, int rank, int world, int max_rows, unsigned* seq, int* status,
                             void* stream);

/* ---- tiled weight layout for the decode kernel -----------------------------------
 * pe_retile rewrites a layer (codes + norms, the reference's row-major layouts) into the
 * layout the decode kernel streams best: for every 16-row tile and every 128-block, the
 * 16 x 64 B (nibble) or 16 x 128 B (byte) codes followed by the 16 fp16 block norms, tiles
 * of a row tile stored one after the other.  A warp then reads one contiguous region
 * with 512-byte requests instead of sixteen 64-byte row pieces, and the norms travel with
 * the codes.  pe_retile_bytes gives the size of the tiled buffer (rows padded to 16).
 * Done once after loading, next to pack_codes_int4 (linear_method.py:228-258); it has no
 * counterpart in the reference.  pe_gemv_tiled = pe_gemv on such a buffer. */
size_t pe_retile_bytes(int packed, int64_t out_f, int64_t in_f_padded);
int pe_retile(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms, void* tiles,
              int64_t out_f, int64_t in_f_padded, void* stream);
int pe_gemv_tiled(const void* tiles, int packed, const float* ct_scaled, int n_levels, const void* x, int x_kind,
                  int x_dtype, int64_t ld_x, int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch,
                  int out_f, int in_f_padded, void* workspace, size_t workspace_bytes, void* stream);

/* ---- prefill-size matmul (any number of rows; meant for m > 16) -------------------
 * Same result as pe_gemv with the arguments in the same order; the contraction runs on
 * tcgen05 tensor cores in bf16 with fp32 accumulation (activations and dequantised
 * weights are rounded to bf16).  Two launches: activation preparation (pad, rotate when
 * x_kind is PE_X_RAW, bf16) into the workspace, then the matmul.
 *   workspace  at least pe_gemm_workspace_bytes(m, in_f_padded), 256-byte aligned.  Its
 *              first int32 is a status word written by the kernel: 0 on success, 1..10
 *              if a bounded device-side wait ran out (the output is then undefined).
 * More than 256 rows run on pairs of CTAs (thread-block clusters of two, one tensor-core
 * operation per pair); the launch needs no more than the usual one-CTA-per-SM residency.
 * Replaces polar_matmul's batched branch: polar_gemm / polar_gemm_packed
 * (polar_gemm.py:312-418, 526-534) and the epilogue of linear_method.py:214-221. */
size_t pe_gemm_workspace_bytes(int m, int in_f_padded);
/* Launches of up to 256 rows on layers that give few 256-row tiles split K over the SMs when the workspace also
 * holds their fp32 partials: this size (>= pe_gemm_workspace_bytes) makes room for them.  With less, pe_gemm runs
 * unsplit.  Same result either way up to the order of the fp32 sums (fixed for a given shape and GPU). */
size_t pe_gemm_workspace_bytes_splitk(int m, int out_f, int in_f_padded);
int pe_gemm(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
            const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
            int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int m, int out_f,
            int in_f_padded, void* workspace, size_t workspace_bytes, void* stream);

/* ---- one-token matmul with the preceding glue op folded in ---------------------------
 * y (1, out_f) = pe_gemv of one fp16 activation row that is computed on the fly:
 *   PE_PRO_ADD_RMSNORM  r = half(x + half(delta)) over in_f elements (delta fp16 / fp32, may be NULL);
 *                       input = half(r * rsqrt(mean(r^2) + eps)) * norm_weight (the rounding steps of
 *                       pe_add_rmsnorm); r is also stored to resid_out (fp16, may be NULL, must not be x)
 *   PE_PRO_SILU_MUL     x = [gate | up], 2 * in_f fp16; input = half(silu(gate)) * up (pe_silu_mul)
 * so that the residual-add + norm in front of q/k/v and gate/up, and the activation in front of down,
 * cost no launch of their own at decode time.  in_f a multiple of 4 (8 for PE_PRO_SILU_MUL), all
 * pointers 16-byte aligned.  Layers the batch-1 kernel does not take (few rows, rows that are not a
 * multiple of 128 bytes, more than 64 chunks) return PE_ERR_SHAPE: run the glue op and pe_gemv then.
 * The reference leaves these ops to the serving framework (linear_method.py:157-222 receives the
 * already normalised activations); no counterpart there. */
int pe_gemv_pro(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                const float* ct_scaled, int n_levels, int prologue, const void* x, int in_f, const void* delta,
                int delta_dtype, const void* norm_weight, void* resid_out, float eps, void* y, int y_dtype,
                const void* bias, int out_f, int in_f_padded, void* stream);

/* ---- decode-size matmul without caller scratch ----------------------------------
 * Same computation and arguments as pe_gemv, minus workspace / workspace_bytes.  It has
 * no counterpart in the reference.  It is meant for integrations that are not in a
 * position to allocate device memory when a layer runs: servers that give all free HBM
 * to their own cache at start-up, after which an extra cudaMalloc may fail, and glue
 * code that sits below the framework's allocator and cannot call it.  The scratch is an
 * 8 MiB array inside the library image (pe_gemv_noalloc_max_bytes()); every GPU that
 * loads the library holds those 8 MiB until the process exits.
 *
 *  - Shapes whose pe_gemv_workspace_bytes() exceeds the array return PE_ERR_LIMIT
 *    (all 9B-class decoder projections at batch <= 16 fit; a 151,936-row head fits up
 *    to batch 6).
 *  - The call allocates nothing and frees nothing.  The first call on each device looks
 *    up the array's device address (cudaGetSymbolAddress) with that device current;
 *    make that first call outside of any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents; the entry point clears the counters it needs, in stream order, before
 *    the kernel.  Two calls that overlap on the GPU (different streams) race on it:
 *    keep them on one stream or order them with events.
 *  - A bounded device-side wait that runs out leaves a PE_STATUS_* value in a word of the
 *    array; pe_gemv_noalloc_status() waits for the stream and returns that word (0 = every
 *    wait completed), clearing it when `clear` is non-zero.  It allocates nothing either. */
size_t pe_gemv_noalloc_max_bytes(void);
int pe_gemv_noalloc_status(int clear, void* stream);
int pe_gemv_noalloc(const void* codes, int packed, int64_t ld_codes, const void* norms, int64_t ld_norms,
                    const float* ct_scaled, int n_levels, const void* x, int x_kind, int x_dtype, int64_t ld_x,
                    int in_f, void* y, int y_dtype, int64_t ld_y, const void* bias, int batch, int out_f,
                    int in_f_padded, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* POLAR_B200_H */
