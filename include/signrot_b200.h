/* signrot_b200 -- C ABI of the B200 (sm_100a) implementation of SignRot's online
 * quantized-linear path.
 *
 * One shared library, libsignrot_b200.so, exports the functions below.  They are what
 * a binding for this path has to call: each comment names the reference interface
 * (file:line inside HYU-ARK-Lab/SignRot) that the entry point replaces.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer into memory owned by the caller; inputs are
 *    borrowed, outputs are written in place; tensors are dense and row-major;
 *  - nothing is allocated, nothing is synchronised and no device memory is read on
 *    the host, so every call may be captured in a CUDA graph;
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *  - activations are IEEE fp16 unless a dtype tag says otherwise; 4-bit codes are
 *    packed two per byte, element 2j in the low nibble of byte j
 *    (signrot/functional/quantization.py:45-53, signrot/kernels/include/int4.h:79-99);
 *  - the return value is SR_OK or an SR_ERR_* code; sr_last_error() then returns a
 *    message for the calling thread.  Argument errors are detected on the host
 *    before anything is launched.
 */
#ifndef SIGNROT_B200_H_
#define SIGNROT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SR_VERSION 100

#define SR_OK 0
#define SR_ERR_INVALID 1      /* bad argument (the reference raises RuntimeError via TORCH_CHECK) */
#define SR_ERR_CUDA 2         /* the CUDA runtime or driver reported an error */
#define SR_ERR_UNSUPPORTED 3  /* valid request that this build has no kernel for */

/* dtype tags */
#define SR_F16 0
#define SR_BF16 1
#define SR_F32 2

/* Read-only operands and early loads.  Kernels of the decode step are launched with programmatic
 * stream serialization: they may start while the kernel before them on the stream is finishing, and
 * they fetch their constant operands -- weights (B / W), weight scales and sums, the hadK table and
 * the sign tables -- BEFORE they wait for that kernel.  Those buffers must therefore not be written
 * by work enqueued earlier on the same stream without a synchronisation in between (a weight that
 * was just packed, a table that was just cast).  Activations, codes, scales of activations, caches
 * and workspaces carry no such restriction.  SIGNROT_B200_PDL=0 removes the early start. */

const char *sr_last_error(void);
int sr_version(void);

/* Device-side status word: 0, or the code of the first bounded wait that expired
 * inside a kernel (such a kernel stops early, its output is undefined).  This call
 * synchronises with the device; it is meant for tests and health checks. */
int sr_device_status(int *status, int clear);

/* Health check of the bounded-wait machinery: one thread of a one-CTA kernel waits `budget_cycles`
 * (1e3 .. 1e7 SM cycles) on a barrier nobody arrives on, gives up, records code 99 in the status word
 * that sr_device_status reads, and the kernel returns normally.  The status word is per device and
 * sticky: while it is non-zero the tensor-core GEMM skips its work, so a caller that sees it must read
 * and clear it (sr_device_status(&s, 1)) before trusting later outputs.  No counterpart in the
 * reference, whose kernels have no device-side waits. */
int sr_selftest_bounded_wait(int64_t budget_cycles, void *stream);

/* ------------------------------------------------------------------ int4 GEMM */

/* C[M,N] int32 = A[M,K] * B[N,K]^T, A packed s4 (a_unsigned = 0) or u4 (1), B packed s4.
 * K % 32 == 0.  Replaces signrot._CUDA.matmul / matmul_ui4_si4
 * (signrot/kernels/bindings.cpp:13-47, gemm.cu:7-85; Python: functional/kernel.py:67-81). */
int sr_matmul_i4(const void *A, const void *B, int64_t M, int64_t N, int64_t K, int a_unsigned, void *C,
                 void *stream);

/* The same product with A taken from a wider code matrix: row m of A starts lda_bytes after row m - 1
 * (lda_bytes >= K / 2, a multiple of 16; A itself 16-byte aligned).  A tensor-parallel rank multiplies its K-slice
 * of the full-row codes this way without copying it out (the reference has no sharded form of this path). */
int sr_matmul_i4_ld(const void *A, int64_t lda_bytes, const void *B, int64_t M, int64_t N, int64_t K, int a_unsigned,
                    void *C, void *stream);

/* out[M,N] fp16 = dequant(A * W^T): the whole of Linear4bit.forward for a packed input
 * (signrot/nn/linear.py:36-50): GEMM, optional asymmetric correction
 * acc -= a_zero[m] * w_sum[n] (a_zero int8 [M], w_sum int32 [N]; both NULL for symmetric
 * activations, in which case A holds signed codes, otherwise unsigned codes), dequant
 * rn_h((float(acc) * a_scale[m]) * w_scale[n]) (signrot/kernels/quant.cu:84-87) and optional
 * fp16 bias add.  The int32 matrix never reaches memory. */
int sr_w4a4_linear(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                   const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *stream);

/* sr_w4a4_linear with a scratch buffer for the long-K shapes whose 256 x 256 output tiles would leave at least half
 * of the GPU idle (e.g. M = 256, K = 14336, N = 4096: 16 tiles for 74 CTA pairs): the K dimension of every tile is
 * split over 2 or 4 CTA pairs, the int32 partial sums meet in `ws` and are added there, so the result is the bit
 * pattern of sr_w4a4_linear.  sr_w4a4_linear_ws_bytes gives the size `ws` needs (0: this shape does not split; then
 * ws may be NULL and the call is sr_w4a4_linear).  `counters`: 1024 int32 in device memory, zero before the first
 * call and never written by anybody else (they only grow, by the number of k-ranges per launch); one buffer serves
 * all calls of a stream, calls that may run at the same time need their own.  ws 16-byte aligned. */
int sr_w4a4_linear_ws_bytes(int64_t M, int64_t N, int64_t K, int64_t *bytes);
int sr_w4a4_linear_ws(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                      const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *ws,
                      int64_t ws_bytes, void *counters, void *stream);

/* Fused edge of the path for decode: gate_proj and up_proj of a SwiGLU MLP and the activation in
 * one launch.  W = [2N, K/2]: the N gate rows followed by the N up rows (w_scale [2N], w_sum [2N]
 * and bias [2N] likewise); out[M, N] fp16 = rn_h(rn_h(silu(gate)) * up) with gate/up the fp16
 * results sr_w4a4_linear would give (signrot/nn/linear.py:36-50) and the SwiGLU arithmetic of
 * _CUDA.swiglu (signrot/kernels/fused.cu:367-381): the same bits as the three separate calls
 * (fake_quant/kernel_utils.py:352-363).  At most 32 rows (SR_ERR_UNSUPPORTED beyond: larger
 * batches run the two projections and sr_swiglu). */
int sr_w4a4_swiglu(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                   const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *stream);

/* P problems C_p = A_p * B_p^T in one launch.  problem_sizes int32 [P,3] rows (m, n, k);
 * ptr_* int64 [P] device addresses; ld* int64 [P] leading dimensions in elements.  All of
 * these arrays live in device memory and are never read on the host.  max_k > 0 promises
 * k_p <= max_k for every problem (lets more CTAs share an SM); 0 = unknown.  A problem with
 * k % 32 != 0 or k beyond the promise is skipped and recorded in the device status word.
 * Two kernels stand behind the call and the choice is made on the device, from the arrays: the layout
 * the reference's MoE block builds (signrot/nn/moe.py:96-111: rows sorted by problem in one activation
 * matrix, stacked weights, one output matrix; equal n, k and leading dimensions; at most 512 problems)
 * with more than 16 rows per problem on average runs on the tensor cores (tcgen05, tensor maps written
 * on the device); any other set of problems, and decode-sized calls, on a CUDA-core kernel.  The
 * integers are the same either way.  Calls from more than 16 streams at once, or two graphs captured on
 * one stream and replayed at the same time, would share the small device-side plan: do not do that.
 * Replaces signrot._CUDA.matmul_grouped (bindings.cpp:49-91, gemm_grouped.cu:19-120). */
int sr_matmul_grouped(const void *problem_sizes, int64_t problem_count, const void *ptr_a, const void *ptr_b,
                      const void *ptr_c, const void *lda, const void *ldb, const void *ldc, int signed_a,
                      int64_t max_k, void *stream);

/* Sparse-MoE expert linear in one launch: rows of A are sorted by expert, expert e owns rows
 * row_offsets[e] .. row_offsets[e+1]-1 (int32 [num_experts + 1], device memory, never read on the
 * host) and multiplies its own weight W[e] (W packed s4 [num_experts, N, K/2]).  Fuses what the
 * reference runs as matmul_grouped followed by sym_dequant_moe (signrot/nn/moe.py:114-162,
 * signrot/kernels/moe.cu:190-233): out[r, n] = rn_h((float(acc) * a_scale[r]) * w_scale[e, n]) with
 * e = expert_ids[r] (int32 [rows]); asymmetric activations pass a_zero int8 [rows] and w_sum int32
 * [num_experts, N].  At most 512 experts.  Few rows per expert (16 or fewer on average) run on the
 * weight-streaming kernel, more on the tcgen05 CTA-pair kernel.  `rows` is the size of A and out;
 * `expected_rows` (0 = rows) is how many of them the offsets are expected to cover, for a caller whose
 * offsets describe a part of A only (an expert-parallel rank passes its own experts' slice of the
 * offsets and rows * local experts / all experts): only the choice of kernel depends on it. */
int sr_grouped_linear(const void *A, const void *a_scale, const void *a_zero, const void *expert_ids,
                      const void *row_offsets, const void *W, const void *w_scale, const void *w_sum, int64_t rows,
                      int64_t num_experts, int64_t N, int64_t K, int64_t expected_rows, void *out, void *stream);

/* ------------------------------------------------------------------ quantizers */

/* Per-row amax -> scale = rn_h(amax/7) (* clip) -> codes clamp(rint(x/scale), -8, 7).
 * q: uint8 [rows, ceil(cols/2)], scale: fp16 [rows].
 * Replaces _CUDA.sym_quant_dynamic (bindings.cpp:316-335, fused.cu:68-138). */
int sr_sym_quant_dynamic(const void *x, int64_t rows, int64_t cols, float clip_ratio, void *q, void *scale,
                         void *stream);

/* Per-row min/max -> scale, zero (fp16 [rows] each) -> unsigned codes 0..15.
 * Replaces _CUDA.asym_quant_dynamic (bindings.cpp:337-360, fused.cu:143-208). */
int sr_asym_quant_dynamic(const void *x, int64_t rows, int64_t cols, float clip_ratio, void *q, void *scale,
                          void *zero, void *stream);

/* The two quantizers above with row r first multiplied by sign[expert_ids[r]] (sign: int8
 * [E, cols] of +-1 or NULL; expert_ids: int32 [rows]).
 * Replaces _CUDA.sym/asym_quant_dynamic_moe (bindings.cpp:111-168, moe.cu:60-199). */
int sr_sym_quant_dynamic_moe(const void *x, const void *sign, const void *expert_ids, int64_t rows, int64_t cols,
                             float clip_ratio, void *q, void *scale, void *stream);
int sr_asym_quant_dynamic_moe(const void *x, const void *sign, const void *expert_ids, int64_t rows, int64_t cols,
                              float clip_ratio, void *q, void *scale, void *zero, void *stream);

/* Quantize with given per-row scale (and zero).  Replaces _CUDA.sym_quant,
 * asym_quant_f16_si4, asym_quant_f16_ui4 (bindings.cpp:215-314, quant.cu:13-231). */
int sr_sym_quant(const void *x, const void *scale, int64_t rows, int64_t cols, void *q, void *stream);
int sr_asym_quant_f16_si4(const void *x, const void *scale, const void *zero, int64_t rows, int64_t cols, void *q,
                          void *stream);
int sr_asym_quant_f16_ui4(const void *x, const void *scale, const void *zero, int64_t rows, int64_t cols, void *q,
                          void *stream);

/* out fp16 [rows, cols] = rn_h((float(q) * scale_row[r]) * scale_col[c]), q int32.
 * Replaces _CUDA.sym_dequant (bindings.cpp:233-276, quant.cu:66-131). */
int sr_sym_dequant(const void *q, const void *scale_row, const void *scale_col, int64_t rows, int64_t cols,
                   void *out, void *stream);

/* Expert-indexed dequant with the asymmetric correction fused in; w_scales fp16 [E, cols],
 * w_sum int32 [E, cols], zero_row int8 [rows] (zero_row and w_sum both NULL or both set).
 * Replaces _CUDA.sym_dequant_moe (bindings.cpp:170-213, moe.cu:202-238). */
int sr_sym_dequant_moe(const void *q, const void *scale_row, const void *w_scales, const void *expert_ids,
                       const void *zero_row, const void *w_sum, int64_t rows, int64_t cols, void *out,
                       void *stream);

/* out int32 [rows] = sum of the 2*packed_cols 4-bit values of each row.
 * Replaces _CUDA.sum_i4 (bindings.cpp:436-449, quant.cu:233-350). */
int sr_sum_i4(const void *x, int64_t rows, int64_t packed_cols, int is_signed, void *out, void *stream);

/* out int32 [rows, cols] = a_col[r] (int8) * b_row[c] (int32).
 * Replaces _CUDA.matmul_colrow_i8_i32 (bindings.cpp:451-476, quant.cu:352-383). */
int sr_matmul_colrow_i8_i32(const void *a_col, const void *b_row, int64_t rows, int64_t cols, void *out,
                            void *stream);

/* ------------------------------------------------------------------ online rotation */

/* y = ((hadK (x) H_{n/K}) x) * scale over the last dimension, Sylvester order, flat index
 * k*(n/K)+j; then y *= sign (int8 [n] or NULL).  dtype/out_dtype are SR_F16, SR_BF16 or
 * SR_F32.  The Walsh-Hadamard sums are fp32 and rounded to `dtype`, the had-K stage (hadk:
 * K x K matrix in fp16, or fp32 when fp32_mode) rounds again, unless fp32_mode is set (then
 * only the final cast rounds).  Replaces fast_hadamard_transform.hadamard_transform + the
 * had-K matmul + the sign multiply: signrot/functional/hadamard.py:78-87,
 * signrot/nn/hadamard.py:26-42, signrot/transformers/kv_cache.py:70-73. */
int sr_hadamard(const void *x, int dtype, int64_t rows, int64_t n, const void *hadk, int64_t K, float scale,
                const void *sign, int fp32_mode, void *out, int out_dtype, void *stream);

/* Head-wise Hadamard (H_heads (x) I_head_dim) on rows of heads*head_dim values: the o_proj
 * input rotation, fake_quant/quant_utils.py:287-291 without the two transposes. */
int sr_hadamard_heads(const void *x, int dtype, int64_t rows, int64_t heads, int64_t head_dim, float scale,
                      int fp32_mode, void *out, int out_dtype, void *stream);

/* Rotation fused with the per-token quantizer: everything ActQuantWrapper.kernel_quantize
 * does (fake_quant/quant_utils.py:278-292) in one pass over the row.  x is fp16 or bf16
 * (bf16 is first rounded to fp16, quant_utils.py:284).  heads > 0 selects the head-wise
 * transform (then K must be 1); expert_ids (int32 [rows]) selects a row of sign [E, n].
 * asym = 0: signed codes + q_scale; asym = 1: unsigned codes + q_scale + q_zero (fp16).
 * `rotated` (fp16 [rows, n]) optionally receives the rotated row. */
int sr_rotate_quant(const void *x, int dtype, int64_t rows, int64_t n, const void *hadk, int64_t K, float scale,
                    const void *sign, const void *expert_ids, int64_t heads, float clip_ratio, int asym, void *q,
                    void *q_scale, void *q_zero, void *rotated, void *stream);

/* ------------------------------------------------------------------ MoE routing */

/* Routing of a sparse block in one launch (signrot/nn/moe.py:159-190: softmax in fp32, top-k,
 * optional renormalisation, cast, counting and the stable sort of the (token, choice) rows by
 * expert).  logits fp16 [tokens, num_experts].  Outputs: weights fp16 [tokens, top_k]; chosen int32
 * [tokens, top_k] (ties: the lower expert index); for the R = tokens * top_k routed rows in sorted
 * order: tok int32 [R] (source token), eid int32 [R] (expert); inv int32 [R] (sorted position of row
 * t * top_k + j); row_offsets int32 [num_experts + 1].  At most 512 experts and top-8. */
int sr_moe_route(const void *logits, int64_t tokens, int64_t num_experts, int64_t top_k, int renormalize,
                 void *weights, void *chosen, void *tok, void *eid, void *inv, void *row_offsets, void *stream);
/* One copy of a token's packed codes (row_bytes per row, a multiple of 16), scale (fp16) and optional
 * zero (int8) per routed row: q_out[r] = q[tok[r]] (moe.py:192-194). */
int sr_moe_gather(const void *q, const void *scale, const void *zero, const void *tok, int64_t rows, int64_t row_bytes,
                  void *q_out, void *scale_out, void *zero_out, void *stream);
/* out[t] = sum_j rn_h(y[inv[t * top_k + j]] * weights[t, j]) over fp16 rows of `hidden` values, fp32
 * sum, one fp16 rounding: the un-permute and weighted sum of moe.py:231-235.  row_range (int32 [2] on
 * the device, or NULL): only sorted rows lo <= r < hi are added (the rows of an expert-parallel rank's
 * own experts); out_f32 != 0 writes the fp32 sum unrounded (fp32 [tokens, hidden]) for a sum across
 * ranks, otherwise fp16. */
int sr_moe_combine(const void *y, const void *weights, const void *inv, const void *row_range, int64_t tokens,
                   int64_t top_k, int64_t hidden, int out_f32, void *out, void *stream);

/* ------------------------------------------------------------------ offline weight preparation */

/* Per-channel symmetric int4 round-to-nearest of a weight matrix W [N, K] (dtype SR_F16, SR_BF16 or
 * SR_F32), straight to packed codes [N, K/2] and fp16 scales [N].  Replaces, for one linear, the
 * chain rtn_fwrd (fake_quant/gptq_utils.py:411-465: WeightQuantizer.find_params + quantize, with the
 * SignRot sign unfolded before and refolded after on the symmetric grid [-7, 7]) ->
 * ActQuantWrapper.enable_kernel -> Linear4bit.from_float (signrot/nn/linear.py:52-73: round(W / scale),
 * pack_i4).  sign int8 [K] (+-1) or NULL; mse != 0 runs the clipping search of
 * quant_utils.py:488-512 (80 candidates, error norm 2.4; error sums in fp64, so a row whose two best
 * candidates tie within fp32 summation noise may pick the other one). */
int sr_rtn_pack(const void *W, int dtype, int64_t N, int64_t K, const void *sign, int mse, void *packed, void *scale,
                void *stream);

/* ------------------------------------------------------------------ adjacent fused ops */

/* Replaces _CUDA.rmsnorm (bindings.cpp:420-434, fused.cu:278-309). */
int sr_rmsnorm(const void *x, int64_t rows, int64_t cols, float eps, int64_t mean_dim, void *out, void *stream);

/* Fused edge of the path: residual add -> RMSNorm -> per-token int4 quantizer in one pass over the
 * row.  Replaces three launches of the decode graph: the fp16 `hidden + branch` add of the decoder
 * layer, _CUDA.rmsnorm (fused.cu:278-309) and _CUDA.sym_quant_dynamic / asym_quant_dynamic
 * (fused.cu:68-198), with the same rounding points (one fp16 rounding after the add, one after the
 * normalisation), so codes and scales equal those of the three separate calls bit for bit.
 * delta may be NULL (no add).  sum_out (fp16 [rows, cols], needs delta) receives x + delta;
 * normed_out (fp16, optional) the normalised row.  asym = 1 also writes zero (fp16 [rows]).
 * cols must be a multiple of 8 and at most 16384 (SR_ERR_UNSUPPORTED otherwise). */
int sr_add_rmsnorm_quant(const void *x, const void *delta, int64_t rows, int64_t cols, float eps, int64_t mean_dim,
                         float clip_ratio, int asym, void *sum_out, void *normed_out, void *q, void *scale,
                         void *zero, void *stream);
/* In-place rotary embedding on q [B,T,Hq,D], k [B,T,Hk,D]; cos/sin [cos_seqs,T,D].
 * Replaces _CUDA.rope_qk (bindings.cpp:383-409, fused.cu:316-362). */
int sr_rope_qk(void *q, void *k, const void *cosv, const void *sinv, int64_t n_seqs, int64_t seq_len,
               int64_t cos_seqs, int64_t n_q_heads, int64_t n_k_heads, int64_t head_dim, void *stream);
/* Replaces _CUDA.swiglu (bindings.cpp:411-418, fused.cu:367-390). */
int sr_swiglu(const void *gate, const void *up, int64_t numel, void *out, void *stream);
/* q uint8 [rows, cols/2], param fp16 [rows, 2] = (scale, zero).
 * Replaces _CUDA.kv_quant_pack (bindings.cpp:362-381, fused.cu:214-273). */
int sr_kv_quant_pack(const void *x, int64_t rows, int64_t cols, void *q, void *param, void *stream);

/* ------------------------------------------------------------------ int4 paged KV cache
 * kv_data uint8 [pages, layers, 2, heads, page_size, 64], kv_param fp16 [.., page_size, 2],
 * kv_indptr int32 [batch+1], kv_indices int32 [*], last_page_offset int32 [batch]
 * (signrot/transformers/kv_cache.py:185-196, 417-433).  head_dim must be 128. */

/* One already-quantized token per request into its slot.  Replaces _CUDA.append_kv_i4
 * (bindings.cpp:604-644, include/flashinfer/page.cuh:119-164). */
int sr_append_kv_i4(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                    const void *last_page_offset, const void *k, const void *v, const void *k_param,
                    const void *v_param, int64_t num_layers, int64_t layer_idx, int64_t num_heads, int64_t page_size,
                    int64_t head_dim, int64_t batch_size, void *stream);
/* A whole prompt per request; seqlen_indptr int32 [batch+1].  Replaces _CUDA.init_kv_i4
 * (bindings.cpp:561-602, page.cuh:166-219). */
int sr_init_kv_i4(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                  const void *last_page_offset, const void *k, const void *v, const void *k_param,
                  const void *v_param, const void *seqlen_indptr, int64_t total_tokens, int64_t num_layers,
                  int64_t layer_idx, int64_t num_heads, int64_t page_size, int64_t head_dim, int64_t batch_size,
                  void *stream);
/* k, v fp16 [batch, new_tokens, heads, 128]: Hadamard on K (hadamard_k), quantize both and
 * write the slots of the last new_tokens positions of every request, in one launch.
 * Replaces the chain matmul_had_cuda -> kv_quant_pack x2 -> init/append_kv_i4 of
 * MultiLayerPagedKVCache4Bit.update (signrot/transformers/kv_cache.py:308-415). */
int sr_kv_append_quant(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                       const void *last_page_offset, const void *k, const void *v, int64_t batch_size,
                       int64_t new_tokens, int64_t num_layers, int64_t layer_idx, int64_t num_heads,
                       int64_t page_size, int64_t head_dim, int hadamard_k, void *stream);
/* Fused edge of the path: rotary embedding on q and k (_CUDA.rope_qk, signrot/kernels/fused.cu:316-349),
 * then the K/V chain of sr_kv_append_quant, in one launch; same bits as sr_rope_qk followed by
 * sr_kv_append_quant (fake_quant/kernel_utils.py:118-141 + signrot/transformers/kv_cache.py:308-415).
 * q, k, v are fp16, addressed as base + token * stride + head * 128 (strides in elements, multiples
 * of 4), so they may be column ranges of one fused q/k/v projection output.  cos, sin fp16
 * [cos_seqs (1 or batch), new_tokens, 128].  q_out fp16 [batch * new_tokens, num_qo_heads, 128]
 * receives the rotated q (it may alias q when q_stride = num_qo_heads * 128); k_out (optional,
 * [batch * new_tokens, num_kv_heads, 128]) the rotated k for a dense prefill attention. */
int sr_rope_kv_append(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                      const void *last_page_offset, const void *q, const void *k, const void *v, int64_t q_stride,
                      int64_t k_stride, int64_t v_stride, const void *cos, const void *sin, int64_t cos_seqs,
                      void *q_out, void *k_out, int64_t batch_size, int64_t new_tokens, int64_t num_layers,
                      int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                      int64_t head_dim, int hadamard_k, void *stream);
/* Decode step of one layer's attention in ONE launch: sr_rope_kv_append for one new token per request followed by
 * sr_batch_decode_i4, with the bits of the two separate calls.  q, k, v: the projections BEFORE the rotary embedding
 * (fp16, base + request * stride + head * 128, strides in elements: column ranges of one fused q/k/v output are
 * fine); cos, sin fp16 [cos_seqs (1 or batch), 1, 128].  The page tables already describe the sequence INCLUDING the
 * new token.  Every CTA rotates the q heads it needs; the CTA that owns the last page of a (request, KV head) rotates,
 * quantizes and stores the new K and V before it reads that page.  Needs a page size that is a multiple of 16
 * (SR_ERR_UNSUPPORTED otherwise).  o, tmp, num_chunks, hadamard_q as for sr_batch_decode_i4; hadamard_k as for
 * sr_rope_kv_append.  No counterpart in the reference, which runs rope_qk, kv_quant_pack, append_kv_i4 and
 * batch_decode_i4 one after the other (fake_quant/kernel_utils.py:118-158). */
int sr_rope_decode_i4(void *o, const void *q, const void *k, const void *v, int64_t q_stride, int64_t k_stride,
                      int64_t v_stride, const void *cos, const void *sin, int64_t cos_seqs, void *kv_data, void *kv_param,
                      const void *kv_indptr, const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                      int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size, int64_t head_dim,
                      int64_t batch_size, void *tmp, int64_t num_chunks, int hadamard_q, int hadamard_k, void *stream);
/* o, q fp16 [batch, num_qo_heads, 128]; one new token per request attends to its cached
 * sequence.  num_qo_heads is a multiple (1, 2, 4, 8) of num_kv_heads: q head h reads KV head
 * h / (num_qo_heads / num_kv_heads).  tmp fp32 [batch, num_qo_heads, num_chunks, 132] is the
 * split-KV workspace (NULL or num_chunks <= 1: no split); a chunk is an equal share of the request's
 * 16-token blocks.  With 2 or 4 chunks (and a page size that is a multiple of 16) the chunks of a
 * (request, KV head) run as one thread-block cluster and merge through distributed shared memory:
 * tmp must still be given, it is left untouched; with any other count the states go through tmp
 * and a second launch merges them.  The result is the same
 * bits either way.  hadamard_q applies H_128/sqrt(128)
 * to q first (kv_cache.py:157-158).  Replaces _CUDA.batch_decode_i4 (bindings.cpp:508-559,
 * flashinfer.cu:11-55, include/flashinfer/decode.cuh:481-751). */
int sr_batch_decode_i4(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                       const void *kv_indices, const void *last_page_offset, int64_t num_layers, int64_t layer_idx,
                       int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size, int64_t head_dim,
                       int64_t batch_size, void *tmp, int64_t num_chunks, int hadamard_q, void *stream);
/* The same call with the split-KV merge folded into the attention kernel: the CTA of a
 * (request, KV head) that finishes last combines the chunks (same arithmetic, same chunk order as the
 * separate merge pass: identical output).  counters int32 [batch * num_kv_heads] must be zero before
 * the first call; the kernel leaves them zero, so the buffer is reused across calls, layers and
 * CUDA-graph replays on one stream.  Page sizes the tensor-core kernel does not take fall back to
 * the two-launch form. */
int sr_batch_decode_i4_merged(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                              const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                              int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                              int64_t head_dim, int64_t batch_size, void *tmp, int64_t num_chunks, void *counters,
                              int hadamard_q, void *stream);

/* Bookkeeping of one decode step of a uniform-length batch, done on the device so that it can sit at the
 * head of a captured decode graph: reads the token count `length` (int32 [1]), writes the position of
 * the token this step appends (`position`, int64 [1], = count before the step), the page tables of the
 * sequence including that token (kv_indptr int32 [batch+1], kv_indices int32 [>= batch * pages],
 * last_page_offset int32 [batch]; page of (request b, logical page j) = j * batch + b) and the new count.
 * Replaces the host-side refresh the reference's graph runner does between replays
 * (MultiLayerPagedKVCache4Bit.refresh_specs, signrot/transformers/kv_cache.py:435-487, called from
 * fake_quant/kernel_utils.py:205-214). */
int sr_decode_advance(void *length, void *position, void *kv_indptr, void *kv_indices, void *last_page_offset,
                      int64_t batch_size, int64_t page_size, int64_t max_pages, void *stream);

/* sr_batch_decode_i4 for callers that cannot hand over a workspace.  It has no counterpart in
 * the reference.  Some hosts of this library never get to call cudaMalloc: an inference
 * server that plans all device memory up front and gives plug-ins no allocator, a latency-bound
 * serving loop that cannot afford the device-wide synchronisation an allocation implies, or a
 * binding from a language runtime that only passes tensors through.  For them the split-KV
 * partial results go into a buffer that is part of the library image: 1,081,344 floats
 * (4.1 MiB = batch 16 x 32 query heads x 16 chunks x 132), resident on every GPU that loads
 * the library until the process ends.  Inputs, outputs and the cache are still the caller's.
 *  - A call that needs more than that (batch_size * num_qo_heads * num_chunks * 132 floats)
 *    is refused with SR_ERR_UNSUPPORTED and a message that states both numbers.
 *  - The first call on each device looks up the buffer's device address (the device must be
 *    current); make that first call before any stream capture begins.
 *  - All calls share the one buffer.  It is overwritten, never read before being written, so
 *    back-to-back calls on one stream are fine; two calls that can overlap on the GPU (different
 *    streams, or different host threads) race on it and must be serialised by the caller.
 *  - Nothing is allocated or freed here, by the CUDA runtime or any other library. */
int sr_batch_decode_i4_static(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                              const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                              int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                              int64_t head_dim, int64_t batch_size, int64_t num_chunks, int hadamard_q,
                              void *stream);

/* ------------------------------------------------------------------ exchanges over peer memory
 *
 * Tensor- and expert-parallel groups of up to 8 GPUs on one node.  The reference has no multi-GPU form of
 * this path (the kernel model must live on one device: fake_quant/kernel_utils.py:365-366), so these entry
 * points have no counterpart there; they stand where a sharded caller would otherwise put collective-library
 * calls of a few hundred KB (all-gather of a row-parallel linear's input, all-reduce of its int32 partial
 * sums, sum of expert-parallel partial outputs).
 *
 * Set-up (allocates; not capturable): every rank calls sr_peer_region_bytes, sr_peer_alloc (zeroed device
 * memory + a 64-byte inter-process handle), sends the handle to its peers (any host channel), and maps their
 * regions with sr_peer_open.  Tear-down: sr_peer_close on the mapped regions, sr_peer_free on the own one. */
int sr_peer_region_bytes(int64_t world, int64_t slot_bytes, int64_t *bytes);
int sr_peer_alloc(int64_t bytes, void **ptr, void *ipc_handle);
int sr_peer_open(const void *ipc_handle, void **ptr);
int sr_peer_close(void *ptr);
int sr_peer_free(void *ptr);

/* One exchange = one kernel on every rank of the group: write the message into every rank's slot with plain
 * 16-byte peer stores in which every other word is the exchange's sequence number (each line carries its own
 * "arrived" mark, so there is no separate flag and no fence: one trip across the fabric), poll the own slots
 * until every line shows the number (bounded; code 60 + rank in sr_device_status if a rank never arrives),
 * then combine the slots into `out`.  A region holds two sets of slots, used by alternate exchanges.  `regions`: host array of `world` device pointers (own region at [rank]).
 *   mode 0  all-gather of columns: src fp16 [rows, cols] -> out fp16 [rows, world * cols]
 *   mode 1  integer all-reduce + dequant: src int32 [rows, cols] -> out fp16 [rows, cols] =
 *           rn_h((float(sum over ranks) * row_scale[m]) * col_scale[n]), the epilogue of sr_w4a4_linear
 *   mode 2  fp32 all-reduce in rank order: src fp32 [rows, cols] -> out fp16 [rows, cols]
 * rows * cols * element size must fit `slot_bytes`.  Every rank must issue the same sequence of exchanges;
 * nothing is allocated or synchronised, the launch is the same every time (capturable). */
int sr_peer_exchange(int mode, const void *const *regions, int rank, int world, int64_t slot_bytes, const void *src,
                     int64_t rows, int64_t cols, const void *row_scale, const void *col_scale, void *out,
                     void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SIGNROT_B200_H_ */
