/* C ABI of libsonicmoe_b200.so: the sm_100a kernels behind the `sonicmoe` MoE layer.
 *
 * Conventions
 *   - every pointer is a device pointer unless said otherwise; the caller owns all buffers, the
 *     library borrows them for the duration of the stream-ordered launch and allocates nothing;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - functions return SMOE_OK (0) or a negative SMOE_ERR_* code; a non-zero return means nothing
 *     was launched; nothing throws;
 *   - bf16 tensors are row-major and 16-byte aligned; index tensors are int32;
 *   - T tokens, H hidden size, I expert intermediate size, E experts, K experts per token,
 *     TK routed (token, expert) pairs; "grouped" rows are sorted by expert: expert e owns rows
 *     [expert_offset[e], expert_offset[e+1]);
 *   - `status` (optional, may be NULL) is a device int32 the GEMM kernels set to a non-zero
 *     SMOE_ST_* code when one of their bounded waits ran out; the caller zeroes it and reads it.
 *
 * Each entry point cites the operator of the reference (path within the sonic-moe project) that it
 * stands in for.
 */
#ifndef SONICMOE_B200_H_
#define SONICMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SMOE_OK = 0,
  SMOE_ERR_SHAPE = -1,     /* unsupported or inconsistent sizes */
  SMOE_ERR_ALIGNMENT = -2, /* a pointer or pitch is not 16-byte aligned */
  SMOE_ERR_DRIVER = -3,    /* no usable CUDA driver / device */
  SMOE_ERR_TENSORMAP = -4, /* the driver rejected a TMA descriptor */
  SMOE_ERR_LAUNCH = -5,    /* the kernel launch itself failed */
  SMOE_ERR_DTYPE = -6,     /* unknown dtype code */
  SMOE_ERR_WORKSPACE = -7, /* workspace missing or too small */
  SMOE_ERR_NOALLOC_LIMIT = -8 /* size exceeds what the allocation-free entry point's built-in scratch holds */
};

enum { SMOE_ST_OK = 0, SMOE_ST_TIMEOUT_PRODUCER = 1, SMOE_ST_TIMEOUT_MMA = 2, SMOE_ST_TIMEOUT_EPILOGUE = 3 };

/* dtype codes for tensors whose type the caller chooses */
enum { SMOE_F32 = 0, SMOE_BF16 = 1, SMOE_I32 = 2, SMOE_I64 = 3 };

/* Library version, for the loader to check that it found the right build. */
int smoe_abi_version(void);

/* ---------------------------------------------------------------------------------------------
 * Router: top-k, softmax over the winners, histogram / prefix sum, grouped-row index vectors
 * ------------------------------------------------------------------------------------------- */

/* Per row of logits (T,E) [SMOE_F32 or SMOE_BF16]: the K largest values, largest first, equal values
 * ordered by lower column; scores (T,K) fp32 = softmax over those K values; indices (T,K) int32.
 * Replaces sonicmoe::_softmax_topk_fwd / _topk_fwd (sonicmoe/functional/forward.py:20-50, 224-237;
 * kernel sonicmoe/functional/topk_softmax.py:86-193). */
int smoe_topk_softmax(const void* logits, int logits_dtype, float* scores, int* indices, int T, int E, int K,
                      void* stream);

/* dlogits (T,E) [SMOE_F32 or SMOE_BF16], every element written: dlogits[t, indices[t,k]] =
 * score[t,k] * (dscore[t,k] - sum_j dscore[t,j] score[t,j]), zero elsewhere.
 * Replaces sonicmoe::_softmax_topk_bwd (sonicmoe/functional/backward.py:488-556) and the zero fill
 * before it (sonicmoe/functional/__init__.py:107). */
int smoe_softmax_topk_backward(void* dlogits, int dlogits_dtype, const float* dscore, const float* score,
                               const int* indices, int T, int E, int K, void* stream);

/* count[e] = #{i : x[i] == e}, cumsum[e] = count[0] + ... + count[e] (cumsum may be NULL); x is
 * SMOE_I32 or SMOE_I64 of length n; ids outside [0,E) are ignored.  workspace: device scratch of
 * smoe_count_cumsum_workspace_bytes(E) bytes (needed for E <= 4096).
 * Replaces sonicmoe::count_cumsum_cuda (sonicmoe/count_cumsum/__init__.py:11-29, kernel.cu:93-203). */
size_t smoe_count_cumsum_workspace_bytes(int E);
int smoe_count_cumsum(const void* x, int x_dtype, long long n, int E, int* count, int* cumsum, void* workspace,
                      void* stream);

/* Allocation-free form of smoe_count_cumsum (same arguments minus the workspace, same results).  It has no
 * counterpart in the reference.  It exists for hosts that can hand this library nothing but the input and
 * output buffers: a runtime whose device memory is planned ahead of time and owns the only allocator, or a call
 * site where cudaMalloc's implicit device-wide synchronisation cannot be tolerated.  The scratch is a 512 KiB
 * array compiled into the library (held by every GPU that loads it), which limits E to
 * smoe_count_cumsum_noalloc_max_experts() = 1024; a larger E returns SMOE_ERR_NOALLOC_LIMIT.  The first call on
 * a device resolves the array's address and should happen before any stream capture.  Calls on one device share
 * the array: they must not overlap on the GPU (issue them on one stream, or order the streams). */
int smoe_count_cumsum_noalloc_max_experts(void);
int smoe_count_cumsum_noalloc(const void* x, int x_dtype, long long n, int E, int* count, int* cumsum,
                              void* stream);

/* From the flat expert id of each of n routed pairs: expert_count (E), expert_offset (E+1, leading 0),
 * and a stable counting sort by expert: s_scatter_idx[r] = flat slot of grouped row r,
 * s_reverse_scatter_idx[slot] = r, x_gather_idx[r] = token of row r (slot / K, or token_idx[slot] when
 * token_idx != NULL).  E <= 4096.  workspace: smoe_route_metadata_workspace_bytes(E) bytes.
 * Replaces count_cumsum + TC_topk_router_metadata / general_routing_router_metadata
 * (sonicmoe/functional/__init__.py:19-82). */
size_t smoe_route_metadata_workspace_bytes(int E);
int smoe_route_metadata(const int* expert_idx, const int* token_idx, long long n, int E, int K, int* expert_count,
                        int* expert_offset, int* s_scatter_idx, int* s_reverse_scatter_idx, int* x_gather_idx,
                        void* workspace, void* stream);

/* offsets[t] = number of entries of the ascending vector sorted_idx (length n) that are < t, t = 0..T.
 * Replaces the per-token count_cumsum / bincount of general_routing_router_metadata
 * (sonicmoe/functional/__init__.py:66-73). */
int smoe_sorted_offsets(const int* sorted_idx, long long n, int T, int* offsets, void* stream);

/* Token rounding: after the top-K choice, round every expert's token count to a multiple of `tile`
 * (SMOE_ROUND_DOWN floor, SMOE_ROUND_UP ceil, SMOE_ROUND_NEAREST nearest with ties to even, each capped at T) by
 * dropping the expert's lowest-ranked top-K tokens or admitting its best-ranked other tokens.  Ranking of the
 * tokens of one expert: tokens whose top-K holds the expert, by score; then the others by (score - 1), rounded in
 * the scores' dtype; equal values by lower token id.
 * scores (T,E) [SMOE_F32 or SMOE_BF16]: probabilities with the top-K entries already renormalised; topk_idx (T,K).
 * Outputs: expert_count (E) = rounded counts; the kept pairs as tokens / experts (ascending token, ascending
 * expert within a token), at most `capacity` of them written; num_pairs (1) = their number (sum of expert_count).
 * workspace: smoe_token_rounding_workspace_bytes(T,E) bytes, 16-byte aligned.
 * Replaces the ranking matrix, the argsort over tokens, the count mask and the final argsort of
 * forward_token_choice_rounding (benchmarks/moe-token-rounding.py:153-191), whose tie order is unspecified. */
enum { SMOE_ROUND_DOWN = 0, SMOE_ROUND_UP = 1, SMOE_ROUND_NEAREST = 2 };
size_t smoe_token_rounding_workspace_bytes(int T, int E);
int smoe_token_rounding_select(const void* scores, int scores_dtype, const int* topk_idx, int T, int E, int K,
                               int tile, int mode, int* expert_count, int* tokens, int* experts, int* num_pairs,
                               int capacity, void* workspace, void* stream);

/* out[t,:] = sum over p in [token_offset[t], token_offset[t+1]) (or [t*K, (t+1)*K) when token_offset is
 * NULL) of weights[p] * src[reverse_idx[p], :]; weights NULL = 1, else SMOE_F32 / SMOE_BF16; src, out
 * bf16 with H columns; fp32 accumulation.  Replaces sonicmoe::_router_forward and
 * sonicmoe::_token_broadcast_backward (sonicmoe/functional/forward.py:181-202, backward.py:464-484;
 * kernel sonicmoe/functional/reduction_over_k_gather.py:447-556). */
int smoe_gather_sum(const void* src, void* out, const void* weights, int weights_dtype, const int* reverse_idx,
                    const int* token_offset, int T, int H, int K, void* stream);

/* dst (bf16) = src (fp32), n elements, n % 8 == 0: finishes the fused scatter-reduce output. */
int smoe_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);

/* ds[s_scatter_idx[r]] = sum_c ds_partial[c, r]; ds is SMOE_F32 or SMOE_BF16.
 * Replaces the ds_partial reduction of _down_projection_backward (sonicmoe/functional/backward.py:391-408). */
int smoe_ds_reduce(const float* ds_partial, const int* s_scatter_idx, void* ds, int ds_dtype, int TK, int ncols,
                   void* stream);

/* ---------------------------------------------------------------------------------------------
 * Grouped GEMMs (tcgen05 / TMEM / TMA)
 * ------------------------------------------------------------------------------------------- */

/* z[r, :] = x[x_gather_idx[r], :] @ W1[e]^T, y1[r, j] = silu(z[r, 2j]) * z[r, 2j+1] for every grouped
 * row r of expert e.  x (T,H); w1 (E,2I,H) gate/up rows interleaved; z (TK,2I) or NULL (inference);
 * y1 (TK,I).  Replaces sonicmoe::_up_projection_forward (sonicmoe/functional/forward.py:53-126). */
int smoe_up_projection_forward(const void* x, const void* w1, void* z, void* y1, const int* expert_offset,
                               const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                               void* stream);

/* y2[r, :] = y1[r, :] @ W2[e]^T.  w2 (E,H,I); y2 (TK,H).
 * Replaces sonicmoe::_down_projection_forward (sonicmoe/functional/forward.py:132-175). */
int smoe_down_projection_forward(const void* y1, const void* w2, void* y2, const int* expert_offset, int H, int I,
                                 int E, int TK, int* status, void* stream);

/* Layers whose tokens have exactly one routed row each (top-1 routing; the rows an expert-parallel rank receives):
 * the combine is a permutation, so the down projection writes o[x_gather_idx[r], :] = score[s_scatter_idx[r]] *
 * bf16(y2[r, :]) directly (scores NULL = 1) and the dX GEMM writes dx[x_gather_idx[r], :] directly -- no y2 /
 * dx_expanded buffer, no gather-and-sum pass.  Every row of o / dx is written exactly once when x_gather_idx is a
 * permutation of 0..TK-1.  Same results, bit for bit, as smoe_down_projection_forward + smoe_gather_sum (K = 1) and
 * smoe_up_projection_backward_dx + smoe_gather_sum (K = 1).  (Reference: the K = 1 case of _down_projection_forward +
 * _router_forward, forward.py:132-202, and of _up_projection_backward + _token_broadcast_backward,
 * backward.py:195-280, 464-484.) */
int smoe_down_projection_forward_rows(const void* y1, const void* w2, void* o, const void* scores, int scores_are_bf16,
                                      const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                      int H, int I, int E, int TK, int* status, void* stream);
int smoe_up_projection_backward_dx_rows(const void* dz, const void* w1, void* dx, const int* expert_offset,
                                        const int* x_gather_idx, int H, int I, int E, int TK, int* status,
                                        void* stream);

/* Fused down projection + router-weighted scatter-reduce: o_acc[x_gather_idx[r], :] += score(r) * (y1[r] @ W2[e]^T)
 * with fp32 atomics; o_acc (T,H) fp32 must be zero on entry.  score(r) = scores[s_scatter_idx[r]].
 * Replaces _down_projection_forward followed by _router_forward (sonicmoe/functional/forward.py:132-202). */
int smoe_down_projection_forward_scatter(const void* y1, const void* w2, float* o_acc, const void* scores,
                                         int scores_are_bf16, const int* expert_offset, const int* x_gather_idx,
                                         const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                         void* stream);

/* dy1 = dout[x_gather_idx[r]] @ W2[e]; y1 recomputed from z; dz = dswiglu(z) * dy1 * s, y1s = y1 * s,
 * ds_partial[c, r] = sum over the c-th 128-column block of dy1 * y1.  ds_partial has
 * smoe_ds_partial_columns(I) * TK floats.  Replaces the dz kernel of sonicmoe::_down_projection_backward
 * (sonicmoe/functional/backward.py:286-389). */
int smoe_down_projection_backward_act(const void* dout, const void* w2, const void* z, const void* scores,
                                      int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                      const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                      int T, int H, int I, int E, int TK, int* status, void* stream);
int smoe_ds_partial_columns(int I);

/* dx_expanded[r, :] = dz[r, :] @ W1[e].  dx_expanded (TK,H).
 * Replaces the dx kernel of sonicmoe::_up_projection_backward (sonicmoe/functional/backward.py:259-280). */
int smoe_up_projection_backward_dx(const void* dz, const void* w1, void* dx_expanded, const int* expert_offset, int H,
                                   int I, int E, int TK, int* status, void* stream);

/* dW2[e] (H,I) = sum over rows r of expert e of dout[x_gather_idx[r], :]^T y1s[r, :]; zeros for an empty expert.
 * Replaces the dw2 kernel of sonicmoe::_down_projection_backward (sonicmoe/functional/backward.py:438-458). */
int smoe_down_projection_weight_grad(const void* dout, const void* y1s, void* dw2, const int* expert_offset,
                                     const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                     void* stream);

/* dW1[e] (2I,H) = sum over rows r of expert e of dz[r, :]^T x[x_gather_idx[r], :].
 * Replaces the dw1 kernel of sonicmoe::_up_projection_backward (sonicmoe/functional/backward.py:237-257). */
int smoe_up_projection_weight_grad(const void* x, const void* dz, void* dw1, const int* expert_offset,
                                   const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                   void* stream);

/* The two weight gradients added to what dw2 / dw1 already hold: dW += (the chunk's gradient rounded to bf16),
 * added in fp32 and rounded to bf16.  An expert without rows, and TK == 0, leave the buffer untouched.
 * A batch whose rows arrive in several chunks (the micro-batches of the expert-parallel exchange) stores the first
 * chunk with the calls above and adds the later ones here.  That is the accumulation autograd performs for a
 * weight used twice, without its extra read-add-write pass over both gradient tensors (the reference's kernels
 * write the gradient of the whole batch at once: sonicmoe/functional/backward.py:237-257, 438-458). */
int smoe_down_projection_weight_grad_accumulate(const void* dout, const void* y1s, void* dw2,
                                                const int* expert_offset, const int* x_gather_idx, int T, int H, int I,
                                                int E, int TK, int* status, void* stream);
int smoe_up_projection_weight_grad_accumulate(const void* x, const void* dz, void* dw1, const int* expert_offset,
                                              const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                              void* stream);

/* ---------------------------------------------------------------------------------------------
 * Any activation of the layer, and expert biases.  Activation codes: 0 swiglu, 1 geglu, 2 reglu (gated:
 * W1[e] has 2I rows, gate row 2j / up row 2j+1), 3 relu_sq, 4 relu, 5 gelu (erf), 6 silu (W1[e] has I rows).
 * N1 = rows of W1[e] (2I or I), a multiple of 128.  Biases are bf16 (E, N1) / (E, H) or NULL.
 * ------------------------------------------------------------------------------------------- */

/* z = x[gather] W1[e]^T + b1[e]; y1 = act(z).  z (TK,N1) or NULL; y1 (TK,I).  Replaces _up_projection_forward
 * with a bias and any activation_type (sonicmoe/functional/forward.py:53-126, grouped_gemm.py:1170-1288, 2439-2452). */
int smoe_up_projection_forward_act(const void* x, const void* w1, const void* b1, void* z, void* y1,
                                   const int* expert_offset, const int* x_gather_idx, int T, int H, int N1, int E,
                                   int TK, int activation, int* status, void* stream);

/* y2 = y1 W2[e]^T + b2[e] (sonicmoe/functional/forward.py:132-175 with b2). */
int smoe_down_projection_forward_bias(const void* y1, const void* w2, const void* b2, void* y2,
                                      const int* expert_offset, int H, int I, int E, int TK, int* status,
                                      void* stream);

/* smoe_down_projection_backward_act for any activation: dz (TK,N1), y1s (TK,I), ds_partial as there. */
int smoe_down_projection_backward_dact(const void* dout, const void* w2, const void* z, const void* scores,
                                       int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                       const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                       int T, int H, int I, int E, int TK, int activation, int* status,
                                       void* stream);

/* out[e, n] = sum over grouped rows r of expert e of w_r * src[row(r), n]; row(r) = gather_idx[r] (or r when NULL),
 * w_r = scores[s_scatter_idx[r]] (or 1 when scores is NULL).  out bf16 (E,N).  db1 = column sums of dz, db2 = score-
 * weighted column sums of dout rows.  Replaces db1_kernel / db2 of db2_and_ds_kernel (sonicmoe/functional/backward.py:36-168). */
int smoe_expert_column_sum(const void* src, long long ld, const int* gather_idx, const void* scores,
                           int scores_dtype, const int* s_scatter_idx, const int* expert_offset, void* out, int E,
                           int N, void* stream);

/* ds[s_scatter_idx[r]] += <dout[x_gather_idx[r], :], b2[e(r), :]> (the "ds += dout . b2" part of db2_and_ds_kernel). */
int smoe_ds_add_bias_term(const void* dout, const void* b2, const int* expert_offset, const int* x_gather_idx,
                          const int* s_scatter_idx, void* ds, int ds_dtype, int E, int H, int TK, void* stream);

/* ---------------------------------------------------------------------------------------------
 * FP8 (E4M3) path: fp32 block scales, scale = amax / 448 (1 for an all-zero block).  Activations: one scale
 * per row and 128 consecutive columns; weights: one scale per 128 x 128 block of each expert's matrix.
 * Requires H % 128 == 0 and I % 128 == 0.  The reference has no FP8 path: these entry points have the
 * argument conventions of their bf16 counterparts above, with every fp8 operand followed by its scales.
 * The weight-gradient GEMMs stay in bf16.
 * ------------------------------------------------------------------------------------------- */

/* q (rows, cols) uint8 E4M3 and scale (rows, cols/128) fp32 from x (rows, cols) bf16; cols % 128 == 0. */
int smoe_fp8_quantize_rows(const void* x, void* q, float* scale, long long rows, int cols, void* stream);

/* q (batch, rows, cols) and scale (batch, ceil(rows/128), cols/128) from w (batch, rows, cols) bf16. */
int smoe_fp8_quantize_blocks(const void* w, void* q, float* scale, int batch, int rows, int cols, void* stream);

/* As smoe_up_projection_forward with xq (T,H) + x_scale (T,H/128), w1q (E,2I,H) + w1_scale (E,2I/128,H/128);
 * z, y1 are written in bf16. */
int smoe_fp8_up_projection_forward(const void* xq, const float* x_scale, const void* w1q, const float* w1_scale,
                                   void* z, void* y1, const int* expert_offset, const int* x_gather_idx, int T, int H,
                                   int I, int E, int TK, int* status, void* stream);

/* As smoe_down_projection_forward with y1q (TK,I) + y1_scale (TK,I/128), w2q (E,H,I) + w2_scale (E,H/128,I/128). */
int smoe_fp8_down_projection_forward(const void* y1q, const float* y1_scale, const void* w2q, const float* w2_scale,
                                     void* y2, const int* expert_offset, int H, int I, int E, int TK, int* status,
                                     void* stream);

/* As smoe_down_projection_backward_act with doutq (T,H) + dout_scale (T,H/128) and the quantised W2; z, dz, y1s bf16. */
int smoe_fp8_down_projection_backward_act(const void* doutq, const float* dout_scale, const void* w2q,
                                          const float* w2_scale, const void* z, const void* scores,
                                          int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                          const int* expert_offset, const int* x_gather_idx,
                                          const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                          void* stream);

/* As smoe_up_projection_backward_dx with dzq (TK,2I) + dz_scale (TK,2I/128) and the quantised W1. */
int smoe_fp8_up_projection_backward_dx(const void* dzq, const float* dz_scale, const void* w1q, const float* w1_scale,
                                       void* dx_expanded, const int* expert_offset, int H, int I, int E, int TK,
                                       int* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * FP8 (E4M3) path with power-of-two block scales in UE8M0 (one byte = exponent + 127), applied by the tensor
 * cores' own block scaling (tcgen05.mma kind::mxf8f6f4.block_scale) instead of in software.  Same block shapes
 * as above; scale = the smallest power of two >= amax / 448 (2^0 for an all-zero block).  Activation scales are
 * (rows, smoe_mxfp8_scale_row_bytes(cols)) bytes: byte b of a row belongs to columns [128 b, 128 b + 128), rows
 * padded to whole 32-bit words (4-byte aligned base).  Weight scales are (batch, ceil(rows/128), cols/128) bytes.
 * The GEMM entry points take the same arguments as their smoe_fp8_* namesakes.  No reference counterpart.
 * ------------------------------------------------------------------------------------------- */
int smoe_mxfp8_scale_row_bytes(int cols);
int smoe_mxfp8_quantize_rows(const void* x, void* q, void* scale, long long rows, int cols, void* stream);
int smoe_mxfp8_quantize_blocks(const void* w, void* q, void* scale, int batch, int rows, int cols, void* stream);
int smoe_mxfp8_up_projection_forward(const void* xq, const void* x_scale, const void* w1q, const void* w1_scale,
                                     void* z, void* y1, const int* expert_offset, const int* x_gather_idx, int T,
                                     int H, int I, int E, int TK, int* status, void* stream);
/* As smoe_mxfp8_up_projection_forward, with y1 leaving the epilogue quantised instead of in bf16: y1q (TK, I) E4M3
 * and y1_scale (TK, smoe_mxfp8_scale_row_bytes(I)) UE8M0 bytes, bit-identical to smoe_mxfp8_quantize_rows applied to
 * the bf16 y1 (padding bytes of y1_scale, present when I/128 is not a multiple of 4, are left to the caller).
 * z == NULL = inference mode. */
int smoe_mxfp8_up_projection_forward_q(const void* xq, const void* x_scale, const void* w1q, const void* w1_scale,
                                       void* z, void* y1q, void* y1_scale, const int* expert_offset,
                                       const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                       void* stream);
int smoe_mxfp8_down_projection_forward(const void* y1q, const void* y1_scale, const void* w2q, const void* w2_scale,
                                       void* y2, const int* expert_offset, int H, int I, int E, int TK, int* status,
                                       void* stream);
int smoe_mxfp8_down_projection_backward_act(const void* doutq, const void* dout_scale, const void* w2q,
                                            const void* w2_scale, const void* z, const void* scores,
                                            int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                            const int* expert_offset, const int* x_gather_idx,
                                            const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                            void* stream);
/* As smoe_mxfp8_down_projection_backward_act, and dz also leaves the epilogue quantised: dzq (TK, 2I) E4M3 and
 * dz_scale (TK, smoe_mxfp8_scale_row_bytes(2I)) UE8M0 bytes, bit-identical to smoe_mxfp8_quantize_rows(dz) (padding
 * bytes of dz_scale, present when 2I/128 is not a multiple of 4, are left to the caller). */
int smoe_mxfp8_down_projection_backward_act_q(const void* doutq, const void* dout_scale, const void* w2q,
                                              const void* w2_scale, const void* z, const void* scores,
                                              int scores_are_bf16, void* dz, void* y1s, float* ds_partial, void* dzq,
                                              void* dz_scale, const int* expert_offset, const int* x_gather_idx,
                                              const int* s_scatter_idx, int T, int H, int I, int E, int TK,
                                              int* status, void* stream);
int smoe_mxfp8_up_projection_backward_dx(const void* dzq, const void* dz_scale, const void* w1q, const void* w1_scale,
                                         void* dx_expanded, const int* expert_offset, int H, int I, int E, int TK,
                                         int* status, void* stream);
/* The one-row-per-token forms (see smoe_down_projection_forward_rows) with FP8 operands. */
int smoe_mxfp8_down_projection_forward_rows(const void* y1q, const void* y1_scale, const void* w2q,
                                            const void* w2_scale, void* o, const void* scores, int scores_are_bf16,
                                            const int* expert_offset, const int* x_gather_idx,
                                            const int* s_scatter_idx, int H, int I, int E, int TK, int* status,
                                            void* stream);
int smoe_mxfp8_up_projection_backward_dx_rows(const void* dzq, const void* dz_scale, const void* w1q,
                                              const void* w1_scale, void* dx, const int* expert_offset,
                                              const int* x_gather_idx, int H, int I, int E, int TK, int* status,
                                              void* stream);

/* ---------------------------------------------------------------------------------------------
 * Fused routing front end
 * ------------------------------------------------------------------------------------------- */

/* One pass over x (T,H) bf16 with router_w (E,H) bf16: logits (T,E) bf16 = round(x . router_w^T, fp32
 * accumulation); scores (T,K) fp32 and indices (T,K) int32 as smoe_topk_softmax gives them on those logits;
 * expert_count (E) int32 = tokens per expert; prob_colsum (E) fp32 = column sums of softmax(logits, dim 1) in fp32
 * (the mean router probability of the load-balancing loss, before normalisation).  Bit-reproducible.
 * Stands in for the router linear + sonicmoe::_softmax_topk_fwd + the softmax and column sum of the aux loss
 * (sonicmoe/functional/__init__.py:438-446, sonicmoe/moe.py:251-274).  Supported when
 * smoe_router_forward_supported(H, E, K): H % 64 == 0, 32 <= E <= 256, E % 32 == 0, K <= 16.
 * workspace: smoe_router_forward_workspace_bytes(E) bytes of device memory. */
int smoe_router_forward_supported(int H, int E, int K);
size_t smoe_router_forward_workspace_bytes(int E);
int smoe_router_forward(const void* x, const void* router_w, void* logits, float* scores, int* indices,
                        int* expert_count, float* prob_colsum, void* workspace, int T, int H, int E, int K,
                        int* status, void* stream);
/* dlogits (T,E) bf16, every element written: the sum of g_logits (T,E) bf16 (optional), of the gradient through
 * the K winners' softmax (dscores, scores (T,K) fp32, indices; optional, as smoe_softmax_topk_backward) and of the
 * gradient g_colsum (E) fp32 of prob_colsum (optional; the row's softmax is recomputed from logits (T,E) bf16).
 * Replaces sonicmoe::_softmax_topk_bwd (sonicmoe/functional/backward.py:488-556) plus autograd's softmax backward
 * of the aux loss. */
int smoe_router_backward(void* dlogits, const void* logits, const float* dscores, const float* scores,
                         const int* indices, const float* g_colsum, const void* g_logits, int T, int E, int K,
                         void* stream);

/* ---------------------------------------------------------------------------------------------
 * Expert parallelism over peer memory (one node, NVLink / NVSwitch).  The reference has no distributed
 * code (sonicmoe/moe.py:260 skips even the aux-loss reduction), so these have no counterpart there; they
 * carry the dispatch / combine exchange of an expert-sharded layer.
 * ------------------------------------------------------------------------------------------- */
enum { SMOE_MAX_PEERS = 16, SMOE_PEER_HANDLE_BYTES = 64 };

/* A device buffer other processes of the node can map (cudaMalloc + zero fill) and its release.  These two are
 * the only functions of the library that allocate; every rank calls them once per exchange buffer, not per step. */
int smoe_peer_alloc(size_t bytes, void** ptr /* host out */);
int smoe_peer_free(void* ptr);
/* CUDA IPC: export a smoe_peer_alloc buffer as 64 opaque bytes (host memory) to hand to the other ranks; map a
 * buffer another rank exported (peer access to its GPU is enabled on first use); unmap it. */
int smoe_peer_export(const void* ptr, unsigned char* handle64 /* host out */);
int smoe_peer_open(const unsigned char* handle64 /* host */, void** ptr /* host out */);
int smoe_peer_close(void* ptr);
/* Stream-ordered copy of a contiguous segment between any two device buffers (local or mapped peer memory);
 * runs on a copy engine, leaves the multiprocessors to the GEMMs. */
int smoe_peer_copy(void* dst, const void* src, size_t bytes, void* stream);
/* Arrival flags without a kernel: the stream itself writes a 32-bit value to device memory of this GPU, or waits
 * until each of `count` consecutive 32-bit words at addr is >= value (cyclic comparison, so a counter may wrap).
 * A sender copies its data and then (same stream, smoe_peer_copy of 4 bytes) its exchange counter into the
 * receiver's flag word; the receiver's stream waits on the words of all senders.  Neither side occupies a
 * multiprocessor, so the hand-shake proceeds while persistent GEMM kernels hold every one of them (an NCCL
 * barrier kernel would wait for a free multiprocessor and then keep it from the next GEMM).
 * The reference has no multi-GPU path; these serve sonicmoe/expert_parallel.py of this library.
 * Returns SMOE_ERR_DRIVER when the driver offers no stream memory operations. */
int smoe_stream_write_value(void* addr, unsigned int value, void* stream);
int smoe_stream_wait_values(const void* addr, int count, unsigned int value, void* stream);
/* smoe_gather_sum whose output rows are cut into num_segments consecutive segments, each written to its own
 * destination: output row t of segment s (segment_start[s] <= t < segment_start[s+1]) goes to row
 * t - segment_start[s] of the (rows, H) bf16 buffer segment_ptr[s], which may be mapped peer memory (16-byte
 * peer stores).  With K = 1 and no weights it is the dispatch of routed token rows fused with their gather;
 * with token_offset it is the return of per-token sums fused with the reduction.  segment_ptr (num_segments)
 * and segment_start (num_segments + 1, first 0, last T) are HOST arrays; num_segments <= SMOE_MAX_PEERS.
 * The grid walks the output rows from first_row (0 <= first_row < T) round to first_row - 1: ranks that each pass
 * the first row of their right-hand neighbour's segment write to different destinations at any one time instead of
 * all to rank 0 first (every link then carries one sender's traffic, not everybody's).
 * The caller orders the ranks (a barrier after the launch) before anybody reads what was written. */
int smoe_gather_sum_to_peers(const void* src, const void* weights, int weights_dtype, const int* reverse_idx,
                             const int* token_offset, int T, int H, int K, void* const* segment_ptr /* host */,
                             const int* segment_start /* host */, int num_segments, int first_row, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SONICMOE_B200_H_ */
