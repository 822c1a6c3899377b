/*
 * dist_moe_b200 -- C ABI of the routed-expert hot path (sm_100a).
 *
 * Every entry point is `extern "C"`, takes raw device pointers, sizes and a
 * CUDA stream (passed as void*; it is a cudaStream_t), launches asynchronously
 * on that stream, never synchronises, never allocates device memory, and
 * returns 0 on success, a negative DM_RC_* for an argument error, or a positive
 * cudaError_t.  Contract violations that only the device can see (unequal token
 * counts between ranks, receive capacity exceeded, invalid expert id, a peer
 * that never arrived) are reported through `status` (int32[8], word 0 = first
 * DM_STATUS_* code) instead of trapping, and make the dependent kernels no-ops.
 *
 * Each declaration names the reference interface it stands in for
 * (paths relative to the dist_moe repository).
 */
#ifndef DIST_MOE_B200_H_
#define DIST_MOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DM_RC_OK 0
#define DM_RC_BAD_ARG (-1)
#define DM_RC_UNSUPPORTED_SHAPE (-2)
#define DM_RC_TOO_LARGE (-3)
#define DM_RC_NO_DRIVER (-4)

#define DM_STATUS_OK 0
#define DM_STATUS_TOKEN_COUNT_MISMATCH 1
#define DM_STATUS_CAPACITY_EXCEEDED 2
#define DM_STATUS_INVALID_EXPERT_ID 3
#define DM_STATUS_BARRIER_TIMEOUT 4
#define DM_STATUS_PIPELINE_TIMEOUT 5
#define DM_STATUS_ARENA_OVERFLOW 6

/* Bytes of the routing-buffer header that precedes the int16 expert ids
 * (dist_moe/_buffers.py:33-35). Word 0 of the header is the int32 token count. */
#define DM_ROUTING_HEADER_BYTES 128

/* Library version / build probe; returns the compiled SM architecture (1000). */
int dm_version(void);

/* ---------------------------------------------------------------------------
 * Publication  (dist_moe/kernels/triton/conditional_copy.py:158-212, 302-361
 * `copy_routing_and_dispatch`; 133-155 `copy_routing`)
 *   dispatch_local[0 : T*D]   = x            (bf16, skipped when x == NULL)
 *   routing_local header      = int32 T
 *   routing_local ids         = int16(ids)   (ids are int32 or int64)
 * validate != 0 checks ids in [-1, E) and reports DM_STATUS_INVALID_EXPERT_ID.
 * ------------------------------------------------------------------------- */
int dm_publish(const void* x_bf16, const void* ids, int ids_are_int64, void* dispatch_local,
               void* routing_local, int64_t T, int64_t D, int K, int E, int validate, int* status,
               void* stream);

/* ---------------------------------------------------------------------------
 * Expert-parallel device barrier (dist_moe/_triton_ops.py:61-102
 * `symmetric_memory_barrier`; kernel dist_moe/kernels/triton/barrier.py:31-61).
 * signal_pads: device array of `ep` addresses, one uint32 pad per rank, pad
 * layout [channel][ep].  `cond` (int32*, may be NULL) predicates the barrier on
 * the device.  The wait is bounded by timeout_ns; on expiry the kernel records
 * DM_STATUS_BARRIER_TIMEOUT and returns.
 * ------------------------------------------------------------------------- */
int dm_barrier(const uint64_t* signal_pads, int rank, int ep, int channel, const int* cond,
               uint64_t timeout_ns, int* status, void* stream);

/* ---------------------------------------------------------------------------
 * Routing metadata (dist_moe/_routing_metadata.py:718-1102
 * `dist_dispatch_routing`; kernels
 * dist_moe/kernels/triton/dist_dispatch_routing_kernel.py:298-956).
 *
 * Inputs: the peers' published routing buffers (device array of `ep`
 * addresses), the peers' dispatch/combine buffer addresses, strides in bytes.
 * Outputs (all device):
 *   counts[e_local]         rows per local expert (rounded up to m_multiple_of when > 0)
 *   per_rank[ep]            rows every rank receives (same rounding)
 *   expert_offsets[e_local+1] exclusive prefix of counts; last entry = rows received
 *   fwd/bwd/sct pointer tables int64[ptrs_size]; rows ordered by (local expert,
 *   source rank, token); padding rows hold 0.  bwd may be NULL.
 * Workspace: int32 words, at least dm_route_workspace_words(...).
 * A capacity violation sets DM_STATUS_CAPACITY_EXCEEDED and zeroes the counts.
 * ------------------------------------------------------------------------- */
int64_t dm_route_workspace_words(int64_t T, int ep, int E);
int dm_route(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs, const uint64_t* combine_ptrs,
             int rank, int ep, int64_t T, int K, int E, int64_t gather_stride_bytes,
             int64_t bwd_gather_stride_bytes, int64_t scatter_stride_bytes, int m_multiple_of,
             int64_t capacity_rows, int64_t ptrs_size, int32_t* counts, int32_t* per_rank,
             int32_t* expert_offsets, int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs,
             int64_t* scatter_ptrs, int32_t* workspace, int64_t workspace_words, int* status,
             void* stream);
/* dm_route that also writes `real_counts[e_local]`, the rows of every local expert before rounding up to
 * m_multiple_of (zero after a capacity violation).  dm_gemm_blockscaled_swapped sizes its tiles from it. */
int dm_route_counted(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs, const uint64_t* combine_ptrs,
                     int rank, int ep, int64_t T, int K, int E, int64_t gather_stride_bytes,
                     int64_t bwd_gather_stride_bytes, int64_t scatter_stride_bytes, int m_multiple_of,
                     int64_t capacity_rows, int64_t ptrs_size, int32_t* counts, int32_t* real_counts,
                     int32_t* per_rank, int32_t* expert_offsets, int64_t* fwd_gather_ptrs,
                     int64_t* bwd_gather_ptrs, int64_t* scatter_ptrs, int32_t* workspace, int64_t workspace_words,
                     int* status, void* stream);

/* ---------------------------------------------------------------------------
 * dm_route_static: the same routing metadata without a caller-provided workspace.
 * (No counterpart in the reference: its launcher allocates seven temporaries per call.)
 *
 * Some hosts may not allocate device memory at the point where they route: code that
 * runs inside a memory-pool-free region of a serving loop, a plugin whose allocator
 * belongs to the embedding framework, or a process that has already handed all free
 * HBM to a KV cache.  For them the intermediate counters live in one fixed array inside
 * the library image, DM_ROUTE_STATIC_MAX_WORDS int32 words (256 KiB); every GPU that
 * loads the library carries that array until the process exits.
 *
 * Limits and rules:
 *   - the shape must satisfy dm_route_workspace_words(T, ep, E) <= DM_ROUTE_STATIC_MAX_WORDS,
 *     otherwise the call returns DM_RC_TOO_LARGE and launches nothing;
 *   - the first call on each device looks up the array's device address (with that device
 *     current);
 *   - the call itself performs no cudaMalloc/cudaFree and calls no allocating routine;
 *     inputs and outputs are still the caller's;
 *   - all calls on a device share the array.  Each call clears the part that must start
 *     at zero and overwrites the rest, so back-to-back calls on one stream are fine, but
 *     two calls whose kernels overlap on the GPU (different streams) race on it.
 * Outputs are identical to dm_route's.
 * ------------------------------------------------------------------------- */
#define DM_ROUTE_STATIC_MAX_WORDS 65536
int dm_route_static(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs, const uint64_t* combine_ptrs,
                    int rank, int ep, int64_t T, int K, int E, int64_t gather_stride_bytes,
                    int64_t bwd_gather_stride_bytes, int64_t scatter_stride_bytes, int m_multiple_of,
                    int64_t capacity_rows, int64_t ptrs_size, int32_t* counts, int32_t* per_rank,
                    int32_t* expert_offsets, int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs,
                    int64_t* scatter_ptrs, int* status, void* stream);

/* Kernel selection for dm_route / dm_route_static: non-zero (default) lets calls with ep * T <= 1024 run the whole
 * routing step in one single-CTA launch (the decode regime; the reference's single-launch path,
 * dist_moe/_routing_metadata.py:265-300); zero keeps every call on the three general kernels.  Both produce the
 * same tables bit for bit (rows ordered by local expert, source rank, token).  Returns the previous setting. */
int dm_set_route_decode_kernel(int enabled);
int dm_route_decode_kernel_enabled(void); /* the current setting, without changing it */

/* ---------------------------------------------------------------------------
 * Activation-arena planner, BF16
 * (dist_moe/_activation_buffer.py:2318-2591 `get_forward_plan`/`get_backward_plan`;
 * kernels dist_moe/_activation_buffer_planner_kernel.py:1068-1477).
 * All state tensors are device int64 and updated in place exactly as the
 * reference does.  fwd_state = [x, x_gathered, h1, h2, h3, slot id],
 * bwd_offsets = [x_gathered, h1, h2, grad_h2, grad_h3_gathered, grad_h1].
 * need_recompute is one byte (bool).  Overflow sets DM_STATUS_ARENA_OVERFLOW.
 * ------------------------------------------------------------------------- */
int dm_plan_fwd_bf16(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                     int64_t* buffer_offsets, int64_t* peak_min_free, uint8_t* need_recompute,
                     int32_t* recompute_cond, int64_t* fwd_state, const int64_t* slot_selector,
                     int64_t* moe_layer_id, int ep, int64_t num_tokens, int K, int64_t D, int64_t F,
                     int64_t slot_bytes, int num_slots, int num_moe_layers, int scratch_only,
                     int* status, void* stream);
int dm_plan_bwd_bf16(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                     int64_t* buffer_offsets, int64_t* peak_min_free, const uint8_t* need_recompute,
                     const int64_t* fwd_state, int64_t* bwd_offsets, int64_t* moe_layer_id, int ep,
                     int64_t num_tokens, int K, int64_t D, int64_t F, int64_t slot_bytes, int num_slots,
                     int* status, void* stream);

/* ---------------------------------------------------------------------------
 * Activation-arena planner, block-scaled paths
 * (dist_moe/_activation_buffer.py:2108-2315 `_get_blockscaled_forward_plan` / `_get_blockscaled_backward_plan`;
 * kernels dist_moe/_activation_buffer_planner_kernel.py:293-647 and 651-1065).
 * Same state tensors as the BF16 planner.  What is placed are bundles: quantised data immediately followed by its
 * scale factors; row bundles feed the forward / input-gradient GEMMs, column bundles the weight-gradient GEMMs.
 * `storage` (host int[6]) = {operand element bytes, values per storage element, scale element bytes,
 * row-scale storage multiple, per-row global-scale bytes, scale vector length} (the reference's
 * BlockscaledStorageConfig, dist_moe/_activation_buffer.py:958-1075): MXFP8 {1,1,1,4,0,32}, NVFP4 {1,2,1,4,4,16}.
 *   fwd_offsets[10] = {x, 0, h1, 0, h3, x_row, x_col, h2_row, h2_col, slot selector} (entry 9 is recorded so that
 *                      the backward rewinds the slot the forward used);
 *   fwd_activation_offsets[2*9]: groups {W13 dispatch, W2 combine} of
 *                      {a_q, b_q, c, a_scale, b_scale, source_x, source_y, col_q, col_scale}; -1 = not present;
 *   bwd_offsets[16] = {0|x_gathered, h1, 0|h2, grad_h2, 0|grad_h3_gathered, 0|grad_h1, x_row, x_col, h2_row, h2_col,
 *                      grad_h3_row, grad_h3_col, dxy_row, dxy_col, x_row global scales, h2_row global scales};
 *   bwd_activation_offsets[6*9]: groups {recompute dispatch, recompute combine, W2 dgrad, W2 wgrad, W13 dgrad,
 *                      W13 wgrad}.
 * per_rank_snapshot (optional) receives a copy of per_rank.  Rows above capacity_rows set
 * DM_STATUS_CAPACITY_EXCEEDED, an overflowing slot or scratch region DM_STATUS_ARENA_OVERFLOW (the reference
 * asserts on the device).
 * ------------------------------------------------------------------------- */
int dm_plan_fwd_blockscaled(const int32_t* recv_rows, const int32_t* per_rank, int32_t* per_rank_snapshot,
                            int64_t* saved_bytes_per_rank, int64_t* buffer_offsets, int64_t* peak_min_free,
                            uint8_t* need_recompute, int32_t* recompute_cond, int64_t* fwd_offsets,
                            int64_t* fwd_activation_offsets, const int64_t* slot_selector, int64_t* moe_layer_id,
                            int ep, int64_t num_tokens, int K, int64_t D, int64_t F, const int* storage,
                            int64_t capacity_rows, int64_t slot_bytes, int num_slots, int num_moe_layers, int mega,
                            int inference_mode, int scratch_only, int native_backward, int interleaved_fc13,
                            int* status, void* stream);
int dm_plan_bwd_blockscaled(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                            int64_t* buffer_offsets, int64_t* peak_min_free, const uint8_t* need_recompute,
                            const int64_t* fwd_offsets, int64_t* bwd_offsets, int64_t* bwd_activation_offsets,
                            int64_t* moe_layer_id, int ep, int64_t num_tokens, int K, int64_t D, int64_t F,
                            const int* storage, int64_t capacity_rows, int64_t slot_bytes, int num_slots, int mega,
                            int native_backward, int* status, void* stream);

/* ---------------------------------------------------------------------------
 * Row gather (the gather half of dist_moe/kernels/dist_grouped_gemm.py:1148-1237
 * `dist_grouped_gemm_fprop_dispatch` and 1441-1489 `..._dgrad_dispatch`):
 *   dst[r, :] = *(ptrs[r])   for r < *num_rows, a zero row where ptrs[r] == 0.
 * dst = dst_base + (dst_offset ? *dst_offset : 0).  Sources may be peer memory.
 * ------------------------------------------------------------------------- */
int dm_gather_rows(const int64_t* ptrs, const int32_t* num_rows, void* dst_base, const int64_t* dst_offset,
                   int64_t row_bytes, int64_t max_rows, const int* cond, void* stream);

/* Device-predicated copy (dist_moe/kernels/triton/conditional_copy.py:482-630).
 * Copies `bytes` from src(+*src_offset) to dst(+*dst_offset) when cond is NULL
 * or (*cond != 0) == (expect != 0). */
int dm_cond_copy(const void* src_base, const int64_t* src_offset, void* dst_base, const int64_t* dst_offset,
                 int64_t bytes, const int* cond, int expect, void* stream);

/* ---------------------------------------------------------------------------
 * SwiGLU (dist_moe/kernels/triton/swiglu.py:272-504 `swiglu_fwd`, 671-925 `swiglu_bwd`)
 *   h1 = [gate | up] rows of 2F bf16, h2 rows of F bf16, fp32 math.
 *   clamped: g = min(gate, limit), u = clamp(up, +-limit), h2 = g*sigmoid(alpha*g)*(u+1).
 *   clip_stats (fp32[3], may be NULL) += [#gate > clip_limit, #|up| > clip_limit, #valid].
 * Row count is read from *num_rows.
 * ------------------------------------------------------------------------- */
int dm_swiglu_fwd(const void* h1_base, const int64_t* h1_offset, void* h2_base, const int64_t* h2_offset,
                  const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped, float alpha, float limit,
                  float* clip_stats, float clip_limit, const int* cond, void* stream);
int dm_swiglu_bwd(const void* h1_base, const int64_t* h1_offset, const void* grad_h2_base,
                  const int64_t* grad_h2_offset, void* grad_h1_base, const int64_t* grad_h1_offset,
                  const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped, float alpha, float limit,
                  void* stream);

/* ---------------------------------------------------------------------------
 * Top-k reduction and its backward
 * (dist_moe/kernels/triton/broadcast_n_reduction.py:70-183 `scale_and_sum`,
 *  723-805 `reduce_from_topk`, 386-511 `broadcast_and_scale`).
 *   scale_and_sum:       out[t,:] = bf16( sum_k scores[t,k] * h3[t,k,:] ), routes with id < 0 skipped;
 *                        scores == NULL means weight 1 (reduce_from_topk).
 *                        save_base(+*save_offset) (may be NULL) receives a copy of h3 when save_cond is
 *                        NULL or (*save_cond != 0) == (save_expect != 0).
 *   broadcast_and_scale: grad_h3[t,k,:] = bf16(scores[t,k] * grad_out[t,:]);
 *                        grad_scores[t,k] = sum_d h3[t,k,d] * grad_out[t,d]  (0 for id < 0).
 * scores are fp32 or bf16 (scores_are_bf16); ids int32 or int64.
 * ------------------------------------------------------------------------- */
int dm_scale_and_sum(const void* h3, const void* scores, int scores_are_bf16, const void* ids, int ids_are_int64,
                     void* out, int64_t T, int K, int64_t D, void* save_base, const int64_t* save_offset,
                     const int* save_cond, int save_expect, void* stream);
int dm_broadcast_and_scale(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                           int ids_are_int64, const void* h3_base, const int64_t* h3_offset, void* grad_h3,
                           float* grad_scores, int64_t T, int K, int64_t D, void* stream);
/* dm_broadcast_and_scale with the expert outputs read from `h3_alt` when *use_alt != 0 (recomputed into the
 * communication buffer), else from h3_base + *h3_offset (saved in the activation slot): the choice the planner
 * made on the device, without copying the saved outputs back first. */
int dm_broadcast_and_scale_select(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                                  int ids_are_int64, const void* h3_base, const int64_t* h3_offset, const void* h3_alt,
                                  const int* use_alt, void* grad_h3, float* grad_scores, int64_t T, int K, int64_t D,
                                  void* stream);
/* Zero the rows of a bf16 [T, K, D] route tensor whose expert id is negative, before a Python callback reads it
 * (dist_moe/kernels/triton/conditional_copy.py:215-235 `zero_out_padded_rows_`, 364-380 its kernel). */
int dm_zero_padded_rows(void* routes_TKD, const void* ids, int ids_are_int64, int64_t T, int K, int64_t D, void* stream);

/* ---------------------------------------------------------------------------
 * BF16 grouped GEMMs on tcgen05/TMEM fed by TMA
 * (dist_moe/kernels/dist_grouped_gemm.py:1148-1237 fprop dispatch, 1498-1556
 *  fprop combine, 1441-1489 dgrad dispatch, 1559-1608 dgrad combine;
 *  dist_moe/kernels/grouped_gemm.py:640- `grouped_gemm_wgrad`).
 *
 * Activations live in the arena: an operand is (arena_base, arena_bytes,
 * device int64 byte offset).  Rows of local expert e are
 * [expert_offsets[e], expert_offsets[e+1]); padding rows are zero rows whose
 * scatter pointer is 0.  The allocation behind an operand must extend at least
 * 256 rows past the operand's last row (guard tail): edge tiles read, but never
 * use, what lies there.
 *
 *  dm_gemm_fprop:   C[r, :] = A[r, :] * W[e]^T           W = [e_local, N, Kd] (Kd contiguous)
 *     fuse_swiglu != 0: W = [e_local, 2, F, Kd]; writes h1 = C (2F wide) and h2 = SwiGLU(h1).
 *     scatter_ptrs != NULL: row r of C goes to scatter_ptrs[r] (peer memory) instead of C.
 *  dm_gemm_dgrad:   C[r, :] = A[r, :] * W[e]             W = [e_local, Kd, N] (N contiguous), A = [rows, Kd]
 *     scatter_ptrs as above.
 *  dm_gemm_wgrad:   dW[e] (+)= dY[e]^T * X[e]            dY = [rows, N], X = [rows, Kd], dW = [e_local, N, Kd]
 *     out_is_fp32 selects fp32 or bf16 dW; accumulate != 0 adds into dW (the fp32 accumulator is rounded to
 *     dW's type and added in L2 by bulk tensor reduce-adds, the reference's TMA reduce-add store).  dW must be
 *     16-byte aligned.
 * ------------------------------------------------------------------------- */
typedef struct {
  void* base;             /* arena (or any 256-byte aligned allocation) */
  int64_t bytes;          /* extent of that allocation, including the guard tail */
  const int64_t* offset;  /* device byte offset of the operand, NULL = 0 */
} dm_operand;

int dm_gemm_fprop(dm_operand a, const void* w, dm_operand c, dm_operand h2, const int64_t* scatter_ptrs,
                  const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N,
                  int64_t Kd, int fuse_swiglu, int clamped, float alpha, float limit, const int* cond, int num_sms,
                  int* status, void* stream);
int dm_gemm_dgrad(dm_operand a, const void* w, dm_operand c, const int64_t* scatter_ptrs,
                  const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N,
                  int64_t Kd, const int* cond, int num_sms, int* status, void* stream);
/* Fused dispatch: the same GEMMs, but the rows of A are first pulled through `gather_ptrs` (peer memory
 * allowed) by four extra warps of every CTA of the persistent kernel while the tensor cores already work
 * on the rows that have landed; `a` names where the pulled rows are kept (x_gathered / grad_h3_gathered,
 * needed again by the weight-gradient GEMMs).  gather_flags: int32[max_rows/128 + 2] scratch, cleared by
 * the call.  Replaces dist_grouped_gemm_fprop_dispatch / ..._dgrad_dispatch in one launch
 * (dist_moe/kernels/dist_grouped_gemm.py:1148-1237, 1441-1489). */
int dm_gemm_fprop_dispatch(const int64_t* gather_ptrs, int32_t* gather_flags, dm_operand a, const void* w,
                           dm_operand c, dm_operand h2, const int32_t* expert_offsets, int e_local, int64_t max_rows,
                           int64_t N, int64_t Kd, int fuse_swiglu, int clamped, float alpha, float limit,
                           const int* cond, int num_sms, int* status, void* stream);
int dm_gemm_dgrad_dispatch(const int64_t* gather_ptrs, int32_t* gather_flags, dm_operand a, const void* w,
                           dm_operand c, const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N,
                           int64_t Kd, const int* cond, int num_sms, int* status, void* stream);
int dm_gemm_wgrad(dm_operand dy, dm_operand x, void* dw, int out_is_fp32, int accumulate,
                  const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N,
                  int64_t Kd, int num_sms, int* status, void* stream);


/* ---------------------------------------------------------------------------
 * Block-scaled grouped GEMM on tcgen05 with scale factors in TMEM
 * (dist_moe/_blockscaled_ops.py:172-932: `dist_blockscaled_grouped_gemm_fprop_dispatch`,
 *  `..._fprop_swiglu_fwd_combine`; kernels dist_moe/kernels/dist_blockscaled_grouped_gemm_kernel.py).
 *   format 0 = MXFP8 (E4M3 data, E8M0 scale per 32), 1 = NVFP4 (packed E2M1 data, E4M3 scale per 16).
 *   A   [rows, Kd] quantised, row-major, with blocked scales `sfa` (rows padded to 128);
 *   W   [e_local, N, Kd] quantised with blocked scales `sfb`, one blocked group per expert;
 *   C   bf16 [rows, N] = dequant(A) * dequant(W)^T, optionally times row_scale_inv[row] (fp32, per
 *       token) and expert_scale_inv[e] (fp32) in that order (the NVFP4 global scales);
 *   scatter_ptrs != NULL sends row r of C to scatter_ptrs[r] instead;
 *   swiglu_interleaved != 0: W is W13 with rows interleaved in groups of 8 gate / 8 up rows
 *       (dist_moe/_blockscaled_weight.py:16-39); writes h2 = bf16(SwiGLU(bf16 gate, bf16 up)) [rows, N/2]
 *       and, when C is given, h1 = [gate | up] in the canonical (not interleaved) column order.
 * Every expert's row range must start on a multiple of 128 (routing with m_multiple_of = 128).
 * ------------------------------------------------------------------------- */
int dm_gemm_blockscaled(int format, dm_operand a, dm_operand sfa, const void* w, const void* sfb, dm_operand c,
                        dm_operand h2, const int64_t* scatter_ptrs, dm_operand row_scale_inv,
                        const float* expert_scale_inv, const int32_t* expert_offsets, int e_local, int64_t max_rows,
                        int64_t N, int64_t Kd, int swiglu_interleaved, int clamped, float alpha, float limit,
                        const int* cond, int num_sms, int* status, void* stream);

/* The same product for experts that received few rows (decode): weights on the 128-row side of the MMA, the
 * expert's rows on the N side in steps of 32, so that a K stage costs MMAs of N = 32 or 64 instead of a 128-row
 * tile and the layer is bound by streaming the weights once.  Replaces the reference's compact decode tiles
 * (dist_moe/kernels/chunked_mega_blockscaled_policy.py:60-95, 32-row M tiles).  Arguments as dm_gemm_blockscaled
 * plus `expert_counts` (int32 [e_local], real rows inside each 128-padded group; NULL = the whole group).  With
 * swiglu_interleaved only h2 is written (C must be NULL).  Forward only. */
int dm_gemm_blockscaled_swapped(int format, dm_operand a, dm_operand sfa, const void* w, const void* sfb, dm_operand c,
                                dm_operand h2, const int64_t* scatter_ptrs, dm_operand row_scale_inv,
                                const float* expert_scale_inv, const int32_t* expert_offsets,
                                const int32_t* expert_counts, int e_local, int64_t max_rows, int64_t N, int64_t Kd,
                                int swiglu_interleaved, int clamped, float alpha, float limit, const int* cond,
                                int num_sms, int* status, void* stream);

/* dm_gemm_blockscaled(MXFP8, swiglu_interleaved) whose epilogue quantises h2 on the way out: h2_q receives the
 * E4M3 bytes ([rows, N/2]) and h2_sf the blocked E8M0 scales of 1 x 32 blocks, bit-identical to dm_quant_mxfp8_row
 * applied to the bf16 h2 the plain call writes; h2 itself is not written (the reference's
 * `..._fprop_swiglu_fwd_combine` producers quantise h2 in the same place, dist_moe/_blockscaled_ops.py:172-420).
 */
int dm_gemm_blockscaled_swiglu_mxfp8(dm_operand a, dm_operand sfa, const void* w, const void* sfb, dm_operand h2_q,
                                     dm_operand h2_sf, const int32_t* expert_offsets, int e_local, int64_t max_rows,
                                     int64_t N, int64_t Kd, int clamped, float alpha, float limit, const int* cond,
                                     int num_sms, int* status, void* stream);

 /* the current setting, without changing it */

/* MXFP8 training backward GEMMs (dist_moe/_blockscaled_ops.py: `dist_blockscaled_grouped_gemm_dgrad_dispatch`,
 * `..._dgrad_swiglu_bwd_combine`, `blockscaled_grouped_gemm_wgrad`; sequencing dist_moe/_blockscaled.py:2284-2512).
 *
 * dm_gemm_blockscaled_dgrad: C[r, n] = sum_k dY[r, k] * W[e][k, n], bf16 rows (or scattered to scatter_ptrs[r];
 *   a null pointer skips the row).  dY [rows, Kd] is row-quantised E4M3 with blocked scales; W is the SAME
 *   qdata the forward reads ([e_local, Kd, N], 32x32-tile quantised, dist_moe/_blockscaled.py:858-881), read
 *   N-major, with the scales of the transposed orientation: per expert a blocked group of N rows x Kd/32 columns.
 *
 * dm_gemm_blockscaled_wgrad: dW[e][m, n] (=|+=) sum_{r in expert e} dY[r, m] * X[r, n], fp32 or bf16.
 *   dY_col [rows, M] and X_col [rows, N] are E4M3 quantised along the row dimension (32 consecutive rows of a
 *   column share one E8M0 scale); their scales are blocked with the feature as row index and row/32 as column
 *   index, (max_rows/32 + 3)/4 column atoms per row atom (what dm_quant_mxfp8_col writes for max_rows rows).
 *   Padding rows of an expert must hold zero data. */
int dm_gemm_blockscaled_dgrad(dm_operand dy, dm_operand sf_dy, const void* w, const void* sfb_dgrad, dm_operand c,
                              const int64_t* scatter_ptrs, const int32_t* expert_offsets, int e_local,
                              int64_t max_rows, int64_t N, int64_t Kd, const int* cond, int num_sms, int* status,
                              void* stream);
int dm_gemm_blockscaled_wgrad(dm_operand dy_col, dm_operand sf_dy_col, dm_operand x_col, dm_operand sf_x_col, void* dw,
                              int dw_is_fp32, int accumulate, const int32_t* expert_offsets, int e_local,
                              int64_t max_rows, int64_t M, int64_t N, const int* cond, int num_sms, int* status,
                              void* stream);
/* dm_gemm_blockscaled_wgrad for column bundles that the arena planner sized from the device row count: the scale
 * layout of dY_col / X_col then has expert_offsets[e_local] / 128 column atoms instead of max_rows / 128, so that a
 * bundle takes exactly dim * rows / 32 scale bytes (dist_moe/_activation_buffer_planner_kernel.py:146-161).  The
 * *_at quantisers below write that layout. */
int dm_gemm_blockscaled_wgrad_compact(dm_operand dy_col, dm_operand sf_dy_col, dm_operand x_col, dm_operand sf_x_col,
                                      void* dw, int dw_is_fp32, int accumulate, const int32_t* expert_offsets,
                                      int e_local, int64_t max_rows, int64_t M, int64_t N, const int* cond,
                                      int num_sms, int* status, void* stream);

/* ---------------------------------------------------------------------------
 * Fused post-expert RMSNorm + weighted top-k reduction
 * (dist_moe/kernels/norm/fused_rmsnorm_combine.py:576-765 forward, 802-1018 backward,
 *  427-466 the unfused composition that defines the numerics):
 *   y = cast_norm(g * h3 * rstd), rstd = rsqrt(mean((g*h3)^2) + eps), out = bf16(sum_k s_k * y_k);
 *   g = gamma + gain_center when gamma (bf16[D]) is given, else 1.  rstd_out (fp32[T,K], may be
 *   NULL) receives rstd (0 for skipped routes).  save_* as in dm_scale_and_sum.
 *   Backward writes grad_h3 (may alias h3) and grad_scores; rstd == NULL recomputes it from h3.
 * ------------------------------------------------------------------------- */
int dm_rmsnorm_combine_fwd(const void* h3, const void* scores, int scores_are_bf16, const void* ids,
                           int ids_are_int64, const void* gamma, float gain_center, float eps, int norm_is_bf16,
                           int use_kahan, void* out, float* rstd_out, int64_t T, int K, int64_t D, void* save_base,
                           const int64_t* save_offset, const int* save_cond, int save_expect, void* stream);
int dm_rmsnorm_combine_bwd(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                           int ids_are_int64, const void* h3_base, const int64_t* h3_offset, const float* rstd,
                           float eps, int norm_is_bf16, int use_kahan, void* grad_h3, float* grad_scores, int64_t T,
                           int K, int64_t D, void* stream);

/* ---------------------------------------------------------------------------
 * Block-scaled quantisers (dist_moe/_quantization.py:66-133 `quantize_for_format`;
 * dist_moe/kernels/blockscaled_quantize.py:5219 `quantize_block_scaled`, 5451
 * `quantize_block_scaled_axes`, 5080 `_quantize_nvfp4_per_token`;
 * dist_moe/kernels/scale_factor_layout.py:414 `natural_to_cublas_blocked`).
 * Inputs are bf16, row-major.  Scale bytes are written in natural row-major order or, with
 * blocked != 0, in 128x4 atoms: atom*512 + (row%32)*16 + (row/32%4)*4 + col%4, atoms ordered
 * (row atom, column atom), rows padded to 128 and scale columns to 4.
 *   dm_quant_mxfp8_row    1x32 blocks along C: q[R,C] e4m3, scales [R, C/32] e8m0; row strides in bytes
 *                         (0 = dense) let it fill the packed inference dispatch row [q | scales | pad].
 *   dm_quant_mxfp8_col    32x1 blocks along the rows: q[R,C], scales [C, ceil(max_rows/32)].
 *   dm_quant_mxfp8_tile32 32x32 tiles of W[experts*N, K]: shared q, row_scales [experts*N, K/32]
 *                         and (optional) col_scales [experts*K, N/32]; blocked groups are per expert.
 *   dm_quant_nvfp4_token  per-token NVFP4: packed e2m1 pairs (even element in the low nibble),
 *                         e4m3 scales per 16 elements and the fp32 inverse row scale, each with its
 *                         own byte stride so that the packed dispatch row [q | scales | inv | pad]
 *                         (dist_moe/_blockscaled.py:408-507) and dense outputs use the same kernel.
 *   dm_quant_nvfp4_weight per-expert NVFP4 with a given fp32 global scale per expert.
 *   dm_sf_swizzle         natural scale bytes -> blocked atoms.
 *   dm_gather_packed_rows rows [q | natural scales | fp32 inverse scale] fetched through a pointer table
 *                         (peer memory allowed; the gather half of the block-scaled dispatch,
 *                         dist_moe/kernels/dispatch_quant.py:1437-1560) and unpacked into dense q rows,
 *                         blocked scales and a per-row inverse-scale vector; null pointers give zero rows.
 * num_rows (device int32, may be NULL) bounds the rows that are processed.
 * ------------------------------------------------------------------------- */
int dm_quant_mxfp8_row(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                       int64_t q_row_stride, void* scales, int64_t scale_row_stride, int blocked, void* stream);
int dm_quant_mxfp8_col(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q, void* scales,
                       int blocked, void* stream);
/* Row- and column-quantised copies of one bf16 [rows, C] matrix in a single pass over the input (the pair the
 * MXFP8 training path needs of every activation: rows for the next GEMM, columns for the weight gradient; the
 * reference emits both from its in-GEMM quantising producers, dist_moe/kernels/dist_blockscaled_grouped_gemm_kernel.py:112-222).
 * Outputs are bit-identical to dm_quant_mxfp8_row (blocked scales) and dm_quant_mxfp8_col (blocked scales). C % 32 == 0. */
int dm_quant_mxfp8_rowcol(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q_row,
                          void* scales_row_blocked, void* q_col, void* scales_col_blocked, void* stream);
/* The same pair with the dispatch gather folded in: row r is read through row_ptrs[r] (peer memory allowed, a
 * null pointer is a row of zeros), so the gathered bf16 rows are never written (the reference's gather+quantise
 * dispatch, dist_moe/_blockscaled.py:461-507 `_stage_blockscaled_dispatch`). */
int dm_quant_mxfp8_rowcol_gather(const int64_t* row_ptrs, const int32_t* num_rows, int64_t max_rows, int64_t C,
                                 void* q_row, void* scales_row_blocked, void* q_col, void* scales_col_blocked,
                                 void* stream);
/* SwiGLU of h1 = [rows, 2F] ([gate | up]) rounded to bf16 as dm_swiglu_fwd rounds it, then quantised both ways:
 * h2 itself is never written (dist_moe/_quantization.py:151-183 `swiglu_fwd_quantize`). F % 32 == 0. */
int dm_swiglu_fwd_quant_mxfp8_rowcol(const void* h1, const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped,
                                     float alpha, float limit, void* q_row, void* scales_row_blocked, void* q_col,
                                     void* scales_col_blocked, void* stream);
/* SwiGLU backward and quantisation in one pass: from h1 = [rows, 2F] and grad_h2 = [rows, F] the row- and/or
 * column-quantised grad_h1 = [dgate | dup] ([rows, 2F]; pass NULL for the pair that is not wanted), grad_h1 rounded
 * to bf16 as dm_swiglu_bwd rounds it and never written (dist_moe/_quantization.py:186-215 `swiglu_bwd_quantize`). */
int dm_swiglu_bwd_quant_mxfp8(const void* h1, const void* grad_h2, const int32_t* num_rows, int64_t max_rows, int64_t F,
                              int clamped, float alpha, float limit, void* q_row, void* scales_row_blocked, void* q_col,
                              void* scales_col_blocked, void* stream);
/* The three fused quantisers above with every activation pointer given as (allocation, device byte offset*), for
 * bundles whose place the arena planner chose on the device (dist_moe/_blockscaled.py:461-507, 1260-1420 pass the
 * planner's offset tables to the reference's quantisers in the same way).  Column scales use the compact layout
 * (see dm_gemm_blockscaled_wgrad_compact); `num_rows` must be the padded row total the planner saw.  `cond`
 * (optional) turns the launch into a no-op when it reads 0 (recompute launches in the backward). */
int dm_quant_mxfp8_rowcol_gather_at(const int64_t* row_ptrs, const int32_t* num_rows, int64_t max_rows, int64_t C,
                                    dm_operand q_row, dm_operand sf_row, dm_operand q_col, dm_operand sf_col,
                                    const int* cond, void* stream);
int dm_swiglu_fwd_quant_mxfp8_rowcol_at(dm_operand h1, const int32_t* num_rows, int64_t max_rows, int64_t F,
                                        int clamped, float alpha, float limit, dm_operand q_row, dm_operand sf_row,
                                        dm_operand q_col, dm_operand sf_col, const int* cond, void* stream);
int dm_swiglu_bwd_quant_mxfp8_at(dm_operand h1, dm_operand grad_h2, const int32_t* num_rows, int64_t max_rows,
                                 int64_t F, int clamped, float alpha, float limit, dm_operand q_row, dm_operand sf_row,
                                 dm_operand q_col, dm_operand sf_col, void* stream);
int dm_quant_mxfp8_tile32(const void* w, int64_t experts, int64_t N, int64_t K, void* q, void* row_scales,
                          void* col_scales, int blocked, void* stream);
int dm_quant_nvfp4_token(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                         int64_t q_row_stride, void* scales, int64_t scale_row_stride, int scales_blocked,
                         void* scale_inv, int64_t inv_row_stride, void* stream);
/* dm_quant_nvfp4_token restricted to the rows r with row_live[r] != 0 (any per-row table whose padding rows hold 0,
 * e.g. the scatter pointers of the routing step): padding rows of a 128-row-padded expert group are left as they
 * are, since nothing consumes their quantised form. */
int dm_quant_nvfp4_token_live(const int64_t* row_live, const void* x, const int32_t* num_rows, int64_t max_rows,
                              int64_t C, void* q, int64_t q_row_stride, void* scales, int64_t scale_row_stride,
                              int scales_blocked, void* scale_inv, int64_t inv_row_stride, void* stream);
int dm_quant_nvfp4_weight(const void* w, const float* global_scale, int64_t experts, int64_t N, int64_t K, void* q,
                          void* scales, int blocked, void* stream);
int dm_sf_swizzle(const void* natural, void* blocked_out, int64_t rows, int64_t cols, void* stream);
int dm_gather_packed_rows(const int64_t* ptrs, const int32_t* num_rows, int64_t max_rows, int64_t q_bytes,
                          int64_t scale_cols, int has_inv, dm_operand q, dm_operand scales_blocked,
                          dm_operand scale_inv, const int* cond, void* stream);

/* ---------------------------------------------------------------------------
 * Host-backed overflow scratch (dist_moe/_vmm.py:149-427 `VMMRegion`): one contiguous virtual range whose
 * sections are physical device memory or pinned host memory, readable and writable by `device`.
 *   dm_vmm_granularity  the recommended physical granularity; section sizes must be multiples of it
 *   dm_vmm_create       reserves the range, creates and maps one allocation per section (host sections on the
 *                       GPU's NUMA node where the driver names one), grants access; returns the base address
 *                       and an opaque handle.  On failure everything created so far is released.
 *   dm_vmm_destroy      unmaps, releases, frees the range.  After a failure the handle stays valid for a retry.
 * Positive return codes >= 1000 are 1000 + CUresult of the failing driver call.
 * ------------------------------------------------------------------------- */
int dm_vmm_granularity(int device, int64_t* granularity_bytes);
int dm_vmm_create(int device, int num_sections, const int64_t* section_bytes, const int* section_is_host,
                  uint64_t* base_out, void** region_out);
int dm_vmm_destroy(void* region);

#ifdef __cplusplus
}
#endif
#endif /* DIST_MOE_B200_H_ */
