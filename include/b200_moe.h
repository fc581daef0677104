/*
 * b200_moe.h - C ABI of the sm_100a mixture-of-experts kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, it is a cudaStream_t / CUstream) and returns 0 when the
 * work was enqueued, -1 on a rejected argument or a launch error (message on
 * stderr) - the convention of the reference's op submitters
 * (libdataflowops/src/submit_ops/moe_ops.c:30-36). Nothing here allocates
 * device memory: all buffers, scratch included, belong to the caller, as in
 * the reference where ops never allocate at submit time. The one exception is
 * b200_build_expert_mapping_static, whose scratch is an array inside the
 * library (see there).
 *
 * Each declaration names the reference interface it stands in for (paths are
 * relative to the reference project root) or says that the reference has no
 * counterpart.
 *
 * Limits: the router and mapping ops take up to B200_MAX_EXPERTS experts; the grouped expert GEMMs
 * (b200_moe_experts_*, b200_moe_block_*, b200_ep_moe_block_*) take up to 1024 experts per call (their group tables
 * live in shared memory) and return -1 beyond; b200_build_expert_mapping_static additionally needs its tables to fit
 * its 4 MiB array (64 experts always do; about 393 experts at large token counts).
 *
 * Threading: like the reference's op table (libdataflow/include/dataflow_table.h:6) the entry points expect one
 * submitting host thread per process and device; the library keeps small caches per device ordinal (kernel
 * attributes, SM count, the address of its status word on that device) that are filled on first use without locking,
 * so one process may drive several devices by switching the current device between calls.
 *
 * Element types use the reference's DataflowDatatype numbering
 * (libdataflow/include/dataflow_common.h:46-74).
 */
#ifndef B200_MOE_H
#define B200_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_DT_NONE 0
#define B200_DT_FP32 3
#define B200_DT_BF16 5

#define B200_MAX_EXPERTS 4096 /* moe/build_expert_mapping.cu:3 MAX_NUM_EXPERTS */
#define B200_MAX_TOP_K 32

/* Library / device identification. Returns 0 and fills sm_count, cc_major, cc_minor of the current device. */
int b200_device_info(int *sm_count, int *cc_major, int *cc_minor);

/* ---- router ------------------------------------------------------------------ */

/*
 * Replaces dataflow_submit_default_select_experts
 * (libdataflowops/include/dataflow_ops.h:216-222; kernel
 * backends/nvidia/src/ops/src/native/src/moe/select_experts.cu:3-295).
 * Per token: top-k of n_experts logits with the reference's slot order and
 * tie rule (equal values keep the lower expert index), softmax over the k
 * kept logits -> token_expert_weights[T,k] (fp32), chosen_experts[T,k] (u16);
 * expert_counts[n_experts+1] += histogram (caller zeroes it; entry n_experts
 * is a finished-block counter as in the reference); expert_counts_cumsum
 * [n_experts] = exclusive prefix sums; host_expert_counts (optional, may be
 * mapped pinned host memory) = counts. x_dt must be B200_DT_FP32 or
 * B200_DT_BF16 (bf16 logits are widened to fp32 before comparing).
 */
int b200_select_experts(int x_dt, int total_tokens, int n_experts, int top_k_experts, const void *X_routed,
                        float *token_expert_weights, uint16_t *chosen_experts, int *expert_counts,
                        int *expert_counts_cumsum, int *host_expert_counts, void *stream);

/*
 * Replaces dataflow_submit_default_build_expert_mapping
 * (dataflow_ops.h:225-228; moe/build_expert_mapping.cu:18-103).
 * Counting-sort scatter: expert_mapping[row] = token, token_mapping[t*k+j] =
 * row; expert_counts_cumsum goes from exclusive to inclusive prefix sums as in
 * the reference. Unlike the reference (atomic arrival order) the order inside
 * an expert is deterministic: tokens ascending, then slots ascending.
 * workspace: at least b200_build_expert_mapping_workspace_bytes() bytes of
 * device scratch, 16-byte aligned; contents need no initialisation.
 */
size_t b200_build_expert_mapping_workspace_bytes(int total_tokens, int num_routed_experts, int num_selected_experts);
int b200_build_expert_mapping(int total_tokens, int num_routed_experts, int num_selected_experts,
                              const uint16_t *chosen_experts, int *expert_counts_cumsum, int *expert_mapping,
                              int *token_mapping, void *workspace, size_t workspace_bytes, void *stream);

/*
 * build_expert_mapping for callers that cannot supply device scratch. (No counterpart in the
 * reference: its kernel keeps its tables in shared memory and atomics.)
 *
 * Who needs it: code that reaches this library through a fixed op signature - the reference's
 * backend calls an op with exactly the arguments of its skeleton, seven for this op, so there
 * is no slot for a workspace pointer - and that runs where allocating is off limits: the
 * framework carves all device memory into its own slabs at start-up and ops must not call
 * cudaMalloc while work is being submitted. Same inputs, outputs and result as
 * b200_build_expert_mapping; the histogram tables sit in a 4 MiB array that is part of the
 * library image on every GPU that loads it, for the life of the process.
 *
 * Limits and rules:
 *  - b200_build_expert_mapping_workspace_bytes(...) must not exceed
 *    b200_build_expert_mapping_static_capacity_bytes() (4 MiB: e.g. 64 experts at any token
 *    count, up to 393 experts at large token counts); larger problems are refused with -1 and a
 *    message, nothing is launched.
 *  - The first call on each device looks up the array's device address (the device must be
 *    current). Make that first call before starting any stream capture.
 *  - All calls on a device share the one array. It keeps whatever the previous call left; that
 *    is harmless because every entry is rewritten before it is read. Two calls that can overlap
 *    on the GPU (different streams, no dependency) race on it - serialise them.
 *  - Nothing is allocated or freed, on the device or through any library, in any call.
 */
size_t b200_build_expert_mapping_static_capacity_bytes(void);
int b200_build_expert_mapping_static(int total_tokens, int num_routed_experts, int num_selected_experts,
                                     const uint16_t *chosen_experts, int *expert_counts_cumsum, int *expert_mapping,
                                     int *token_mapping, void *stream);

/* ---- permute / combine ---------------------------------------------------------- */

/*
 * Replaces dataflow_submit_default_prepare_experts (dataflow_ops.h:230-234;
 * moe/prepare_expert_zone.cu:69-117): expert_zone[token_mapping[t,j], :] = X[t, :].
 * bf16 rows, model_dim % 8 == 0, 16-byte aligned pointers.
 */
int b200_prepare_experts(int total_tokens, int model_dim, int num_selected_experts, const void *X,
                         const int *token_mapping, void *expert_zone, void *stream);

/*
 * prepare_experts with every copied row scaled by its gate weight:
 * expert_zone[token_mapping[t,j], :] = bf16(X[t, :] * token_expert_weights[t,j]).
 * This is the row rewrite that dataflow_submit_router_bwd_x performs on the
 * upstream gradient (moe/router_bwd_x.cu:83-90, 190-192), split from the dot
 * product so the backward needs no recomputed expert output.
 */
int b200_prepare_experts_weighted(int total_tokens, int model_dim, int num_selected_experts, const void *X,
                                  const int *token_mapping, const float *token_expert_weights, void *expert_zone,
                                  void *stream);

/*
 * Replaces dataflow_submit_default_prepare_expert_zone (dataflow_ops.h:236-241;
 * moe/prepare_expert_zone.cu:28-67): gathers one expert's rows; expert_zone
 * points at that expert's first row; expert_counts_cumsum is inclusive.
 */
int b200_prepare_expert_zone(int model_dim, const void *X, int expert_id, const int *expert_counts,
                             const int *expert_counts_cumsum, const int *expert_mapping, void *expert_zone,
                             void *stream);

/*
 * Replaces dataflow_submit_default_merge_experts (dataflow_ops.h:243-249;
 * moe/merge_expert_result.cu:118-247):
 * X_combined[t,:] = bf16(f32(X_combined[t,:]) + sum_j w[t,j] * zone[token_mapping[t,j],:]),
 * fp32 accumulation in slot order, one rounding. token_expert_weights == NULL
 * means all weights 1.0 (the backward un-permute).
 */
int b200_merge_experts(int num_tokens, int model_dim, int top_k_experts, const void *expert_zones,
                       const int *token_mapping, const float *token_expert_weights, void *X_combined,
                       void *stream);

/*
 * The un-permute of the backward in one pass: X_out[t, :] = bf16(sum_j zone[token_mapping[t, j], :]) (fp32 sum in slot
 * order, one rounding), X_out is NOT read. The reference gets the same bits by zeroing dX and calling merge_experts
 * with NULL weights (dataflow_transformer.c:3642-3660); this form saves the memset and the read of the zeros. No
 * separate counterpart in the reference.
 */
int b200_unpermute_experts(int num_tokens, int model_dim, int top_k_experts, const void *expert_zones,
                           const int *token_mapping, void *X_out, void *stream);

/*
 * Replaces dataflow_submit_default_merge_expert_result (dataflow_ops.h:251-259;
 * moe/merge_expert_result.cu:3-115): one expert's read-modify-write combine.
 * num_tokens is that expert's row count, expert_zone its first row.
 */
int b200_merge_expert_result(int num_tokens, int model_dim, int top_k_experts, const void *expert_zone,
                             int expert_id, const int *expert_counts_cumsum, const int *expert_mapping,
                             const float *token_expert_weights, const uint16_t *chosen_experts,
                             void *X_combined, void *stream);

/* ---- router backward --------------------------------------------------------------- */

/*
 * Replaces dataflow_submit_router_bwd_x (dataflow_ops.h:262-272;
 * moe/router_bwd_x.cu:4-92), one expert per call:
 * dX_routed[t, expert_id] = bf16(<expert_out[r,:], upstream_dX[t,:]>) and
 * dX_expert_out[r,:] = bf16(upstream_dX[t,:] * w[t, expert_id]); expert_out and
 * dX_expert_out point at the expert's first row and may be the same buffer.
 */
int b200_router_bwd_x(int num_expert_tokens, int model_dim, int num_routed_experts, int top_k_active,
                      int expert_id, const int *expert_counts_cumsum, const int *expert_mapping,
                      const uint16_t *chosen_experts, const float *token_expert_weights, const void *expert_out,
                      const void *upstream_dX, void *dX_routed, void *dX_expert_out, void *stream);

/*
 * Replaces dataflow_submit_router_gate_bwd_x (dataflow_ops.h:275-280;
 * moe/router_gate_bwd_x.cu:7-57): softmax-over-k Jacobian in place on the k
 * chosen columns of dX_routed[T, E] (bf16).
 */
int b200_router_gate_bwd_x(int num_tokens, int num_routed_experts, int top_k_active,
                           const uint16_t *chosen_experts, const float *token_expert_weights, void *dX_routed,
                           void *stream);

/* ---- activations ---------------------------------------------------------------------- */

/* Replaces dataflow_submit_default_swiglu (dataflow_ops.h:284-287;
 * activations/swiglu.cu:66-151): out = silu(x_w1) * x_w3, bf16, fp32 math. num_cols % 8 == 0. */
int b200_swiglu(int num_rows, int num_cols, const void *x_w1, const void *x_w3, void *out, void *stream);

/* Replaces dataflow_submit_default_swiglu_bwd_x (dataflow_ops.h:290-294;
 * activations/swiglu_bwd_x.cu:111-256). */
int b200_swiglu_bwd_x(int num_rows, int num_cols, const void *x_w1, const void *x_w3, const void *upstream_dX,
                      void *dX_w1, void *dX_w3, void *stream);

/* ---- dense GEMM --------------------------------------------------------------------------- */

/*
 * Replaces the matmul external op: dataflow_submit_matmul
 * (dataflow_ops.h:70-77) -> cublas_matmul
 * (backends/nvidia/src/ops/src/external/matmul_helper/src/matmul_helper.c:774-946).
 * Column-major D[M x N] = alpha * op(A) * op(B) + beta * C with packed leading
 * dimensions (matmul_helper.c:347-420), fp32 accumulation on tcgen05 tensor
 * cores. a_dt = b_dt = B200_DT_BF16; d_dt (and c_dt when C is used) bf16 or
 * fp32; C may be NULL (beta ignored) or alias D. M must be a multiple of 8; so must K
 * unless (to_trans_a == 0 && to_trans_b == 1), and N when to_trans_b == 1 (16-byte rows for TMA).
 * workspace (the reference's kernelWorkspace argument, matmul_op.c:33-53) may be NULL. When it is given, 16-byte
 * aligned, and the product has too few output tiles to fill the GPU but a long reduction (the router's GEMMs), the
 * reduction is cut into up to 16 ranges whose fp32 partial results (M * N * 4 bytes each) go to the workspace and
 * are summed in a fixed order by a second kernel: same result up to fp32 summation order, deterministic.
 */
int b200_matmul(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                float alpha, float beta, const void *A, const void *B, const void *C, void *D,
                uint64_t workspaceBytes, void *workspace, void *stream);

/*
 * The same product on operands that are slices of larger row-major arrays (one head of a [tokens][heads * head_dim]
 * tensor, a score matrix with a padded row pitch): lda, ldb, ldd are the row pitches in elements of A, B and of
 * C = D as stored, multiples of 8. M (the output's column count) must be a multiple of 8 but only a_m_extent of A's M
 * rows / columns need exist: the rest reads as zeros, so a ragged key count can be rounded up without touching memory
 * past the slice. K and N are free. No split reduction. No counterpart in the reference (its matmul op is packed).
 */
int b200_matmul_strided(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                        float alpha, float beta, const void *A, int64_t lda, int a_m_extent, const void *B, int64_t ldb,
                        const void *C, void *D, int64_t ldd, void *stream);

/*
 * The GEMM kernels bound every wait on a barrier (about 2 s). A kernel that gives up records a
 * non-zero code here and returns without finishing its tiles. This call synchronises the
 * device, reports the code (0 = none) and clears it. The reference has no counterpart: its
 * asynchronous errors surface at the next stream sync
 * (backends/nvidia/src/handle/src/cuda_dataflow_handle.c:354-448).
 */
int b200_gemm_status(int *status_out);

/*
 * Tile shape of the GEMM kernels: 1 (default) = pairs of CTAs share one 256-row tcgen05 MMA (cta_group::2),
 * 0 = one CTA per 128-row tile. The environment variable B200_GEMM_PAIR=0 selects 0 at start-up.
 * Results are the same up to fp32 summation order. No counterpart in the reference.
 */
int b200_gemm_set_pair_mode(int on);

/*
 * Work unit of the CTA-pair GEMMs: which kinds of launch let one fetch of the A rows feed two adjacent column tiles
 * (a 256 x 512 output block per CTA pair, a quarter fewer bytes staged per flop) - bit 0 the expert forward / dgrad
 * launches, bit 1 the expert weight gradients, bit 2 the dense matmul. A launch with too few units to fill the GPU
 * that way keeps one column tile per unit unless bit 3 is set. Off by default (mask 0): with both accumulators of a unit
 * finishing together the epilogue is not hidden, and no launch of the layer gains; the environment variable
 * B200_GEMM_WIDE=<0..15> sets the mask at start-up. Results are identical either way (same MMAs per output element,
 * same order). No counterpart in the reference.
 */
int b200_gemm_set_wide_mode(int mask);

/*
 * Runs the GEMM kernels' tile scheduler on the HOST (the same code the device runs) and lists the tiles one launch
 * would process, in processing order: for checking the index arithmetic where there is no GPU. group_mode 0 = dense,
 * 1 = groups along the rows (forward / dgrad), 2 = groups along the reduction (wgrad); pair as in
 * b200_gemm_set_pair_mode, or 2 = CTA pairs with two column tiles per unit (b200_gemm_set_wide_mode);
 * M = output rows (dense, wgrad), N = output columns, K = reduction length; dual_b = 1 for
 * the fused W1 | W3 launch; counts / cumsum_incl are host arrays of num_groups ints (unused when dense);
 * k_splits / k_split_len describe a split reduction (dense only, 0 = none). Writes up to max_tiles records of nine
 * ints {group, first A row, first output row, valid rows, first column, valid columns, loaded columns, first
 * reduction row, reduction length} to out and returns the number of tiles (-1 on bad arguments). No counterpart in
 * the reference.
 */
int b200_gemm_enumerate_tiles(int group_mode, int pair, int M, int N, int K, int dual_b, int num_groups,
                              const int *counts, const int *cumsum_incl, int k_splits, int k_split_len, int max_tiles,
                              int *out);

/* ---- grouped expert GEMMs (additive ops; the reference loops experts on the host) ----------- */

/*
 * Expert weights: W1, W3 are [ffn_dim][model_dim] and W2 is [model_dim][ffn_dim]
 * per expert (models/init_model.py:291-306), bf16; expert e's matrix starts at
 * base + e * stride_elems (the reference packs w1,w3,w2 per expert,
 * libdataflowmodels/src/transformer/src/prep_transformer.c:155-159, so strides
 * larger than one matrix are allowed; they must be multiples of 8 elements).
 * expert_counts_cumsum is the INCLUSIVE cumsum left by build_expert_mapping;
 * expert_counts the histogram from select_experts. Rows of expert e are
 * [cumsum[e]-counts[e], cumsum[e]) of every [R, *] array.
 */

/*
 * Forward of all experts in two launches, replacing the host loop
 * libdataflowmodels/src/transformer/src/dataflow_transformer.c:2848-2940:
 * x1 = Z W1^T, x3 = Z W3^T, h = silu(x1)*x3 (all bf16 [R, ffn_dim]), then
 * Y = h W2^T ([R, model_dim]; may alias zone).
 */
int b200_moe_experts_fwd(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *zone,
                         const void *W1, const void *W3, const void *W2, int64_t w1_stride_elems,
                         int64_t w3_stride_elems, int64_t w2_stride_elems, const int *expert_counts,
                         const int *expert_counts_cumsum, void *x1, void *x3, void *h, void *Y, void *stream);

/*
 * Backward-x of all experts, replacing dataflow_transformer.c:3460-3641
 * without recomputing the W2 forward. dY_zone holds the upstream gradient
 * rows scaled by their gate weight and gathered into expert order
 * (b200_prepare_experts_weighted on dOut - the rows router_bwd_x leaves in the
 * zone); row_weights[R] the gate weight of each routed row. Per row r:
 *   dh     = dY W2 (rounded to bf16 as the reference stores it)
 *   dP[r] += <h[r,:], dh[r,:]> / w_r   (fp32; equals <Y[r,:], dOut[t,:]>, the
 *             dot product router_bwd_x takes against the recomputed output)
 *   (dx1, dx3) = swiglu'(x1, x3, dh);  hs = silu(x1)*x3 again if hs != NULL
 *   dZ     = dx1 W1 + dx3 W3           (must not alias dY_zone while dW2 is
 *                                       still to be computed from it)
 * dP must be zeroed by the caller (the kernel accumulates into it). The partial sums of a row come from several
 * column tiles and are added with fp32 atomics, in whatever order the tiles finish: dP, and the router gradients
 * formed from it, can differ in their last bits between two runs on the same inputs (the reference's router_bwd_x
 * reduces each row inside one block in a fixed order). dx1, dx3, hs and dZ are bit-reproducible.
 */
int b200_moe_experts_bwd_x(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                           const float *row_weights, const void *x1, const void *x3, const void *W1,
                           const void *W3, const void *W2, int64_t w1_stride_elems, int64_t w3_stride_elems,
                           int64_t w2_stride_elems, const int *expert_counts, const int *expert_counts_cumsum,
                           void *dx1, void *dx3, void *hs, float *dP, void *dZ, void *stream);

/*
 * Weight gradients of all experts (dataflow_transformer.c:3548-3560 and
 * 4101-4148), accumulated into bf16 gradient buffers with one rounding
 * (beta = 1, C = D): dW2[e] += dY_e^T hs_e; dW1[e] += dx1_e^T Z_e;
 * dW3[e] += dx3_e^T Z_e. dY_zone is the weight-scaled gathered upstream
 * gradient, hs the SwiGLU output h (saved by the forward or rewritten by
 * b200_moe_experts_bwd_x), zone_x the gathered layer input.
 * Any of the three products is skipped when its gradient pointer is NULL.
 */
int b200_moe_experts_bwd_w(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                           const void *hs, const void *zone_x, const void *dx1, const void *dx3, void *dW1,
                           void *dW3, void *dW2, int64_t dw1_stride_elems, int64_t dw3_stride_elems,
                           int64_t dw2_stride_elems, const int *expert_counts, const int *expert_counts_cumsum,
                           void *stream);

/* The same with beta = 0: the weight gradients are written, not added to, and the old contents of dW1 / dW3 / dW2 are
 * not read (a tenth of the three launches' time at the benchmark shape). For the first micro-batch of a step, in place
 * of zeroing the buffers and accumulating. No counterpart in the reference, whose gradient GEMMs always accumulate. */
int b200_moe_experts_bwd_w_overwrite(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                           const void *hs, const void *zone_x, const void *dx1, const void *dx3, void *dW1,
                           void *dW3, void *dW2, int64_t dw1_stride_elems, int64_t dw3_stride_elems,
                           int64_t dw2_stride_elems, const int *expert_counts, const int *expert_counts_cumsum,
                           void *stream);

/* row_weights[token_mapping[t,j]] = token_expert_weights[t,j]; dP_tok[t, chosen[t,j]] (bf16 [T,E], pre-zeroed)
 * = bf16(dP[token_mapping[t,j]]). Small helpers around the fused backward. */
int b200_scatter_row_weights(int num_tokens, int top_k, const int *token_mapping, const float *token_expert_weights,
                             float *row_weights, void *stream);
int b200_gather_router_grad(int num_tokens, int num_routed_experts, int top_k, const int *token_mapping,
                            const uint16_t *chosen_experts, const float *dP, void *dX_routed, void *stream);

/* ---- the whole MoE feed-forward in one call --------------------------------------------------- */

/*
 * Buffers of one MoE feed-forward: the MoE fields of the reference's Seq_Batch_Saved_Activations
 * (libdataflowmodels/include/seq_batch_structs.h:256-281) plus the workspace its block carves
 * (Seq_Batch_Activation_Workspace, 369-395). R = total_tokens * top_k. All device memory, all the caller's.
 */
typedef struct B200MoeBlock {
  int total_tokens, model_dim, num_experts, top_k, ffn_dim;
  /* bf16 weights: Wr [E][d]; W1, W3 [E][f][d]; W2 [E][d][f]; strides between experts in elements */
  const void *Wr, *W1, *W3, *W2;
  int64_t w1_stride_elems, w3_stride_elems, w2_stride_elems;
  /* written by the forward, read by the backward */
  float *logits;               /* [T][E] fp32 */
  float *token_expert_weights; /* [T][k] */
  uint16_t *chosen_experts;    /* [T][k] */
  int *expert_counts;          /* [E + 1] */
  int *expert_counts_cumsum;   /* [E], inclusive after the forward */
  int *host_expert_counts;     /* optional (NULL): mapped pinned host memory, valid after a stream sync */
  int *expert_mapping;         /* [R] */
  int *token_mapping;          /* [T][k] */
  void *zone, *x1, *x3, *h;    /* bf16 [R][d], [R][f], [R][f], [R][f] */
  void *Y;                     /* bf16 [R][d]: expert outputs before the combine */
  void *mapping_workspace;     /* b200_build_expert_mapping_workspace_bytes(T, E, k) bytes */
  size_t mapping_workspace_bytes;
  void *matmul_workspace;      /* optional (NULL): fp32 scratch for the router GEMMs' split reduction, see b200_matmul */
  size_t matmul_workspace_bytes;
  /* backward workspace (may be NULL for forward-only use) */
  void *dY_zone;               /* bf16 [R][d] */
  float *row_weights, *dP;     /* [R] each */
  void *dx1, *dx3;             /* bf16 [R][f] */
  void *dZ;                    /* bf16 [R][d] (may be the same memory as Y) */
  void *dX_routed;             /* bf16 [T][E] */
} B200MoeBlock;

/*
 * Forward of the MoE part of dataflow_submit_transformer_moe_block
 * (libdataflowmodels/src/transformer/src/dataflow_transformer.c:2710-2974): router GEMM (fp32 logits),
 * select_experts, build_expert_mapping, prepare_experts, all experts' SwiGLU MLP in two grouped launches,
 * merge_experts onto X_combined (which holds the residual). Zeroes the counters itself. Unlike the reference there
 * is no stream synchronisation in the middle (2789) and no host loop over experts: the row counts stay on the
 * device.
 */
int b200_moe_block_fwd(const B200MoeBlock *block, const void *Xn, void *X_combined, void *stream);

/*
 * Stands in for the MoE part of dataflow_submit_transformer_moe_block_recompute (2989-3323) when the forward's
 * workspace (zone, h - and x1, x3 unless they were saved) has been reused before the backward runs: re-gathers the
 * zone from Xn with the saved token_mapping and re-forms h = silu(x1) * x3, from the saved x1, x3
 * (recompute_x1_x3 == 0) or together with x1, x3 from the zone in one grouped launch (recompute_x1_x3 != 0). The W2
 * product is never recomputed: b200_moe_block_bwd does not need it. Results are bit-identical to the forward's.
 * b200_moe_experts_fwd with Y == NULL (and W2 == NULL) is the gate-up launch alone.
 */
int b200_moe_block_recompute(const B200MoeBlock *block, const void *Xn, int recompute_x1_x3, void *stream);

/*
 * The reference's saved-activation levels (libdataflowmodels/include/transformer/seq_batch_structs.h:199-204), for
 * the MoE part of a block. At every level from INP_ONLY up the routing results are kept (router logits, chosen
 * experts, gate weights, counts, cumsum, both mappings: they sit before the "input only" cut-off of the reference's
 * saved-activations buffer, libdataflowmodels/src/transformer/src/prep_seq_batch.c:230-283); x1 and x3 are kept only
 * at FULL (prep_seq_batch.c:320-365); the zone and h are workspace at every level. NONE keeps nothing: no backward.
 */
#define B200_SAVED_ACTIVATION_LEVEL_NONE 0
#define B200_SAVED_ACTIVATION_LEVEL_INP_ONLY 1
#define B200_SAVED_ACTIVATION_LEVEL_INP_ATTN_ONLY 2
#define B200_SAVED_ACTIVATION_LEVEL_FULL 3

/* Bytes of the MoE part of a saved-activations buffer at `level` (0 for NONE or an unknown level): the tensors
 * above in the reference's order, each starting on a 256-byte boundary as in prep_seq_batch.c:230-283. */
uint64_t b200_moe_saved_activations_bytes(int total_tokens, int num_experts, int top_k, int ffn_dim, int level);

/*
 * Copies what `level` keeps out of the block's buffers into `buffer` (device memory, or pinned host memory for the
 * host offload the reference's drivers do between forward and backward) and back. Asynchronous on `stream`, one
 * cudaMemcpyAsync per tensor; the layout is that of b200_moe_saved_activations_bytes. -1 at level NONE.
 */
int b200_moe_block_save_activations(const B200MoeBlock *block, int level, void *buffer, uint64_t buffer_bytes,
                                    void *stream);
int b200_moe_block_restore_activations(const B200MoeBlock *block, int level, const void *buffer, uint64_t buffer_bytes,
                                       void *stream);

/*
 * dataflow_submit_transformer_moe_block_recompute by level (dataflow_transformer.c:2989-3006, 3199-3315): at FULL the
 * reference has nothing to recompute; here the zone is gathered and h formed again from the kept x1, x3 (the
 * backward of this library reads both, the reference re-forms h inside its backward). Below FULL the zone, x1, x3 and
 * h are all formed again from Xn and the kept token_mapping; the router is not re-run. NONE is an error, as in the
 * reference ("cannot recompute with no block input").
 */
int b200_moe_block_recompute_level(const B200MoeBlock *block, const void *Xn, int level, void *stream);

/*
 * Backward of the same: what dataflow_submit_transformer_moe_block_bwd_x (3399-3719) and
 * dataflow_submit_transformer_moe_block_bwd_w (4062-4185) compute between them. dXn [T][d] is overwritten; dWr
 * [E][d], dW1, dW3 [E][f][d], dW2 [E][d][f] (bf16) are accumulated into (beta = 1, one rounding), as the
 * reference's gradient GEMMs do; dW1 / dW3 / dW2 may be NULL to skip the weight gradients. The expert output is not
 * recomputed (3494-3516): the router's dot product comes out of the W2-dgrad epilogue.
 */
int b200_moe_block_bwd(const B200MoeBlock *block, const void *Xn, const void *dOut, void *dXn, void *dWr, void *dW1,
                       void *dW3, void *dW2, void *stream);

/* The same, writing dWr / dW1 / dW3 / dW2 instead of accumulating into them (b200_moe_experts_bwd_w_overwrite and a
 * router weight-gradient GEMM with beta = 0). */
int b200_moe_block_bwd_overwrite(const B200MoeBlock *block, const void *Xn, const void *dOut, void *dXn, void *dWr, void *dW1,
                       void *dW3, void *dW2, void *stream);

/* ---- the reference's model directory -------------------------------------------------------------------- */

/*
 * config.txt of a model directory: the twenty "Name: value" lines the reference parses with one sscanf
 * (libdataflowmodels/src/transformer/src/prep_seq_batch.c:84-130; struct in
 * libdataflowmodels/include/dataflow_models.h:69-90; writer models/init_model.py:153-156). Same fields, same order.
 */
typedef struct B200ModelConfig {
  char embed_dtype[16], attn_dtype[16], router_dtype[16], expert_dtype[16], head_dtype[16];
  int vocab_size, num_layers, model_dim, head_dim, num_q_heads, num_kv_heads;
  char qk_norm_type[16], qk_norm_weight_type[16];
  int num_shared_experts, num_routed_experts, top_k_routed_experts, expert_dim;
  char expert_mlp_type[16];
  int rope_theta;
  float rms_norm_epsilon;
} B200ModelConfig;

int b200_parse_model_config(const char *config_txt_path, B200ModelConfig *out);

/*
 * Byte offsets inside layers/<i>/combined_layer.weight, computed as set_transformer_block_weight_offsets does
 * (libdataflowmodels/src/transformer/src/prep_transformer.c:24-165): attention norm, q, k, v, o, ffn norm, router,
 * then per expert w1, w3, w2, every tensor starting at the running size rounded up to pointer_alignment (0 = packed;
 * the reference's drivers use 256). Experts are equally spaced: expert e's w1 starts at w1_first + e *
 * expert_stride_bytes, likewise w3, w2. Shared experts, if any, precede the routed ones in the file.
 */
typedef struct B200MoeLayerLayout {
  uint64_t attn_norm, w_q, w_k, w_v, w_o, ffn_norm, router;
  uint64_t w1_first, w3_first, w2_first, expert_stride_bytes;
  int num_experts_in_file, first_routed_expert;
  uint64_t raw_bytes, aligned_bytes; /* sum of the tensor sizes; size of the laid-out block = size of the file */
} B200MoeLayerLayout;

int b200_moe_layer_file_layout(const B200ModelConfig *config, int pointer_alignment, B200MoeLayerLayout *out);

/*
 * load_transformer_block (prep_transformer.c:368-388): reads exactly `bytes` (= layout.aligned_bytes) from the file
 * into host_buffer; a file that is shorter or longer is refused. The caller copies the buffer to the device.
 */
int b200_read_layer_file(const char *path, void *host_buffer, uint64_t bytes);

/*
 * bind_transformer_block for the MoE part (prep_transformer.c:316-366): points block->Wr, W1, W3, W2 and the expert
 * strides at the tensors of a layer laid out at layer_base (device memory, a copy of the file), and sets model_dim,
 * num_experts, top_k, ffn_dim from the configuration. bf16 router and expert weights only.
 */
int b200_moe_block_bind_weights(B200MoeBlock *block, const B200ModelConfig *config, const B200MoeLayerLayout *layout,
                                const void *layer_base);

/* ---- expert parallelism over NVLink peer memory (no counterpart in the reference, which is single-GPU) ---- */

/*
 * Rank g of `world` owns experts [g*experts_per_rank, (g+1)*experts_per_rank). peer_buffers is a HOST array of
 * `world` device addresses: entry h is rank h's receive buffer as mapped into this process (entry of this rank =
 * its own buffer). In an owner's buffer the rows of an expert are grouped by source rank; dst_base[e] (device,
 * int[num_experts]) is the first row, in the owner's buffer, of this rank's rows of expert e. A routed pair (t, j)
 * with local row r = token_mapping[t, j] of expert e = chosen_experts[t, j] lives at row
 * dst_base[e] + r - (expert_counts_cumsum[e] - expert_counts[e]) of rank e / experts_per_rank (inclusive cumsum).
 * The kernels use plain peer loads / stores; the caller separates the phases with a barrier across the ranks.
 * capacity_rows is the number of rows every rank's buffer holds: a routed pair whose row would lie past it is
 * skipped (never written or read), so a receive buffer that turns out too small loses rows but is not overrun; the
 * caller compares the received row total with the capacity (on the device, without a host round trip, if it likes).
 */

/* prepare_experts fused with the dispatch: row (t, j) = X[t, :] (times token_expert_weights[t, j] when that pointer
 * is not NULL) is stored straight into its owner's buffer. Only pairs whose expert has an index inside its owner
 * (expert % experts_per_rank) in [local_expert_begin, local_expert_end) are moved, so that the exchange can run in
 * slices under the GEMMs of the previous slice; pass 0 and experts_per_rank for all of them. */
int b200_ep_dispatch_rows(int total_tokens, int model_dim, int top_k, const void *X, const float *token_expert_weights,
                          const int *token_mapping, const uint16_t *chosen_experts, const int *expert_counts,
                          const int *expert_counts_cumsum, const int *dst_base,
                          const unsigned long long *peer_buffers, int world, int num_experts, int experts_per_rank,
                          int64_t capacity_rows, int local_expert_begin, int local_expert_end, void *stream);

/* merge_experts fused with the return: X_combined[t, :] += sum_j w[t, j] * row (t, j), every row loaded from its
 * owner's buffer; token_expert_weights == NULL means 1.0 (backward un-permute). */
int b200_ep_combine_rows(int num_tokens, int model_dim, int top_k, const float *token_expert_weights,
                         const int *token_mapping, const uint16_t *chosen_experts, const int *expert_counts,
                         const int *expert_counts_cumsum, const int *dst_base, const unsigned long long *peer_buffers,
                         int world, int num_experts, int experts_per_rank, int64_t capacity_rows, void *X_combined,
                         void *stream);

/* dX_routed[t, chosen[t, j]] = bf16(dP[row (t, j)] / w[t, j]) with dP (fp32 per routed row, holding w * <Y, dOut> as
 * b200_moe_experts_bwd_x leaves it when row_weights are all 1) read from the owners' buffers. dX_routed pre-zeroed. */
int b200_ep_gather_router_grad(int num_tokens, int top_k, const float *token_expert_weights, const int *token_mapping,
                               const uint16_t *chosen_experts, const int *expert_counts,
                               const int *expert_counts_cumsum, const int *dst_base,
                               const unsigned long long *peer_dP_buffers, int world, int num_experts,
                               int experts_per_rank, int64_t capacity_rows, void *dX_routed, void *stream);

/*
 * GEMM fused with the return exchange. A row tag is (rank << 40) | row. b200_ep_publish_row_tags writes, for every
 * routed pair (t, j) of this rank, the tag (my_rank << 40) | token_mapping[t, j] into entry row (t, j) of the owner's
 * tag array (peer_tag_buffers: host array of `world` device addresses of unsigned long long arrays, addressed like
 * the row buffers above). After a barrier, the owner runs the *_scatter forms of the grouped passes: they are
 * b200_moe_experts_fwd / b200_moe_experts_bwd_x except that the rows of the last GEMM (Y, resp. dZ) are not stored in
 * place: the epilogue stores row r at row (row_tags[r] & (2^40 - 1)) of dest_buffers[row_tags[r] >> 40]
 * ([rows_per_buffer, model_dim] bf16 each; plain stores, peer memory allowed), i.e. straight into the zone-ordered
 * buffer of the token's home rank, where b200_merge_experts / b200_merge_expert_result then run locally. A tag
 * outside (world, rows_per_buffer) is not stored and raises status 5 (b200_gemm_status). No counterpart in the
 * reference, which runs on one GPU.
 */
int b200_ep_publish_row_tags(int num_tokens, int top_k, int my_rank, const int *token_mapping,
                             const uint16_t *chosen_experts, const int *expert_counts, const int *expert_counts_cumsum,
                             const int *dst_base, const unsigned long long *peer_tag_buffers, int world,
                             int num_experts, int experts_per_rank, int64_t capacity_rows, void *stream);

int b200_moe_experts_fwd_scatter(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *zone,
                                 const void *W1, const void *W3, const void *W2, int64_t w1_stride_elems,
                                 int64_t w3_stride_elems, int64_t w2_stride_elems, const int *expert_counts,
                                 const int *expert_counts_cumsum, void *x1, void *x3, void *h,
                                 const unsigned long long *row_tags, const unsigned long long *dest_buffers, int world,
                                 int64_t rows_per_buffer, void *stream);

int b200_moe_experts_bwd_x_scatter(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                                   const float *row_weights, const void *x1, const void *x3, const void *W1,
                                   const void *W3, const void *W2, int64_t w1_stride_elems, int64_t w3_stride_elems,
                                   int64_t w2_stride_elems, const int *expert_counts, const int *expert_counts_cumsum,
                                   void *dx1, void *dx3, void *hs, float *dP, const unsigned long long *row_tags,
                                   const unsigned long long *dest_buffers, int world, int64_t rows_per_buffer,
                                   void *stream);

/*
 * ---- the expert-parallel layer as one C call per direction (no counterpart in the reference) ----
 *
 * Stream-ordered barrier over the ranks of one node, as a kernel: every rank stores a rising epoch number into its
 * slot of every peer's flag array (peer_flags: host array of `world` device addresses of unsigned int[world] arrays,
 * NVLink-mapped, zeroed once before the first barrier) and waits until all slots of its own array have reached that
 * epoch. `epoch` is a device word of this rank (zeroed once) that the kernel advances. payload (optional): payload_ints
 * ints that are stored into entry [rank][.] of every peer's payload array (peer_payload: int[world][payload_ints]
 * each) before the flag is raised - the counts exchange of the layer rides on its first barrier. The wait is bounded
 * (2 s unless b200_ep_set_barrier_timeout_ms says otherwise): a rank that never arrives raises status 1
 * (b200_ep_status, which synchronises the device and clears the word) and the kernel returns; nothing hangs.
 * Every rank must issue the same sequence of barriers, and the ranks must be synchronised on the host once after
 * the flag arrays were zeroed.
 */
int b200_ep_barrier(const unsigned long long *peer_flags, int world, int rank, unsigned int *epoch, const int *payload,
                    int payload_ints, const unsigned long long *peer_payload, void *stream);
int b200_ep_set_barrier_timeout_ms(int ms);
int b200_ep_status(int *status_out);

/*
 * Exchange plan of one rank from the gathered counts (int[world][num_experts]: row s = per-expert row counts of rank
 * s's tokens, global expert ids), in one launch: local_counts / local_cumsum [experts_per_rank] = rows this rank
 * receives per local expert and their inclusive prefix sums, clipped to capacity_rows; dst_base[num_experts] as the
 * b200_ep_* kernels take it; overflow[0] is set to 1 (never cleared) when the unclipped total exceeds the capacity.
 */
int b200_ep_plan(const int *gathered_counts, int world, int rank, int experts_per_rank, int64_t capacity_rows,
                 int *local_counts, int *local_cumsum, int *dst_base, int *overflow, void *stream);

/* dWr[i] = bf16(f32(dWr[i]) + sum over ranks, in rank order, of partial_r[i]); peer_partials: host array of `world`
 * device addresses of bf16 arrays of num_elements (a multiple of 8) elements; call it after a barrier. */
int b200_ep_reduce_router_grad(const unsigned long long *peer_partials, int world, int64_t num_elements, void *dWr,
                               void *stream);

/*
 * One rank's share of the expert-parallel layer. Rank g of `world` owns experts [g*E/world, (g+1)*E/world) with
 * their W1 / W3 / W2 (and gradients); tokens are data-parallel (total_tokens per rank); Wr is replicated. The peer_*
 * members are HOST arrays of `world` device addresses: entry h = the named buffer of rank h as mapped into this
 * process (entry `rank` = this rank's own buffer, which is also given as a plain pointer). Receive-side buffers hold
 * capacity_rows rows (1.5 * T * k is ample for balanced routing); rows that would not fit are dropped and
 * overflow[0] is raised, nothing is overrun. R = total_tokens * top_k.
 */
typedef struct B200EpMoeBlock {
  int world, rank;
  int total_tokens, model_dim, num_experts, top_k, ffn_dim;
  int64_t capacity_rows;
  const void *Wr;               /* [E][d], replicated */
  const void *W1, *W3, *W2;     /* this rank's experts: [E/world][f][d], [E/world][f][d], [E/world][d][f] */
  int64_t w1_stride_elems, w3_stride_elems, w2_stride_elems;
  /* token side (this rank's tokens, all E experts) */
  float *logits;                /* [T][E] */
  float *token_expert_weights;  /* [T][k] */
  uint16_t *chosen_experts;     /* [T][k] */
  int *expert_counts;           /* [E + 1] */
  int *expert_counts_cumsum;    /* [E] */
  int *expert_mapping, *token_mapping; /* [R] each */
  void *mapping_workspace;
  size_t mapping_workspace_bytes;
  void *matmul_workspace;       /* optional */
  size_t matmul_workspace_bytes;
  void *dX_routed;              /* bf16 [T][E] (backward) */
  /* exchange plan */
  int *gathered_counts;         /* int [world][E], this rank's copy of peer_counts */
  int *local_counts, *local_cumsum; /* [E/world] */
  int *dst_base;                /* [E] */
  int *overflow;                /* [1], zeroed by the caller */
  unsigned int *barrier_epoch;  /* [1], zeroed once */
  const unsigned long long *peer_flags;  /* unsigned int [world] per rank, zeroed once */
  const unsigned long long *peer_counts; /* = gathered_counts of every rank */
  /* expert side: rows received from every rank, expert-contiguous */
  void *zone_recv;              /* bf16 [capacity][d] */
  unsigned long long *tags_recv; /* [capacity] */
  void *x1, *x3, *h;            /* bf16 [capacity][f] */
  const unsigned long long *peer_zone, *peer_tags;
  /* home side: expert outputs of this rank's routed pairs, in its own zone order */
  void *Y_home;                 /* bf16 [R][d] */
  const unsigned long long *peer_Y_home;
  /* backward (may be NULL for forward-only use) */
  void *dY_recv;                /* bf16 [capacity][d] */
  float *dP_recv;               /* [capacity] */
  void *dx1, *dx3;              /* bf16 [capacity][f] */
  const float *ones;            /* [capacity] of 1.0f */
  void *dZ_home;                /* bf16 [R][d] */
  void *dWr_partial;            /* bf16 [E][d] */
  const unsigned long long *peer_dY, *peer_dP, *peer_dZ_home, *peer_dWr;
} B200EpMoeBlock;

/*
 * Forward: route locally, counts to every rank on the first barrier, plan, rows and row tags into the owners'
 * buffers (peer stores), barrier, this rank's experts over everything it received with the W2 GEMM's epilogue storing
 * each Y row straight into its home rank's buffer, barrier, local weighted combine onto X_combined. 13 launches, three
 * of them barriers; no host synchronisation, no collective library. Backward mirrors it and ends with the sum of
 * the router weight gradient over the ranks; dXn is overwritten, dWr / dW1 / dW3 / dW2 are accumulated into (dW*
 * cover this rank's experts and may be NULL).
 */
int b200_ep_moe_block_fwd(const B200EpMoeBlock *block, const void *Xn, void *X_combined, void *stream);
int b200_ep_moe_block_bwd(const B200EpMoeBlock *block, const void *Xn, const void *dOut, void *dXn, void *dWr, void *dW1,
                          void *dW3, void *dW2, void *stream);

/*
 * ---- the bandwidth-bound ops of the block around the MoE feed-forward, and of the head ----------------------------
 *
 * bf16 tensors, fp32 arithmetic; any other datatype code returns -1. Argument order and meaning follow the
 * reference's submitters minus the handle (the stream replaces stream_id); every tensor must be 16-byte aligned and
 * n_cols / embed_dim / head_dim multiples of 8. The reference builds its kernels with --use_fast_math
 * (backends/nvidia/src/ops/Makefile:19-21); these use full-precision expf / powf / sincosf / division, so results
 * agree with the reference's to bf16 rounding, not bit for bit.
 */

/* dataflow_submit_default_rms_norm (libdataflowops/include/dataflow_ops.h:151-154; kernel norm/rms_norm.cu:226-340):
 * out = bf16(x * r * w) per row, r = rsqrt(mean(x^2) + eps); r is kept in rms_vals[row] unless rms_vals is NULL. */
int b200_rms_norm(int fwd_dt, int n_rows, int n_cols, float eps, const void *rms_weight, const void *X, void *out,
                  float *rms_vals, void *stream);

/* dataflow_submit_default_rms_norm_recompute (dataflow_ops.h:157-160; norm/rms_norm_recompute.cu:63-133): the same
 * output from the kept rms_vals. */
int b200_rms_norm_recompute(int fwd_dt, int n_rows, int n_cols, const void *rms_weight, const float *rms_vals, const void *X,
                            void *out, void *stream);

/* dataflow_submit_default_rms_norm_bwd_x (dataflow_ops.h:165-169; norm/rms_norm_bwd_x.cu:241-394): ACCUMULATES into dX:
 * dX = bf16(f32(dX) + r * (up * w - (C / n) * x * r)), C = sum over the row of (x r w) * up; X_out, when not NULL,
 * receives the recomputed forward output. n_cols up to 8192. eps is unused (as in the reference). */
int b200_rms_norm_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float *fwd_rms_vals,
                        const void *rms_weight, const void *X_inp, const void *upstream_dX, void *dX, void *X_out,
                        void *stream);

/* dataflow_submit_default_rms_norm_bwd_w (dataflow_ops.h:172-176; norm/rms_norm_bwd_w.cu:225-325 and
 * rms_norm_bwd_w_combine.cu:200-294): dW[c] = bf16(f32(dW[c]) + sum over rows of up * x * r). Two launches: fp32
 * partial sums of row slices in the workspace, then their sum in slice order (deterministic). The workspace decides
 * how many slices run: b200_rms_norm_bwd_w_workspace_bytes gives the size that fills the GPU (2 slices per SM); a
 * smaller one works with fewer slices, less than one fp32 row of n_cols is an error. */
uint64_t b200_rms_norm_bwd_w_workspace_bytes(int n_rows, int n_cols);
int b200_rms_norm_bwd_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float *fwd_rms_vals,
                        const void *X_inp, const void *upstream_dX, void *dW, uint64_t workspace_bytes, void *workspace,
                        void *stream);

/* dataflow_submit_default_rope / _rope_bwd_x (dataflow_ops.h:195-203; attention_misc/rope.cu:152-256,
 * rope_bwd_x.cu:146-248): in place on the interleaved pairs (2i, 2i+1) of every head of X_q [num_tokens][model_dim]
 * and X_k [num_tokens][num_kv_heads * head_dim] (X_k may be NULL); angle = seq_positions[token] * theta^(-2i/head_dim);
 * the backward applies the inverse rotation. head_dim up to 256. */
int b200_rope(int fwd_dt, int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta, const int *seq_positions,
              void *X_q, void *X_k, void *stream);
int b200_rope_bwd_x(int bwd_dt, int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta,
                    const int *seq_positions, void *dX_q, void *dX_k, void *stream);

/* dataflow_submit_default_softmax (dataflow_ops.h:298-301; loss_misc/softmax.cu:249-394): row-wise softmax,
 * out = bf16(exp(x - max) / sum); X and out may be the same buffer. */
int b200_softmax(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void *X, void *out, void *stream);

/* dataflow_submit_default_cross_entropy_loss (dataflow_ops.h:303-306; loss_misc/cross_entropy.cu:48-68): pred_logits
 * holds the softmax OUTPUT; loss_vec[row] = -log(p[row][label]) and p[row][label] -= 1 in place, which leaves the
 * gradient of the summed loss with respect to the logits in the buffer. loss_vec has n_rows + 1 entries. */
int b200_cross_entropy_loss(int bwd_dt, int n_rows, int n_cols, void *pred_logits, const uint32_t *labels, float *loss_vec,
                            void *stream);

/* dataflow_submit_default_set_average_loss (dataflow_ops.h:308; cross_entropy.cu:70-119):
 * loss_vec[n_tokens] = mean(loss_vec[0 .. n_tokens)). */
int b200_set_average_loss(int n_tokens, float *loss_vec, void *stream);

/* dataflow_submit_default_adamw_step (dataflow_ops.h:310-315; optimizer/adamw_step.cu:6-65): m = b1 m + (1-b1) g;
 * v = b2 v + (1-b2) g^2; p -= lr * ((m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps) + wd * p); all four tensors bf16,
 * updated in place with one rounding each; step_num counts from 1. */
int b200_adamw_step(int param_dt, int grad_dt, int mean_dt, int var_dt, uint64_t num_els, int step_num, float lr, float beta1,
                    float beta2, float weight_decay, float epsilon, void *param, const void *grad, void *mean, void *var,
                    void *stream);

/* dataflow_submit_default_embedding_table / _bwd_w (dataflow_ops.h:136-146; preprocess/embedding_table.cu:81-116,
 * embedding_table_bwd_w.cu:99-145): the batch's token ids sorted (sorted_token_ids), the position each came from
 * (sorted_token_mapping), and for unique token u the range [start[u], start[u+1]) of sorted positions holding it.
 * Forward: output[position] = table[id]. Backward: the gradient rows of a token are summed in bf16 in sorted order
 * (one rounding per addition, as the reference does) and added to grad_embedding_table[id]. */
int b200_embedding_table(int fwd_dt, int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                         const uint32_t *sorted_token_mapping, const uint32_t *unique_token_sorted_inds_start,
                         const void *embedding_table, void *output, void *stream);
int b200_embedding_table_bwd_w(int bwd_dt, int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                               const uint32_t *sorted_token_mapping, const uint32_t *unique_token_sorted_inds_start,
                               const void *grad_stream, void *grad_embedding_table, void *stream);

/*
 * ---- attention ------------------------------------------------------------------------------------------------
 *
 * dataflow_submit_attention / dataflow_submit_attention_bwd (libdataflowops/include/dataflow_ops.h:70-105), which the
 * reference forwards to an external flash-attention library (backends/nvidia/src/ops/src/external/attention_helper):
 * softmax(Q K^T / sqrt(head_dim)) V per sequence and head over packed variable-length sequences, grouped query heads
 * (query head h reads key / value head h / (num_q_heads / num_kv_heads)), optionally causal with the last query of a
 * sequence aligned to its last key. x_q, x_attn_out, dx_out, dx_q: [total_q][num_q_heads * head_dim]; x_k, x_v, dx_k,
 * dx_v: [total_k][num_kv_heads * head_dim]; softmax_lse: fp32 [num_q_heads][total_q] (log-sum-exp of the scaled
 * scores, written by the forward, read by the backward). bf16 only.
 *
 * Differences from the reference's signature: the sequence offsets and lengths are HOST arrays here (the fused kernels
 * take them as a launch parameter, 48 sequences per launch; the GEMM-by-GEMM form loops over them on the host);
 * dx_q / dx_k / dx_v are overwritten.
 *
 * head_dim 64 and 128 run fused tcgen05 kernels (csrc/attention_sm100.cu): the forward for both (scores in tensor
 * memory, probabilities through shared memory, no workspace), the backward for 128 (dK, dV accumulated in tensor
 * memory per block of 128 keys, dQ added into an fp32 accumulator in the workspace with red.add and rounded once -
 * the order of those additions is not fixed, so dQ may differ in the last bit between runs). Every other head size,
 * and the backward at 64, runs this library's tensor-core GEMMs on head slices with the score matrix of one
 * (sequence, head, 4096-row chunk) in the workspace. The arithmetic of both forms (fp32 scores and statistics,
 * probabilities rounded to bf16 before they multiply V or dO, fp32 accumulation, one rounding per output,
 * probabilities re-formed from the log-sum-exp in the backward) is that of the published algorithm.
 *
 * b200_attention_workspace_bytes mirrors dataflow_get_attention_workspace_size (dataflow_ops.h:93-97): the bytes a
 * forward (is_training = 0) or a forward and backward (1) need for batches of at most max_total_q packed query rows
 * and sequences of at most max_seqlen_q / max_seqlen_k. It may be 0 (fused forward); the calls then ignore the
 * workspace arguments.
 */
uint64_t b200_attention_workspace_bytes(int is_training, int num_q_heads, int num_kv_heads, int head_dim, int max_total_q,
                                        int max_seqlen_q, int max_seqlen_k);

int b200_attention_fwd(int fwd_dt, int num_seqs, int total_q, int total_k, const int *q_seq_offsets, const int *q_seq_lens,
                       int max_seqlen_q, const int *k_seq_offsets, const int *k_seq_lens, int max_seqlen_k, int num_q_heads,
                       int num_kv_heads, int head_dim, const void *x_q, const void *x_k, const void *x_v, void *x_attn_out,
                       float *softmax_lse, int is_causal, uint64_t workspaceBytes, void *workspace, void *stream);

int b200_attention_bwd(int bwd_dt, int num_seqs, int total_q, int total_k, const int *q_seq_offsets, const int *q_seq_lens,
                       int max_seqlen_q, const int *k_seq_offsets, const int *k_seq_lens, int max_seqlen_k, int num_q_heads,
                       int num_kv_heads, int head_dim, const void *x_q, const void *x_k, const void *x_v,
                       const void *x_attn_out, const float *softmax_lse, const void *dx_out, void *dx_q, void *dx_k,
                       void *dx_v, int is_causal, uint64_t workspaceBytes, void *workspace, void *stream);

/* The fused attention kernels (head_dim 64 and 128) bound every wait on a barrier to two seconds; one that runs out
 * records a code (21-26: which hand-over gave up) and the launch ends early with wrong results. Synchronises the device,
 * returns the recorded code through status_out (0 = none) and clears it. No counterpart in the reference. */
int b200_attention_status(int *status_out);

/*
 * ---- a whole decoder block ---------------------------------------------------------------------------------------
 *
 * RMSNorm -> q / k / v projections -> RoPE -> causal attention -> output projection + residual -> RMSNorm -> MoE
 * feed-forward + residual: what dataflow_submit_transformer_moe_block (dataflow_transformer.c:2588-2986) issues op by
 * op, and its backward (_bwd_x 3386-3719, _bwd_w 4060-4185), as one call each. All buffers are the caller's; the
 * sequence description (offsets, lengths) is a HOST array as for b200_attention_fwd; positions is a device array of the
 * tokens' positions in their sequences. Saved by the forward for the backward: rms1, q, k (after RoPE), v, attn, lse,
 * x_mid, rms2, xn2 and what the MoE part keeps (B200MoeBlock). xn is scratch in both directions.
 */
typedef struct B200TransformerBlock {
  int total_tokens, model_dim, num_q_heads, num_kv_heads, head_dim, theta;
  float eps;
  int num_seqs, max_seqlen;
  const int *seq_offsets, *seq_lens; /* HOST [num_seqs] */
  const int *positions;              /* device [T] */
  /* bf16 weights: attn_norm, ffn_norm [d]; wq [Hq*hd][d]; wk, wv [Hkv*hd][d]; wo [d][Hq*hd] */
  const void *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm;
  float *rms1, *rms2;                /* [T] */
  void *q, *k, *v, *attn;            /* bf16 [T][Hq*hd], [T][Hkv*hd] x 2, [T][Hq*hd] */
  float *lse;                        /* [Hq][T] */
  void *x_mid, *xn2, *xn;            /* bf16 [T][d] */
  void *attn_workspace;              /* b200_attention_workspace_bytes(is_training = 1, ...) */
  uint64_t attn_workspace_bytes;
  B200MoeBlock moe;                  /* the feed-forward part; its Xn is xn2 */
} B200TransformerBlock;

/* gradients the backward accumulates into (bf16, the shapes of the weights); with overwrite != 0 it writes them
 * instead and never reads their old contents (first micro-batch of a step: no zeroing pass is needed) */
typedef struct B200TransformerBlockGrads {
  void *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *router, *W1, *W3, *W2;
  int overwrite;
} B200TransformerBlockGrads;

/* backward scratch, shared by every block of a model */
typedef struct B200TransformerBlockScratch {
  void *dxn, *dattn, *dq, *dk, *dv; /* bf16 [T][d], [T][Hq*hd], [T][Hq*hd], [T][Hkv*hd] x 2 */
  void *norm_workspace;             /* b200_rms_norm_bwd_w_workspace_bytes(T, d) */
  uint64_t norm_workspace_bytes;
} B200TransformerBlockScratch;

/* out [T][d] = block(x); x and out are two buffers (x is read again by the backward). */
int b200_transformer_block_fwd(const B200TransformerBlock *block, const void *x, void *out, void *stream);

/* dx [T][d] holds the gradient at the block's output on entry and at its input on return; the weight gradients are
 * accumulated into (beta = 1), as by the reference's gradient GEMMs and norm kernels, unless grads->overwrite is set. */
int b200_transformer_block_bwd(const B200TransformerBlock *block, const void *x, void *dx, const B200TransformerBlockGrads *grads,
                               const B200TransformerBlockScratch *scratch, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MOE_H */
