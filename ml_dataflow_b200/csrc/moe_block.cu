// Host-side driver of one MoE feed-forward, forward and backward, on the entry points of this library: the op
// sequence a C caller (the reference's transformer block) issues, without its mid-layer host synchronisation and
// without its per-expert loop. Nothing here launches a kernel of its own or allocates; every buffer is the caller's.
//
// Reference sequence that this stands in for (libdataflowmodels/src/transformer/src/dataflow_transformer.c):
//   forward     dataflow_submit_transformer_moe_block         2710-2974 (router GEMM ... merge_experts)
//   backward-x  dataflow_submit_transformer_moe_block_bwd_x   3399-3719
//   backward-w  dataflow_submit_transformer_moe_block_bwd_w   4062-4185
#include "common.cuh"
#include "../../include/b200_moe.h"

static int check_block(const char *op, const B200MoeBlock *b) {
  B200_REQUIRE(b != nullptr, "%s: null block description", op);
  B200_REQUIRE(b->total_tokens >= 0 && b->model_dim > 0 && b->num_experts >= 1 && b->top_k >= 1 &&
                   b->top_k <= b->num_experts && b->ffn_dim > 0,
               "%s: bad shape (T %d, d %d, E %d, k %d, f %d)", op, b->total_tokens, b->model_dim, b->num_experts,
               b->top_k, b->ffn_dim);
  B200_REQUIRE(b->Wr && b->W1 && b->W3 && b->W2, "%s: weight pointer missing", op);
  B200_REQUIRE(b->logits && b->token_expert_weights && b->chosen_experts && b->expert_counts &&
                   b->expert_counts_cumsum && b->expert_mapping && b->token_mapping && b->mapping_workspace,
               "%s: routing buffer missing", op);
  B200_REQUIRE(b->zone && b->x1 && b->x3 && b->h && b->Y, "%s: activation buffer missing", op);
  return 0;
}

extern "C" int b200_moe_block_fwd(const B200MoeBlock *b, const void *Xn, void *X_combined, void *stream) {
  if (check_block("moe_block_fwd", b)) return -1;
  B200_REQUIRE(Xn && X_combined, "moe_block_fwd: Xn / X_combined missing");
  const int T = b->total_tokens, d = b->model_dim, E = b->num_experts, k = b->top_k, f = b->ffn_dim;
  if (T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  // router logits, fp32: logits[T][E] = Xn . Wr^T (reference call: transa = 1, M = E, K = d, N = T)
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_NONE, B200_DT_FP32, 1, 0, E, d, T, 1.0f, 0.0f, b->Wr, Xn, nullptr,
                  b->logits, b->matmul_workspace_bytes, b->matmul_workspace, stream))
    return -1;
  // the reference's caller zeroes the counters before select_experts (2737-2747)
  B200_CUDA(cudaMemsetAsync(b->expert_counts, 0, sizeof(int) * (size_t)(E + 1), s));
  B200_CUDA(cudaMemsetAsync(b->expert_counts_cumsum, 0, sizeof(int) * (size_t)E, s));
  if (b200_select_experts(B200_DT_FP32, T, E, k, b->logits, b->token_expert_weights, b->chosen_experts,
                          b->expert_counts, b->expert_counts_cumsum, b->host_expert_counts, stream))
    return -1;
  if (b200_build_expert_mapping(T, E, k, b->chosen_experts, b->expert_counts_cumsum, b->expert_mapping,
                                b->token_mapping, b->mapping_workspace, b->mapping_workspace_bytes, stream))
    return -1;
  if (b200_prepare_experts(T, d, k, Xn, b->token_mapping, b->zone, stream)) return -1;
  // all experts in two launches; the per-expert row counts are read on the device, so no host sync (2789) is needed
  if (b200_moe_experts_fwd(T * k, d, f, E, b->zone, b->W1, b->W3, b->W2, b->w1_stride_elems, b->w3_stride_elems,
                           b->w2_stride_elems, b->expert_counts, b->expert_counts_cumsum, b->x1, b->x3, b->h, b->Y,
                           stream))
    return -1;
  return b200_merge_experts(T, d, k, b->Y, b->token_mapping, b->token_expert_weights, X_combined, stream);
}

extern "C" int b200_moe_block_recompute(const B200MoeBlock *b, const void *Xn, int recompute_x1_x3, void *stream) {
  if (check_block("moe_block_recompute", b)) return -1;
  B200_REQUIRE(Xn, "moe_block_recompute: Xn missing");
  const int T = b->total_tokens, d = b->model_dim, E = b->num_experts, k = b->top_k, f = b->ffn_dim;
  if (T == 0) return 0;
  // the routing tables are small and always kept; the zone is re-gathered as the reference does (3202)
  if (b200_prepare_experts(T, d, k, Xn, b->token_mapping, b->zone, stream)) return -1;
  if (recompute_x1_x3)  // x1, x3 and h again from the zone (3252-3273), all experts in one launch, no W2 product
    return b200_moe_experts_fwd(T * k, d, f, E, b->zone, b->W1, b->W3, nullptr, b->w1_stride_elems, b->w3_stride_elems,
                                b->w2_stride_elems, b->expert_counts, b->expert_counts_cumsum, b->x1, b->x3, b->h,
                                nullptr, stream);
  return b200_swiglu(T * k, f, b->x1, b->x3, b->h, stream);  // x1, x3 were saved: only h is re-formed
}

extern "C" int b200_moe_block_bwd(const B200MoeBlock *b, const void *Xn, const void *dOut, void *dXn, void *dWr,
                                  void *dW1, void *dW3, void *dW2, void *stream) {
  if (check_block("moe_block_bwd", b)) return -1;
  B200_REQUIRE(Xn && dOut && dXn && dWr, "moe_block_bwd: Xn / dOut / dXn / dWr missing");
  B200_REQUIRE(b->dY_zone && b->row_weights && b->dP && b->dx1 && b->dx3 && b->dZ && b->dX_routed,
               "moe_block_bwd: backward workspace missing");
  const int T = b->total_tokens, d = b->model_dim, E = b->num_experts, k = b->top_k, f = b->ffn_dim;
  if (T == 0) return 0;
  const int R = T * k;
  cudaStream_t s = (cudaStream_t)stream;
  // dY rows = w * dOut in expert order: the rewrite router_bwd_x performs on the zone (router_bwd_x.cu:83-90)
  if (b200_prepare_experts_weighted(T, d, k, dOut, b->token_mapping, b->token_expert_weights, b->dY_zone, stream))
    return -1;
  if (b200_scatter_row_weights(T, k, b->token_mapping, b->token_expert_weights, b->row_weights, stream)) return -1;
  B200_CUDA(cudaMemsetAsync(b->dP, 0, sizeof(float) * (size_t)R, s));
  // W2 dgrad + SwiGLU' + router dot product, then dZ = dx1 W1 + dx3 W3; no recompute of the W2 forward (3494-3516)
  if (b200_moe_experts_bwd_x(R, d, f, E, b->dY_zone, b->row_weights, b->x1, b->x3, b->W1, b->W3, b->W2,
                             b->w1_stride_elems, b->w3_stride_elems, b->w2_stride_elems, b->expert_counts,
                             b->expert_counts_cumsum, b->dx1, b->dx3, nullptr, b->dP, b->dZ, stream))
    return -1;
  // the three weight gradients (h and the gathered zone are still resident from the forward)
  if (dW1 || dW3 || dW2) {
    if (b200_moe_experts_bwd_w(R, d, f, E, b->dY_zone, b->h, b->zone, b->dx1, b->dx3, dW1, dW3, dW2,
                               b->w1_stride_elems, b->w3_stride_elems, b->w2_stride_elems, b->expert_counts,
                               b->expert_counts_cumsum, stream))
      return -1;
  }
  // un-permute into a zeroed dXn (3666-3682)
  B200_CUDA(cudaMemsetAsync(dXn, 0, 2 * (size_t)T * d, s));
  if (b200_merge_experts(T, d, k, b->dZ, b->token_mapping, nullptr, dXn, stream)) return -1;
  // router: dP -> [T][E] on the chosen columns, gate Jacobian, then the two router GEMMs (3707-3719, 4174-4185)
  B200_CUDA(cudaMemsetAsync(b->dX_routed, 0, 2 * (size_t)T * E, s));
  if (b200_gather_router_grad(T, E, k, b->token_mapping, b->chosen_experts, b->dP, b->dX_routed, stream)) return -1;
  if (b200_router_gate_bwd_x(T, E, k, b->chosen_experts, b->token_expert_weights, b->dX_routed, stream))
    return -1;
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, 0, 0, d, E, T, 1.0f, 1.0f, b->Wr,
                  b->dX_routed, dXn, dXn, 0, nullptr, stream))
    return -1;
  return b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, 0, 1, d, T, E, 1.0f, 1.0f, Xn,
                     b->dX_routed, dWr, dWr, b->matmul_workspace_bytes, b->matmul_workspace, stream);
}
