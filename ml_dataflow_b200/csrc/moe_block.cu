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

// accumulate: the weight gradients are added to (the reference's beta = 1); otherwise they are written, and the old
// contents of the gradient buffers are not read
static int moe_block_bwd(const B200MoeBlock *b, const void *Xn, const void *dOut, void *dXn, void *dWr, void *dW1,
                         void *dW3, void *dW2, bool accumulate, void *stream) {
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
    if ((accumulate ? b200_moe_experts_bwd_w : b200_moe_experts_bwd_w_overwrite)(
            R, d, f, E, b->dY_zone, b->h, b->zone, b->dx1, b->dx3, dW1, dW3, dW2, b->w1_stride_elems, b->w3_stride_elems,
            b->w2_stride_elems, b->expert_counts, b->expert_counts_cumsum, stream))
      return -1;
  }
  // un-permute (3666-3682: merge_experts onto a zeroed dXn there; here one pass that overwrites, same bits)
  if (b200_unpermute_experts(T, d, k, b->dZ, b->token_mapping, dXn, stream)) return -1;
  // router: dP -> [T][E] on the chosen columns, gate Jacobian, then the two router GEMMs (3707-3719, 4174-4185)
  B200_CUDA(cudaMemsetAsync(b->dX_routed, 0, 2 * (size_t)T * E, s));
  if (b200_gather_router_grad(T, E, k, b->token_mapping, b->chosen_experts, b->dP, b->dX_routed, stream)) return -1;
  if (b200_router_gate_bwd_x(T, E, k, b->chosen_experts, b->token_expert_weights, b->dX_routed, stream))
    return -1;
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, 0, 0, d, E, T, 1.0f, 1.0f, b->Wr,
                  b->dX_routed, dXn, dXn, 0, nullptr, stream))
    return -1;
  return b200_matmul(B200_DT_BF16, B200_DT_BF16, accumulate ? B200_DT_BF16 : B200_DT_NONE, B200_DT_BF16, 0, 1, d, T, E, 1.0f,
                     accumulate ? 1.0f : 0.0f, Xn, b->dX_routed, accumulate ? dWr : nullptr, dWr, b->matmul_workspace_bytes,
                     b->matmul_workspace, stream);
}

extern "C" int b200_moe_block_bwd(const B200MoeBlock *b, const void *Xn, const void *dOut, void *dXn, void *dWr,
                                  void *dW1, void *dW3, void *dW2, void *stream) {
  return moe_block_bwd(b, Xn, dOut, dXn, dWr, dW1, dW3, dW2, true, stream);
}

extern "C" int b200_moe_block_bwd_overwrite(const B200MoeBlock *b, const void *Xn, const void *dOut, void *dXn, void *dWr,
                                            void *dW1, void *dW3, void *dW2, void *stream) {
  return moe_block_bwd(b, Xn, dOut, dXn, dWr, dW1, dW3, dW2, false, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Saved-activation contract of the MoE part (libdataflowmodels/include/transformer/seq_batch_structs.h:199-286).
// What the reference keeps per level: the routing results (x_routed, chosen_experts, token_expert_weights,
// expert_counts, expert_counts_cumsum, expert_mapping, token_mapping) at every level that can run a backward - they
// sit before `inp_only_cutoff` in its saved-activations buffer (prep_seq_batch.c:230-283) - and x_1, x_3 only at
// SAVED_ACTIVATION_LEVEL_FULL (prep_seq_batch.c:320-365). The zone and h are workspace at every level. The layout
// below is the reference's: that order, each tensor starting on a 256-byte boundary.
// ---------------------------------------------------------------------------------------------------------------

namespace {

struct SavedPiece {
  void *dev;       // where the tensor lives in the block
  uint64_t bytes;
  uint64_t offset;  // in the saved-activations buffer
};

// fills `pieces` (at most 9) and returns how many; *total = bytes of the buffer
int saved_pieces(const B200MoeBlock *b, int level, SavedPiece *pieces, uint64_t *total) {
  const uint64_t T = (uint64_t)b->total_tokens, E = (uint64_t)b->num_experts, k = (uint64_t)b->top_k,
                 f = (uint64_t)b->ffn_dim;
  const uint64_t R = T * k;
  int n = 0;
  uint64_t at = 0;
  auto add = [&](void *p, uint64_t bytes) {
    at = (at + 255) & ~255ull;
    pieces[n].dev = p;
    pieces[n].bytes = bytes;
    pieces[n].offset = at;
    at += bytes;
    n++;
  };
  add(b->logits, T * E * sizeof(float));
  add(b->chosen_experts, R * sizeof(uint16_t));
  add(b->token_expert_weights, R * sizeof(float));
  add(b->expert_counts, (E + 1) * sizeof(int));
  add(b->expert_counts_cumsum, E * sizeof(int));
  add(b->expert_mapping, R * sizeof(int));
  add(b->token_mapping, R * sizeof(int));
  if (level == B200_SAVED_ACTIVATION_LEVEL_FULL) {
    add(b->x1, R * f * 2);
    add(b->x3, R * f * 2);
  }
  *total = at;
  return n;
}

int check_level(const char *op, int level) {
  B200_REQUIRE(level >= B200_SAVED_ACTIVATION_LEVEL_NONE && level <= B200_SAVED_ACTIVATION_LEVEL_FULL,
               "%s: unknown saved-activation level %d", op, level);
  B200_REQUIRE(level != B200_SAVED_ACTIVATION_LEVEL_NONE, "%s: nothing is saved at level NONE, no backward can follow", op);
  return 0;
}

}  // namespace

extern "C" uint64_t b200_moe_saved_activations_bytes(int total_tokens, int num_experts, int top_k, int ffn_dim,
                                                     int level) {
  if (level <= B200_SAVED_ACTIVATION_LEVEL_NONE || level > B200_SAVED_ACTIVATION_LEVEL_FULL) return 0;
  B200MoeBlock b;
  memset(&b, 0, sizeof(b));
  b.total_tokens = total_tokens;
  b.num_experts = num_experts;
  b.top_k = top_k;
  b.ffn_dim = ffn_dim;
  SavedPiece pieces[9];
  uint64_t total = 0;
  saved_pieces(&b, level, pieces, &total);
  return total;
}

static int copy_saved(const char *op, const B200MoeBlock *b, int level, void *buffer, uint64_t buffer_bytes, bool save,
                      void *stream) {
  if (check_block(op, b) || check_level(op, level)) return -1;
  B200_REQUIRE(buffer != nullptr, "%s: null buffer", op);
  SavedPiece pieces[9];
  uint64_t total = 0;
  const int n = saved_pieces(b, level, pieces, &total);
  B200_REQUIRE(buffer_bytes >= total, "%s: the buffer holds %llu bytes, level %d needs %llu", op,
               (unsigned long long)buffer_bytes, level, (unsigned long long)total);
  unsigned char *base = static_cast<unsigned char *>(buffer);
  for (int i = 0; i < n; i++) {
    if (pieces[i].bytes == 0) continue;
    // the buffer may be device memory or pinned host memory: the copy kind is taken from the pointers
    if (save)
      B200_CUDA(cudaMemcpyAsync(base + pieces[i].offset, pieces[i].dev, pieces[i].bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    else
      B200_CUDA(cudaMemcpyAsync(pieces[i].dev, base + pieces[i].offset, pieces[i].bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  }
  return 0;
}

extern "C" int b200_moe_block_save_activations(const B200MoeBlock *block, int level, void *buffer, uint64_t buffer_bytes,
                                               void *stream) {
  return copy_saved("moe_block_save_activations", block, level, buffer, buffer_bytes, true, stream);
}

extern "C" int b200_moe_block_restore_activations(const B200MoeBlock *block, int level, const void *buffer,
                                                  uint64_t buffer_bytes, void *stream) {
  return copy_saved("moe_block_restore_activations", block, level, const_cast<void *>(buffer), buffer_bytes, false, stream);
}

extern "C" int b200_moe_block_recompute_level(const B200MoeBlock *block, const void *Xn, int level, void *stream) {
  if (check_level("moe_block_recompute_level", level)) return -1;
  // FULL: x1 and x3 were kept, only the zone and h are formed again; below FULL they come back from the zone too
  return b200_moe_block_recompute(block, Xn, level == B200_SAVED_ACTIVATION_LEVEL_FULL ? 0 : 1, stream);
}
