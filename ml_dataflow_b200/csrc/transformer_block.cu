// A whole decoder block from C: RMSNorm -> q / k / v projections -> RoPE -> attention -> output projection + residual
// -> RMSNorm -> MoE feed-forward + residual, forward and backward, as one call each over a struct of caller-owned
// buffers. It stands where the reference's block drivers stand (dataflow_submit_transformer_moe_block,
// libdataflowmodels/src/transformer/src/dataflow_transformer.c:2588-2986; _bwd_x 3386-3719; _bwd_w 4060-4185) and issues
// the same ops in the same order, each through this library's entry point for it; nothing is allocated and nothing
// waits for the device.
#include "common.cuh"
#include "../../include/b200_moe.h"

namespace {

const int BF = B200_DT_BF16;

// out[T][o] = x[T][i] . w[o][i]^T (+ residual): the column-major call the reference makes for a linear layer
int linear(int T, int i, int o, const void *x, const void *w, const void *residual, void *out, void *stream) {
  return b200_matmul(BF, BF, residual ? BF : B200_DT_NONE, BF, 1, 0, o, i, T, 1.0f, residual ? 1.0f : 0.0f, w, x, residual,
                     out, 0, nullptr, stream);
}
// dx[T][i] (+)= dy[T][o] . w[o][i]
int linear_dx(int T, int i, int o, const void *dy, const void *w, void *dx, bool accumulate, void *stream) {
  return b200_matmul(BF, BF, accumulate ? BF : B200_DT_NONE, BF, 0, 0, i, o, T, 1.0f, accumulate ? 1.0f : 0.0f, w, dy,
                     accumulate ? dx : nullptr, dx, 0, nullptr, stream);
}
// dw[o][i] (+)= dy[T][o]^T . x[T][i]
int linear_dw(int T, int i, int o, const void *dy, const void *x, void *dw, bool accumulate, void *stream) {
  return b200_matmul(BF, BF, accumulate ? BF : B200_DT_NONE, BF, 0, 1, i, T, o, 1.0f, accumulate ? 1.0f : 0.0f, x, dy,
                     accumulate ? dw : nullptr, dw, 0, nullptr, stream);
}

int check_block(const char *op, const B200TransformerBlock *b) {
  B200_REQUIRE(b != nullptr, "%s: null block", op);
  B200_REQUIRE(b->total_tokens > 0 && b->model_dim > 0 && b->head_dim > 0 && b->num_q_heads > 0 && b->num_kv_heads > 0 &&
                   b->num_q_heads % b->num_kv_heads == 0,
               "%s: bad dimensions", op);
  B200_REQUIRE(b->num_seqs > 0 && b->seq_offsets && b->seq_lens && b->positions, "%s: the packed sequences are not described", op);
  B200_REQUIRE(b->attn_norm && b->wq && b->wk && b->wv && b->wo && b->ffn_norm, "%s: null weight", op);
  B200_REQUIRE(b->rms1 && b->q && b->k && b->v && b->attn && b->lse && b->x_mid && b->rms2 && b->xn2 && b->xn,
               "%s: null activation buffer", op);
  B200_REQUIRE(b->moe.total_tokens == b->total_tokens && b->moe.model_dim == b->model_dim,
               "%s: the MoE part is sized for %d x %d, the block for %d x %d", op, b->moe.total_tokens, b->moe.model_dim,
               b->total_tokens, b->model_dim);
  return 0;
}

}  // namespace

extern "C" int b200_transformer_block_fwd(const B200TransformerBlock *b, const void *x, void *out, void *stream) {
  if (check_block("transformer_block_fwd", b)) return -1;
  B200_REQUIRE(x && out && x != out, "transformer_block_fwd: x and out must be two buffers");
  const int T = b->total_tokens, d = b->model_dim, Dq = b->num_q_heads * b->head_dim, Dk = b->num_kv_heads * b->head_dim;
  if (b200_rms_norm(BF, T, d, b->eps, b->attn_norm, x, b->xn, b->rms1, stream)) return -1;
  if (linear(T, d, Dq, b->xn, b->wq, nullptr, b->q, stream)) return -1;
  if (linear(T, d, Dk, b->xn, b->wk, nullptr, b->k, stream)) return -1;
  if (linear(T, d, Dk, b->xn, b->wv, nullptr, b->v, stream)) return -1;
  if (b200_rope(BF, T, Dq, b->head_dim, b->num_kv_heads, b->theta, b->positions, b->q, b->k, stream)) return -1;
  if (b200_attention_fwd(BF, b->num_seqs, T, T, b->seq_offsets, b->seq_lens, b->max_seqlen, b->seq_offsets, b->seq_lens,
                         b->max_seqlen, b->num_q_heads, b->num_kv_heads, b->head_dim, b->q, b->k, b->v, b->attn, b->lse, 1,
                         b->attn_workspace_bytes, b->attn_workspace, stream))
    return -1;
  if (linear(T, Dq, d, b->attn, b->wo, x, b->x_mid, stream)) return -1;
  if (b200_rms_norm(BF, T, d, b->eps, b->ffn_norm, b->x_mid, b->xn2, b->rms2, stream)) return -1;
  // the MoE combine accumulates onto the residual
  B200_CUDA(cudaMemcpyAsync(out, b->x_mid, (size_t)T * d * 2, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return b200_moe_block_fwd(&b->moe, b->xn2, out, stream);
}

extern "C" int b200_transformer_block_bwd(const B200TransformerBlock *b, const void *x, void *dx, const B200TransformerBlockGrads *g,
                                          const B200TransformerBlockScratch *s, void *stream) {
  if (check_block("transformer_block_bwd", b)) return -1;
  B200_REQUIRE(x && dx && g && s, "transformer_block_bwd: null argument");
  B200_REQUIRE(g->attn_norm && g->wq && g->wk && g->wv && g->wo && g->ffn_norm && g->router && g->W1 && g->W3 && g->W2,
               "transformer_block_bwd: null gradient buffer");
  B200_REQUIRE(s->dxn && s->dattn && s->dq && s->dk && s->dv && s->norm_workspace, "transformer_block_bwd: null scratch buffer");
  const int T = b->total_tokens, d = b->model_dim, Dq = b->num_q_heads * b->head_dim, Dk = b->num_kv_heads * b->head_dim;
  const bool acc = g->overwrite == 0;
  if (!acc) {  // the norm-weight kernels only accumulate: start them from zero
    B200_CUDA(cudaMemsetAsync(g->attn_norm, 0, (size_t)d * 2, (cudaStream_t)stream));
    B200_CUDA(cudaMemsetAsync(g->ffn_norm, 0, (size_t)d * 2, (cudaStream_t)stream));
  }
  // MoE part: dx is the gradient at the block's output and also flows through the residual unchanged
  if ((acc ? b200_moe_block_bwd : b200_moe_block_bwd_overwrite)(&b->moe, b->xn2, dx, s->dxn, g->router, g->W1, g->W3, g->W2,
                                                                 stream))
    return -1;
  if (b200_rms_norm_bwd_w(BF, BF, T, d, b->eps, b->rms2, b->x_mid, s->dxn, g->ffn_norm, s->norm_workspace_bytes,
                          s->norm_workspace, stream))
    return -1;
  if (b200_rms_norm_bwd_x(BF, BF, T, d, b->eps, b->rms2, b->ffn_norm, b->x_mid, s->dxn, dx, nullptr, stream)) return -1;
  // attention part: x_mid = x + attn . wo^T
  if (linear_dw(T, Dq, d, dx, b->attn, g->wo, acc, stream)) return -1;
  if (linear_dx(T, Dq, d, dx, b->wo, s->dattn, false, stream)) return -1;
  if (b200_attention_bwd(BF, b->num_seqs, T, T, b->seq_offsets, b->seq_lens, b->max_seqlen, b->seq_offsets, b->seq_lens,
                         b->max_seqlen, b->num_q_heads, b->num_kv_heads, b->head_dim, b->q, b->k, b->v, b->attn, b->lse,
                         s->dattn, s->dq, s->dk, s->dv, 1, b->attn_workspace_bytes, b->attn_workspace, stream))
    return -1;
  if (b200_rope_bwd_x(BF, T, Dq, b->head_dim, b->num_kv_heads, b->theta, b->positions, s->dq, s->dk, stream)) return -1;
  if (b200_rms_norm_recompute(BF, T, d, b->attn_norm, b->rms1, x, b->xn, stream)) return -1;
  if (linear_dw(T, d, Dq, s->dq, b->xn, g->wq, acc, stream)) return -1;
  if (linear_dw(T, d, Dk, s->dk, b->xn, g->wk, acc, stream)) return -1;
  if (linear_dw(T, d, Dk, s->dv, b->xn, g->wv, acc, stream)) return -1;
  if (linear_dx(T, d, Dq, s->dq, b->wq, s->dxn, false, stream)) return -1;
  if (linear_dx(T, d, Dk, s->dk, b->wk, s->dxn, true, stream)) return -1;
  if (linear_dx(T, d, Dk, s->dv, b->wv, s->dxn, true, stream)) return -1;
  if (b200_rms_norm_bwd_w(BF, BF, T, d, b->eps, b->rms1, x, s->dxn, g->attn_norm, s->norm_workspace_bytes, s->norm_workspace,
                          stream))
    return -1;
  return b200_rms_norm_bwd_x(BF, BF, T, d, b->eps, b->rms1, b->attn_norm, x, s->dxn, dx, nullptr, stream);
}
