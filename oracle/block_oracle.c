/*
 * CPU oracle for the bandwidth-bound ops around the MoE feed-forward inside a transformer block and its head:
 * RMSNorm (forward, recompute, backward-x, backward-w), RoPE (forward, backward), softmax, cross-entropy, the
 * average loss, AdamW and the embedding table (forward, backward-w), all bf16 with fp32 arithmetic.
 *
 * THIS FILE IS TEST INFRASTRUCTURE, like moe_oracle.c: a plain-C restatement of the reference's CUDA kernels, used
 * only to check the sm_100a kernels. Nothing in the product path links or calls it.
 *
 * Parity status: the reference has no golden vectors for these ops. The restatement is pinned by running the
 * reference's own kernels, compiled from its sources in place (oracle/Makefile, target ref), on the GPU
 * (tests/test_reference_block_kernels_gpu.py). The reference is built with --use_fast_math (backends/nvidia/src/
 * ops/Makefile:19-21): its expf / powf / sincosf / division are the approximate hardware forms; this file uses libm,
 * so the pin is to tolerance, with the reference's fast-math error stated in the test.
 *
 * "norm/", "attention_misc/", "loss_misc/", "optimizer/", "preprocess/" stand for the directories of those names
 * under backends/nvidia/src/ops/src/native/src/ of the reference. bf16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float b2f(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f2b(float f) { /* round to nearest even, as __float2bfloat16_rn */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* ---- RMSNorm ------------------------------------------------------------------------------------------------- */

/* norm/rms_norm.cu:226-340: r = rsqrt(sum(x^2) / n + eps) kept in rms_vals[row] (may be NULL);
 * out = bf16(x * r * w), the products formed left to right in fp32. */
void orc_rms_norm_bf16(int n_rows, int n_cols, float eps, const uint16_t *w, const uint16_t *X, uint16_t *out,
                       float *rms_vals) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_rows; r++) {
    const uint16_t *x = X + (size_t)r * n_cols;
    double ssd = 0.0; /* order-free value of the sum the reference forms as a tree of fp32 partial sums */
    for (int c = 0; c < n_cols; c++) ssd += (double)(b2f(x[c]) * b2f(x[c]));
    const float ss = (float)ssd, inv_n = 1.0f / (float)n_cols;
    const float rv = 1.0f / sqrtf(ss * inv_n + eps);
    if (rms_vals) rms_vals[r] = rv;
    for (int c = 0; c < n_cols; c++) out[(size_t)r * n_cols + c] = f2b(b2f(x[c]) * rv * b2f(w[c]));
  }
}

/* norm/rms_norm_recompute.cu:63-133: the same output from kept rms_vals. */
void orc_rms_norm_recompute_bf16(int n_rows, int n_cols, const uint16_t *w, const float *rms_vals, const uint16_t *X,
                                 uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_rows; r++)
    for (int c = 0; c < n_cols; c++)
      out[(size_t)r * n_cols + c] = f2b((b2f(X[(size_t)r * n_cols + c]) * rms_vals[r]) * b2f(w[c]));
}

/* norm/rms_norm_bwd_x.cu:241-394: C = sum_c (x*r*w) * up (the unrounded fp32 output times the upstream gradient);
 * dX[c] = bf16(f32(dX[c]) + r * (up*w - (C / n) * (x * r)));  X_out (optional) = bf16(x*r*w). */
void orc_rms_norm_bwd_x_bf16(int n_rows, int n_cols, const float *rms_vals, const uint16_t *w, const uint16_t *X,
                             const uint16_t *up, uint16_t *dX, uint16_t *X_out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_rows; r++) {
    const size_t o = (size_t)r * n_cols;
    const float rv = rms_vals[r];
    double Csum = 0.0;
    for (int c = 0; c < n_cols; c++) {
      const float ov = b2f(X[o + c]) * rv * b2f(w[c]);
      if (X_out) X_out[o + c] = f2b(ov);
      Csum += (double)(ov * b2f(up[o + c]));
    }
    const float c_div_n = (float)Csum / (float)n_cols;
    for (int c = 0; c < n_cols; c++) {
      const float deriv = rv * (b2f(up[o + c]) * b2f(w[c]) - c_div_n * (b2f(X[o + c]) * rv));
      dX[o + c] = f2b(b2f(dX[o + c]) + deriv);
    }
  }
}

/* norm/rms_norm_bwd_w.cu:225-325 and rms_norm_bwd_w_combine.cu:200-294: per column the fp32 sum over rows of
 * up * x * r, added to f32(dW) and rounded once. The reference sums per-block partials; the order here is by row. */
void orc_rms_norm_bwd_w_bf16(int n_rows, int n_cols, const float *rms_vals, const uint16_t *X, const uint16_t *up,
                             uint16_t *dW) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < n_cols; c++) {
    double acc = 0.0; /* order-free reference value of the column sum */
    for (int r = 0; r < n_rows; r++) {
      const size_t o = (size_t)r * n_cols + c;
      acc += (double)(b2f(up[o]) * b2f(X[o]) * rms_vals[r]);
    }
    dW[c] = f2b(b2f(dW[c]) + (float)acc);
  }
}

/* ---- RoPE ---------------------------------------------------------------------------------------------------- */

/* attention_misc/rope.cu:152-256 (sign = +1) and rope_bwd_x.cu:146-248 (sign = -1, the inverse rotation): in place,
 * interleaved pairs (2i, 2i+1) of every head; angle = pos * theta^(-2i / head_dim) in fp32;
 * even' = cos*even - s*sin*odd, odd' = cos*odd + s*sin*even, one rounding each. X_k may be NULL. */
static void rope_rows(int num_tokens, int row_dim, int head_dim, int theta, const int *seq_positions, uint16_t *X,
                      float sign) {
  const int pairs = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < num_tokens; t++) {
    float cs[128], sn[128];
    for (int i = 0; i < pairs; i++) {
      const float inv_freq = powf((float)theta, -(float)(2 * i) / (float)head_dim);
      const float ang = (float)seq_positions[t] * inv_freq;
      cs[i] = cosf(ang);
      sn[i] = sinf(ang);
    }
    uint16_t *row = X + (size_t)t * row_dim;
    for (int c = 0; c < row_dim; c += 2) {
      const int i = (c % head_dim) / 2;
      const float e = b2f(row[c]), o = b2f(row[c + 1]);
      row[c] = f2b(cs[i] * e - sign * sn[i] * o);
      row[c + 1] = f2b(cs[i] * o + sign * sn[i] * e);
    }
  }
}

void orc_rope_bf16(int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta, const int *seq_positions,
                   uint16_t *X_q, uint16_t *X_k) {
  rope_rows(num_tokens, model_dim, head_dim, theta, seq_positions, X_q, 1.0f);
  if (X_k) rope_rows(num_tokens, num_kv_heads * head_dim, head_dim, theta, seq_positions, X_k, 1.0f);
}

void orc_rope_bwd_x_bf16(int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta,
                         const int *seq_positions, uint16_t *dX_q, uint16_t *dX_k) {
  rope_rows(num_tokens, model_dim, head_dim, theta, seq_positions, dX_q, -1.0f);
  if (dX_k) rope_rows(num_tokens, num_kv_heads * head_dim, head_dim, theta, seq_positions, dX_k, -1.0f);
}

/* ---- softmax, cross-entropy, average loss ----------------------------------------------------------------- */

/* loss_misc/softmax.cu:249-394: out = bf16(exp(x - max) / sum exp(x - max)) per row, fp32. The reference folds the
 * maximum and the sum in one online pass; the value is the same up to fp32 rounding. */
void orc_softmax_bf16(int n_rows, int n_cols, const uint16_t *X, uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_rows; r++) {
    const uint16_t *x = X + (size_t)r * n_cols;
    float mx = -3.402823466e38f;
    for (int c = 0; c < n_cols; c++) mx = fmaxf(mx, b2f(x[c]));
    double sumd = 0.0;
    for (int c = 0; c < n_cols; c++) sumd += (double)expf(b2f(x[c]) - mx);
    const float sum = (float)sumd;
    for (int c = 0; c < n_cols; c++) out[(size_t)r * n_cols + c] = f2b(expf(b2f(x[c]) - mx) / sum);
  }
}

/* loss_misc/cross_entropy.cu:48-68: on softmax OUTPUT p (named pred_logits there): loss_vec[row] = -log(p[label]),
 * then p[label] = bf16(f32(p[label]) - 1) in place, which leaves dLoss/dlogits in the buffer. */
void orc_cross_entropy_loss_bf16(int n_rows, int n_cols, uint16_t *p, const uint32_t *labels, float *loss_vec) {
  for (int r = 0; r < n_rows; r++) {
    uint16_t *e = p + (size_t)r * n_cols + labels[r];
    loss_vec[r] = -1.0f * logf(b2f(*e));
    *e = f2b(b2f(*e) - 1.0f);
  }
}

/* loss_misc/cross_entropy.cu:70-119: loss_vec[num_tokens] = mean of loss_vec[0 .. num_tokens). */
void orc_set_average_loss(int num_tokens, float *loss_vec) {
  double s = 0.0;
  for (int i = 0; i < num_tokens; i++) s += (double)loss_vec[i];
  loss_vec[num_tokens] = (float)(s / (double)num_tokens);
}

/* ---- AdamW --------------------------------------------------------------------------------------------------- */

/* optimizer/adamw_step.cu:6-65 (bf16 param / grad / mean / var, fp32 arithmetic, step_num counts from 1). */
void orc_adamw_step_bf16(uint64_t num_els, int step_num, float lr, float beta1, float beta2, float weight_decay,
                         float epsilon, uint16_t *param, const uint16_t *grad, uint16_t *mean, uint16_t *var) {
  const float c1 = 1.0f - powf(beta1, (float)step_num), c2 = 1.0f - powf(beta2, (float)step_num);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)num_els; i++) {
    const float p = b2f(param[i]), g = b2f(grad[i]);
    const float m_t = beta1 * b2f(mean[i]) + (1.0f - beta1) * g;
    const float v_t = beta2 * b2f(var[i]) + (1.0f - beta2) * g * g;
    const float m_hat = m_t / c1, v_hat = v_t / c2;
    param[i] = f2b(p - lr * (m_hat / (sqrtf(v_hat) + epsilon) + weight_decay * p));
    mean[i] = f2b(m_t);
    var[i] = f2b(v_t);
  }
}

/* ---- embedding table ---------------------------------------------------------------------------------------- */

/* preprocess/embedding_table.cu:81-116: tokens are given sorted by id; unique token u covers sorted positions
 * [starts[u], starts[u+1]); every such position i writes table[id] to output row sorted_token_mapping[i]. */
void orc_embedding_table_bf16(int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                              const uint32_t *sorted_token_mapping, const uint32_t *starts, const uint16_t *table,
                              uint16_t *output) {
  for (int u = 0; u < num_unique_tokens; u++) {
    const uint32_t id = sorted_token_ids[starts[u]];
    for (uint32_t i = starts[u]; i < starts[u + 1]; i++)
      memcpy(output + (size_t)sorted_token_mapping[i] * embed_dim, table + (size_t)id * embed_dim, 2 * (size_t)embed_dim);
  }
}

/* preprocess/embedding_table_bwd_w.cu:99-145: per unique token the gradient rows are added up IN BF16, in sorted
 * order, starting from zero (one rounding per addition), and the sum is added to the table row in bf16. */
void orc_embedding_table_bwd_w_bf16(int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                                    const uint32_t *sorted_token_mapping, const uint32_t *starts,
                                    const uint16_t *grad_stream, uint16_t *grad_table) {
  for (int u = 0; u < num_unique_tokens; u++) {
    const uint32_t id = sorted_token_ids[starts[u]];
    for (int c = 0; c < embed_dim; c++) {
      uint16_t agg = 0;
      for (uint32_t i = starts[u]; i < starts[u + 1]; i++)
        agg = f2b(b2f(agg) + b2f(grad_stream[(size_t)sorted_token_mapping[i] * embed_dim + c]));
      uint16_t *g = grad_table + (size_t)id * embed_dim + c;
      *g = f2b(b2f(*g) + b2f(agg));
    }
  }
}

/* ---- attention ------------------------------------------------------------------------------------------------- */

/* The op the reference takes from an external flash-attention library (dataflow_ops.h:70-105; flash-attention 2 / 3,
 * Dao et al.): per sequence and query head, softmax(Q K^T / sqrt(d)) V with fp32 scores and statistics, probabilities
 * rounded to bf16 before they multiply V, fp32 accumulation and one rounding of O; causal = the last query of a
 * sequence sees every key, query i sees keys up to i + (Tk - Tq). Query head h reads key / value head
 * h / (Hq / Hkv). lse[h][total_q] = log-sum-exp of the scaled scores. Parity unpinned: the library is not in the
 * reference tree; this restates the published algorithm (tests check it against float64 softmax attention). */
static int attn_vis(int i, int Tq, int Tk, int causal) {
  if (!causal) return Tk;
  int v = i + 1 + (Tk - Tq);
  return v < 0 ? 0 : (v > Tk ? Tk : v);
}

void orc_attention_fwd_bf16(int num_seqs, int total_q, const int *q_off, const int *q_len, const int *k_off, const int *k_len,
                            int Hq, int Hkv, int hd, const uint16_t *Q, const uint16_t *K, const uint16_t *V, uint16_t *O,
                            float *lse, int causal) {
  const int group = Hq / Hkv;
  const float scale = 1.0f / sqrtf((float)hd);
  const size_t Dq = (size_t)Hq * hd, Dk = (size_t)Hkv * hd;
  for (int s = 0; s < num_seqs; s++) {
    const int Tq = q_len[s], Tk = k_len[s];
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int h = 0; h < Hq; h++) {
      for (int i = 0; i < Tq; i++) {
        const int vis = attn_vis(i, Tq, Tk, causal);
        const uint16_t *q = Q + (size_t)(q_off[s] + i) * Dq + (size_t)h * hd;
        float *sc = (float *)malloc(sizeof(float) * (size_t)(vis > 0 ? vis : 1));
        float m = -INFINITY;
        for (int j = 0; j < vis; j++) {
          const uint16_t *k = K + (size_t)(k_off[s] + j) * Dk + (size_t)(h / group) * hd;
          float acc = 0.0f;
          for (int c = 0; c < hd; c++) acc += b2f(q[c]) * b2f(k[c]);
          sc[j] = acc * scale;
          m = fmaxf(m, sc[j]);
        }
        double sum = 0.0;
        for (int j = 0; j < vis; j++) sum += (double)expf(sc[j] - m);
        uint16_t *o = O + (size_t)(q_off[s] + i) * Dq + (size_t)h * hd;
        for (int j = 0; j < vis; j++) sc[j] = b2f(f2b(expf(sc[j] - m) / (float)sum)); /* the probability as bf16 */
        for (int c = 0; c < hd; c++) {
          float acc = 0.0f;
          for (int j = 0; j < vis; j++) acc += sc[j] * b2f(V[(size_t)(k_off[s] + j) * Dk + (size_t)(h / group) * hd + c]);
          o[c] = f2b(acc);
        }
        lse[(size_t)h * total_q + q_off[s] + i] = vis > 0 ? m + logf((float)sum) : -INFINITY;
        free(sc);
      }
    }
  }
}

/* Backward of the same: P = exp(S - lse) (bf16 where it multiplies dO), dP = dO V^T, delta_i = sum_c dO O,
 * dS = P (dP - delta) (bf16 where it multiplies K and Q), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO; the key /
 * value gradients are summed in fp32 over the query heads of a group and rounded once. dQ, dK, dV are overwritten. */
void orc_attention_bwd_bf16(int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len, const int *k_off,
                            const int *k_len, int Hq, int Hkv, int hd, const uint16_t *Q, const uint16_t *K,
                            const uint16_t *V, const uint16_t *O, const float *lse, const uint16_t *dO, uint16_t *dQ,
                            uint16_t *dK, uint16_t *dV, int causal) {
  const int group = Hq / Hkv;
  const float scale = 1.0f / sqrtf((float)hd);
  const size_t Dq = (size_t)Hq * hd, Dk = (size_t)Hkv * hd;
  float *aK = (float *)calloc((size_t)total_k * Dk, sizeof(float));
  float *aV = (float *)calloc((size_t)total_k * Dk, sizeof(float));
  for (int s = 0; s < num_seqs; s++) {
    const int Tq = q_len[s], Tk = k_len[s];
#pragma omp parallel for schedule(dynamic)
    for (int g = 0; g < Hkv; g++) { /* one thread owns the accumulators of a key / value head */
      for (int h = g * group; h < (g + 1) * group; h++) {
        for (int i = 0; i < Tq; i++) {
          const int vis = attn_vis(i, Tq, Tk, causal);
          const size_t qo = (size_t)(q_off[s] + i) * Dq + (size_t)h * hd;
          const float l = lse[(size_t)h * total_q + q_off[s] + i];
          float delta = 0.0f;
          for (int c = 0; c < hd; c++) delta += b2f(dO[qo + c]) * b2f(O[qo + c]);
          float *dq = (float *)calloc((size_t)hd, sizeof(float));
          for (int j = 0; j < vis; j++) {
            const size_t ko = (size_t)(k_off[s] + j) * Dk + (size_t)g * hd;
            float sc = 0.0f, dp = 0.0f;
            for (int c = 0; c < hd; c++) {
              sc += b2f(Q[qo + c]) * b2f(K[ko + c]);
              dp += b2f(dO[qo + c]) * b2f(V[ko + c]);
            }
            const float p = b2f(f2b(expf(sc * scale - l)));
            const float ds = b2f(f2b(p * (dp - delta)));
            for (int c = 0; c < hd; c++) {
              aV[ko + c] += p * b2f(dO[qo + c]);
              aK[ko + c] += scale * ds * b2f(Q[qo + c]);
              dq[c] += ds * b2f(K[ko + c]);
            }
          }
          for (int c = 0; c < hd; c++) dQ[qo + c] = f2b(scale * dq[c]);
          free(dq);
        }
      }
    }
    for (int j = 0; j < Tk; j++)
      for (size_t c = 0; c < Dk; c++) {
        const size_t o = (size_t)(k_off[s] + j) * Dk + c;
        dK[o] = f2b(aK[o]);
        dV[o] = f2b(aV[o]);
      }
  }
  free(aK);
  free(aV);
}
