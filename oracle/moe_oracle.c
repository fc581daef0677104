/*
 * CPU oracle for the mixture-of-experts layer ops.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is a plain-C restatement of what the
 * reference's CUDA kernels compute, used only to check the sm_100a kernels
 * and to time a CPU baseline. Nothing in the product path links or calls it.
 *
 * Parity status: the reference ships no golden vectors, known-answer tests or
 * expected tensors for these ops. The integer/indexing part of this oracle
 * (top-k slot order, counts, cumsums, mappings) is pinned by running the
 * reference's own kernels, compiled from the reference sources, on the GPU
 * (tests/test_reference_kernels_gpu.py). The floating-point part is pinned
 * against golden tensors produced by the reference's PyTorch MoE layer
 * (tests/golden/). The per-expert GEMMs run in closed-source cuBLASLt in the
 * reference: that boundary is "parity unpinned"; GEMM here is defined as an
 * fp32-accumulated dot product with one round-to-nearest-even to bf16.
 *
 * Each function names the reference file:line whose behaviour it restates
 * (paths relative to the reference project root; "moe/" stands for
 * backends/nvidia/src/ops/src/native/src/moe/ and "activations/" for
 * backends/nvidia/src/ops/src/native/src/activations/).
 *
 * bf16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_DT_FP32 3 /* same numeric values as the reference's DataflowDatatype */
#define ORC_DT_BF16 5 /* libdataflow/include/dataflow_common.h:46-74 */

/* ---- bf16 helpers ------------------------------------------------------ */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even, the rounding of CUDA's __float2bfloat16_rn used by
 * every reference kernel (e.g. moe/merge_expert_result.cu:231-234). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP team size (a launcher such as torch.distributed.run exports OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void orc_f32_to_bf16(const float *src, uint16_t *dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}

void orc_bf16_to_f32(const uint16_t *src, float *dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

/* ---- deterministic synthetic inputs ------------------------------------- */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

/* Counter-based N(mean, std) stream: element i of stream `seed` depends only
 * on (seed, i), so any slice can be generated anywhere. Box-Muller on two
 * 24-bit uniforms from one splitmix64 draw. */
static inline float gauss_at(uint64_t seed, uint64_t i) {
  uint64_t r = splitmix64(seed * 0xD1342543DE82EF95ull + i);
  float u1 = ((float)((r >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f); /* (0,1] */
  float u2 = (float)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);           /* [0,1) */
  return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

void orc_fill_normal_f32(float *dst, int64_t n, uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) dst[i] = mean + std * gauss_at(seed, (uint64_t)i);
}

void orc_fill_normal_bf16(uint16_t *dst, int64_t n, uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(mean + std * gauss_at(seed, (uint64_t)i));
}

/* ---- select_experts ----------------------------------------------------- */

/*
 * moe/select_experts.cu:3-295 (fp32 kernel).
 * Per token: walk experts in ascending order keeping k slots. A logit enters
 * only if it is strictly greater than the current minimum (lines 141); it
 * overwrites the minimum slot (147-148); the new minimum is the smallest
 * value, ties going to the slot holding the LARGER expert index (152-163).
 * Slots start at -inf with index 0xFFFF (111-116). Gate weight = softmax over
 * the k kept logits (174-189). Histogram (195-196, 207-209), exclusive scan
 * (236-283), counts copied to host_expert_counts (288-294).
 * expert_counts has E+1 ints and is zeroed by the caller; slot E counts
 * finished thread blocks in the reference (lines 21, 213) and is left alone
 * here. A slot that never filled keeps 0xFFFF and is not counted (the
 * reference would index out of bounds there).
 */
void orc_select_experts_f32(int total_tokens, int n_experts, int top_k, const float *X_routed,
                            float *token_expert_weights, uint16_t *chosen_experts,
                            int *expert_counts, int *expert_counts_cumsum,
                            int *host_expert_counts) {
  int nthreads = orc_num_threads();
  int *local = (int *)calloc((size_t)nthreads * n_experts, sizeof(int));
#pragma omp parallel
  {
#ifdef _OPENMP
    int tid = omp_get_thread_num();
#else
    int tid = 0;
#endif
    int *cnt = local + (size_t)tid * n_experts;
    float *vals = (float *)malloc(sizeof(float) * top_k);
    uint16_t *inds = (uint16_t *)malloc(sizeof(uint16_t) * top_k);
#pragma omp for schedule(static)
    for (int t = 0; t < total_tokens; t++) {
      const float *row = X_routed + (int64_t)t * n_experts;
      float max_val = -INFINITY, min_val = -INFINITY;
      int min_slot = 0;
      for (int j = 0; j < top_k; j++) {
        vals[j] = -INFINITY;
        inds[j] = 0xFFFF;
      }
      for (int e = 0; e < n_experts; e++) {
        float v = row[e];
        if (v > min_val) {
          if (v > max_val) max_val = v;
          vals[min_slot] = v;
          inds[min_slot] = (uint16_t)e;
          min_val = INFINITY;
          min_slot = 0;
          uint16_t min_exp = 0xFFFF;
          for (int j = 0; j < top_k; j++) {
            if (vals[j] < min_val || (vals[j] == min_val && inds[j] > min_exp)) {
              min_val = vals[j];
              min_slot = j;
              min_exp = inds[j];
            }
          }
        }
      }
      float sum = 0.0f;
      for (int j = 0; j < top_k; j++) sum += expf(vals[j] - max_val);
      for (int j = 0; j < top_k; j++) {
        token_expert_weights[(int64_t)t * top_k + j] = expf(vals[j] - max_val) / sum;
        chosen_experts[(int64_t)t * top_k + j] = inds[j];
        if (inds[j] < n_experts) cnt[inds[j]]++;
      }
    }
    free(vals);
    free(inds);
  }
  for (int e = 0; e < n_experts; e++) {
    int s = 0;
    for (int th = 0; th < nthreads; th++) s += local[(size_t)th * n_experts + e];
    expert_counts[e] += s;
  }
  free(local);
  int run = 0;
  for (int e = 0; e < n_experts; e++) {
    expert_counts_cumsum[e] = run;
    run += expert_counts[e];
    if (host_expert_counts) host_expert_counts[e] = expert_counts[e];
  }
}

/* ---- build_expert_mapping ------------------------------------------------ */

/*
 * moe/build_expert_mapping.cu:18-103. Counting-sort scatter.
 * In: expert_counts_cumsum = EXCLUSIVE prefix sums. Out: expert_mapping[row]
 * = token, token_mapping[t*k+j] = row, and expert_counts_cumsum turned into
 * the INCLUSIVE prefix sums (the atomicAdd of line 65 advances each entry by
 * that expert's count).
 * The reference reserves ranges with atomics, so its order inside an expert
 * is arrival order. This oracle fixes the canonical stable order: tokens
 * ascending, slots ascending. Any reference run is a permutation of this
 * inside each expert's range.
 */
void orc_build_expert_mapping(int num_tokens, int num_routed_experts, int num_selected,
                              const uint16_t *chosen_experts, int *expert_counts_cumsum,
                              int *expert_mapping, int *token_mapping) {
  for (int64_t i = 0; i < (int64_t)num_tokens * num_selected; i++) {
    uint16_t e = chosen_experts[i];
    if (e >= num_routed_experts) {
      token_mapping[i] = -1;
      continue;
    }
    int pos = expert_counts_cumsum[e]++;
    expert_mapping[pos] = (int)(i / num_selected);
    token_mapping[i] = pos;
  }
}

/* ---- prepare_experts / prepare_expert_zone ------------------------------- */

/* moe/prepare_expert_zone.cu:69-117: zone[token_mapping[t,j], :] = X[t, :]. */
void orc_prepare_experts(int total_tokens, int model_dim, int num_selected, const uint16_t *X,
                         const int *token_mapping, uint16_t *expert_zones) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < total_tokens; t++) {
    for (int j = 0; j < num_selected; j++) {
      int r = token_mapping[(int64_t)t * num_selected + j];
      if (r < 0) continue;
      memcpy(expert_zones + (int64_t)r * model_dim, X + (int64_t)t * model_dim,
             (size_t)model_dim * 2);
    }
  }
}

/* moe/prepare_expert_zone.cu:28-67: per-expert gather. expert_zone points at
 * this expert's first row; cumsum is inclusive (base = cumsum[e] - count). */
void orc_prepare_expert_zone(int model_dim, const uint16_t *X, int expert_id,
                             const int *expert_counts, const int *expert_counts_cumsum,
                             const int *expert_mapping, uint16_t *expert_zone) {
  int n = expert_counts[expert_id];
  int base = expert_counts_cumsum[expert_id] - n;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n; r++) {
    int t = expert_mapping[base + r];
    memcpy(expert_zone + (int64_t)r * model_dim, X + (int64_t)t * model_dim,
           (size_t)model_dim * 2);
  }
}

/* ---- merge_experts / merge_expert_result --------------------------------- */

/*
 * moe/merge_expert_result.cu:118-247 (and the naive form 250-292).
 * out[t,:] = bf16( f32(out[t,:]) + sum_j w[t,j] * f32(zone[token_mapping[t,j],:]) ),
 * j ascending, fp32 accumulation, one rounding. weights == NULL means 1.0
 * (lines 184-188; used as the backward un-permute).
 */
void orc_merge_experts(int total_tokens, int model_dim, int num_selected,
                       const uint16_t *expert_zones, const int *token_mapping,
                       const float *token_expert_weights, uint16_t *X_combined) {
#pragma omp parallel
  {
    float *acc = (float *)malloc(sizeof(float) * model_dim);
#pragma omp for schedule(static)
    for (int t = 0; t < total_tokens; t++) {
      uint16_t *out = X_combined + (int64_t)t * model_dim;
      for (int c = 0; c < model_dim; c++) acc[c] = bf16_to_f32(out[c]);
      for (int j = 0; j < num_selected; j++) {
        int r = token_mapping[(int64_t)t * num_selected + j];
        if (r < 0) continue;
        float w = token_expert_weights ? token_expert_weights[(int64_t)t * num_selected + j] : 1.0f;
        const uint16_t *z = expert_zones + (int64_t)r * model_dim;
        for (int c = 0; c < model_dim; c++) acc[c] += w * bf16_to_f32(z[c]);
      }
      for (int c = 0; c < model_dim; c++) out[c] = f32_to_bf16(acc[c]);
    }
    free(acc);
  }
}

/* moe/merge_expert_result.cu:3-115: per-expert read-modify-write combine.
 * num_tokens = this expert's row count; expert_zone = its first row;
 * the weight is looked up by scanning the token's chosen_experts (35-42). */
void orc_merge_expert_result(int num_tokens, int model_dim, int top_k, const uint16_t *expert_zone,
                             int expert_id, const int *expert_counts_cumsum,
                             const int *expert_mapping, const float *token_expert_weights,
                             const uint16_t *chosen_experts, uint16_t *X_combined) {
  int base = expert_counts_cumsum[expert_id] - num_tokens;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < num_tokens; r++) {
    int t = expert_mapping[base + r];
    float w = 1.0f;
    if (token_expert_weights) {
      w = 0.0f;
      for (int j = 0; j < top_k; j++)
        if (chosen_experts[(int64_t)t * top_k + j] == (uint16_t)expert_id) {
          w = token_expert_weights[(int64_t)t * top_k + j];
          break;
        }
    }
    if (w == 0.0f) continue;
    const uint16_t *z = expert_zone + (int64_t)r * model_dim;
    uint16_t *out = X_combined + (int64_t)t * model_dim;
    for (int c = 0; c < model_dim; c++)
      out[c] = f32_to_bf16(bf16_to_f32(out[c]) + w * bf16_to_f32(z[c]));
  }
}

/* ---- swiglu --------------------------------------------------------------- */

/* activations/swiglu.cu:153-173: out = silu(x1) * x3 in fp32, one rounding. */
void orc_swiglu(int num_rows, int num_cols, const uint16_t *x_w1, const uint16_t *x_w3,
                uint16_t *out) {
  int64_t n = (int64_t)num_rows * num_cols;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    float a = bf16_to_f32(x_w1[i]), b = bf16_to_f32(x_w3[i]);
    float silu = a / (1.0f + expf(-a));
    out[i] = f32_to_bf16(silu * b);
  }
}

/* activations/swiglu_bwd_x.cu:258-300:
 * dx3 = dy*silu(x1); dx1 = dy*x3*(s + x1*s*(1-s)), s = sigmoid(x1). */
void orc_swiglu_bwd_x(int num_rows, int num_cols, const uint16_t *x_w1, const uint16_t *x_w3,
                      const uint16_t *upstream_dX, uint16_t *dX_w1, uint16_t *dX_w3) {
  int64_t n = (int64_t)num_rows * num_cols;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    float a = bf16_to_f32(x_w1[i]), b = bf16_to_f32(x_w3[i]), g = bf16_to_f32(upstream_dX[i]);
    float s = 1.0f / (1.0f + expf(-a));
    float silu = a * s;
    float dsilu = s + a * (s * (1.0f - s));
    dX_w3[i] = f32_to_bf16(g * silu);
    dX_w1[i] = f32_to_bf16(g * b * dsilu);
  }
}

/* ---- router backward ------------------------------------------------------ */

/*
 * moe/router_bwd_x.cu:95-200 (naive form; optimised form 4-92), one expert.
 * For row r of this expert (token t = expert_mapping[base + r]):
 *   dX_routed[t, expert_id] = bf16( <expert_out[r,:], upstream_dX[t,:]> )   (line 64)
 *   dX_expert_out[r,:]      = bf16( upstream_dX[t,:] * w[t, expert] )        (190-192)
 * expert_out / dX_expert_out point at the expert's first row and may alias.
 * The optimised kernel multiplies in bf16 after rounding w to bf16 (83-86);
 * this oracle keeps the fp32 product, the tolerance covers the difference.
 */
void orc_router_bwd_x(int num_expert_tokens, int model_dim, int num_routed_experts, int top_k,
                      int expert_id, const int *expert_counts_cumsum, const int *expert_mapping,
                      const uint16_t *chosen_experts, const float *token_expert_weights,
                      const uint16_t *expert_out, const uint16_t *upstream_dX,
                      uint16_t *dX_routed, uint16_t *dX_expert_out) {
  int base = expert_counts_cumsum[expert_id] - num_expert_tokens;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < num_expert_tokens; r++) {
    int t = expert_mapping[base + r];
    const uint16_t *y = expert_out + (int64_t)r * model_dim;
    const uint16_t *g = upstream_dX + (int64_t)t * model_dim;
    float dot = 0.0f;
    for (int c = 0; c < model_dim; c++) dot += bf16_to_f32(y[c]) * bf16_to_f32(g[c]);
    dX_routed[(int64_t)t * num_routed_experts + expert_id] = f32_to_bf16(dot);
    float w = 0.0f;
    for (int j = 0; j < top_k; j++)
      if (chosen_experts[(int64_t)t * top_k + j] == (uint16_t)expert_id) {
        w = token_expert_weights[(int64_t)t * top_k + j];
        break;
      }
    if (w == 0.0f) continue;
    uint16_t *o = dX_expert_out + (int64_t)r * model_dim;
    for (int c = 0; c < model_dim; c++) o[c] = f32_to_bf16(bf16_to_f32(g[c]) * w);
  }
}

/*
 * moe/router_gate_bwd_x.cu:7-57. Softmax-over-k Jacobian, in place on the k
 * chosen columns: g_i = p_i * (dp_i - sum_j dp_j p_j); other columns untouched.
 */
void orc_router_gate_bwd_x(int num_tokens, int num_routed_experts, int top_k,
                           const uint16_t *chosen_experts, const float *token_expert_weights,
                           uint16_t *dX_routed) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < num_tokens; t++) {
    uint16_t *row = dX_routed + (int64_t)t * num_routed_experts;
    const uint16_t *ce = chosen_experts + (int64_t)t * top_k;
    const float *w = token_expert_weights + (int64_t)t * top_k;
    float avg = 0.0f;
    for (int j = 0; j < top_k; j++)
      if (ce[j] < num_routed_experts) avg += bf16_to_f32(row[ce[j]]) * w[j];
    for (int j = 0; j < top_k; j++)
      if (ce[j] < num_routed_experts) row[ce[j]] = f32_to_bf16(w[j] * (bf16_to_f32(row[ce[j]]) - avg));
  }
}

/* ---- matmul ---------------------------------------------------------------- */

static inline float load_el(const void *p, int dt, int64_t i) {
  return dt == ORC_DT_FP32 ? ((const float *)p)[i] : bf16_to_f32(((const uint16_t *)p)[i]);
}

/*
 * libdataflowops/include/dataflow_ops.h:21-80 and
 * backends/nvidia/src/ops/src/external/matmul_helper/src/matmul_helper.c:347-420, 774-946.
 * Column-major D[M x N] = alpha * op(A) * op(B) + beta * C with packed leading
 * dimensions: A is K x M when to_trans_a else M x K; B is N x K when
 * to_trans_b else K x N; C, D are M x N. fp32 accumulation
 * (CUBLAS_COMPUTE_32F), one rounding to the output type. C may be NULL or
 * alias D. Element types are ORC_DT_FP32 or ORC_DT_BF16. Returns 0, or -1 on
 * an unsupported type.
 */
int orc_matmul(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M,
               int K, int N, float alpha, float beta, const void *A, const void *B, const void *C,
               void *D) {
  if ((a_dt != ORC_DT_FP32 && a_dt != ORC_DT_BF16) || (b_dt != ORC_DT_FP32 && b_dt != ORC_DT_BF16) ||
      (d_dt != ORC_DT_FP32 && d_dt != ORC_DT_BF16))
    return -1;
  if (M <= 0 || N <= 0) return 0;
  /* K-contiguous fp32 copies: At[m][k], Bt[n][k] */
  float *At = (float *)malloc(sizeof(float) * (size_t)M * (K > 0 ? K : 1));
  float *Bt = (float *)malloc(sizeof(float) * (size_t)N * (K > 0 ? K : 1));
  if (!At || !Bt) {
    free(At);
    free(Bt);
    return -1;
  }
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; m++)
    for (int k = 0; k < K; k++)
      At[(int64_t)m * K + k] =
          load_el(A, a_dt, to_trans_a ? ((int64_t)m * K + k) : ((int64_t)k * M + m));
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++)
    for (int k = 0; k < K; k++)
      Bt[(int64_t)n * K + k] =
          load_el(B, b_dt, to_trans_b ? ((int64_t)k * N + n) : ((int64_t)n * K + k));
  int use_c = (C != NULL) && (beta != 0.0f);
#pragma omp parallel for schedule(dynamic, 4)
  for (int n = 0; n < N; n++) {
    const float *b = Bt + (int64_t)n * K;
    for (int m = 0; m < M; m++) {
      const float *a = At + (int64_t)m * K;
      float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
      for (int k = 0; k < K; k++) acc += a[k] * b[k];
      float v = alpha * acc;
      int64_t o = (int64_t)n * M + m;
      if (use_c) v += beta * load_el(C, c_dt, o);
      if (d_dt == ORC_DT_FP32)
        ((float *)D)[o] = v;
      else
        ((uint16_t *)D)[o] = f32_to_bf16(v);
    }
  }
  free(At);
  free(Bt);
  return 0;
}
