// Causal / full softmax attention over variable-length sequences with grouped query heads, forward and backward:
// the op the reference takes from an external flash-attention library (dataflow_submit_attention / _attention_bwd,
// libdataflowops/include/dataflow_ops.h:70-105). This file holds the entry points and the GEMM-by-GEMM form: per
// sequence and query head a sequence of this library's own tcgen05 GEMMs on strided head slices (b200_matmul_strided)
// with the score matrix in the caller's workspace, and small kernels for the softmax, its backward and the fp32 -> bf16
// hand-over of the key / value gradients. Head sizes 64 and 128 are served by the fused kernels of attention_sm100.cu
// instead (forward both, backward 128), which were first checked against this form. The arithmetic of both follows
// the published algorithm the reference's library implements: scores and softmax statistics in fp32, probabilities
// rounded to bf16 before they multiply V (and dO in the backward), fp32 accumulation, one rounding per output; the
// backward re-forms the probabilities from Q, K and the kept log-sum-exp instead of storing them.
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

// attention_sm100.cu: the fused kernels for head sizes 64 and 128
bool attn_fused_supported(int head_dim);
int attn_fused_fwd(int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len, const int *k_off,
                   const int *k_len, int num_q_heads, int num_kv_heads, int head_dim, const void *Q, const void *K,
                   const void *V, void *O, float *lse, int is_causal, cudaStream_t s);
bool attn_fused_bwd_supported(int head_dim);
uint64_t attn_fused_bwd_workspace(int total_q, int num_q_heads, int head_dim);
int attn_fused_bwd(int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len, const int *k_off,
                   const int *k_len, int num_q_heads, int num_kv_heads, int head_dim, const void *Q, const void *K,
                   const void *V, const void *O, const float *lse, const void *dO, void *dQ, void *dK, void *dV,
                   int is_causal, void *workspace, cudaStream_t s);

constexpr int ATTN_THREADS = 256;
constexpr int ATTN_CACHE = 32;  // scores a thread keeps of one row: rows of up to 8192 keys are read once
constexpr float ATTN_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float attn_block_max(float v, float *scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (ATTN_THREADS >> 5) ? scratch[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

__device__ __forceinline__ float attn_block_sum(float v, float *scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (ATTN_THREADS >> 5) ? scratch[lane] : 0.0f;
  return warp_sum(t);
}

// keys a query row may see: all Tk, or (causal, the last query aligned with the last key) those up to its own position
__device__ __forceinline__ int attn_visible(int row, int Tq, int Tk, int causal) {
  if (!causal) return Tk;
  const int v = row + 1 + (Tk - Tq);
  return v < 0 ? 0 : (v > Tk ? Tk : v);
}

// One block per query row. S holds the scaled scores (fp32, pitch ldS). P = softmax over the visible keys as bf16,
// zeros up to the pitch ldP; lse[row] = max + log(sum) (-inf for a row that sees no key).
__global__ void __launch_bounds__(ATTN_THREADS)
attn_softmax_kernel(int row0, int Tq, int Tk, int causal, const float *__restrict__ S, int64_t ldS,
                    __nv_bfloat16 *__restrict__ P, int64_t ldP, int cols, float *__restrict__ lse) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;  // row of this chunk; row0 + row is the query's position in its sequence
  const int vis = attn_visible(row0 + row, Tq, Tk, causal);
  const float *s = S + (int64_t)row * ldS;
  __nv_bfloat16 *p = P + (int64_t)row * ldP;
  // rows of up to ATTN_THREADS * ATTN_CACHE scores are read once and kept in registers between the three passes
  float cache[ATTN_CACHE];
  const bool cached = vis <= ATTN_THREADS * ATTN_CACHE;
  float m = -INFINITY;
  if (cached) {
#pragma unroll
    for (int i = 0; i < ATTN_CACHE; i++) {
      const int j = i * ATTN_THREADS + threadIdx.x;
      cache[i] = j < vis ? s[j] : -INFINITY;
      m = fmaxf(m, cache[i]);
    }
  } else {
    for (int j = threadIdx.x; j < vis; j += ATTN_THREADS) m = fmaxf(m, s[j]);
  }
  m = attn_block_max(m, scratch);
  float sum = 0.0f;
  if (cached) {
#pragma unroll
    for (int i = 0; i < ATTN_CACHE; i++) {
      cache[i] = exp2f((cache[i] - m) * ATTN_LOG2E);  // 0 for the entries past the visible keys
      sum += cache[i];
    }
  } else {
    for (int j = threadIdx.x; j < vis; j += ATTN_THREADS) sum += exp2f((s[j] - m) * ATTN_LOG2E);
  }
  sum = attn_block_sum(sum, scratch);
  const float inv = vis > 0 ? 1.0f / sum : 0.0f;
  if (cached) {
#pragma unroll
    for (int i = 0; i < ATTN_CACHE; i++) {
      const int j = i * ATTN_THREADS + threadIdx.x;
      if (j < cols) p[j] = __float2bfloat16_rn(j < vis ? cache[i] * inv : 0.0f);
    }
    for (int j = ATTN_CACHE * ATTN_THREADS + threadIdx.x; j < cols; j += ATTN_THREADS) p[j] = __float2bfloat16_rn(0.0f);
  } else {
    for (int j = threadIdx.x; j < cols; j += ATTN_THREADS)
      p[j] = __float2bfloat16_rn(j < vis ? exp2f((s[j] - m) * ATTN_LOG2E) * inv : 0.0f);
  }
  if (threadIdx.x == 0) lse[row] = vis > 0 ? m + logf(sum) : -INFINITY;
}

// backward: the probabilities again from the scaled scores and the kept log-sum-exp
__global__ void __launch_bounds__(ATTN_THREADS)
attn_probs_kernel(int row0, int Tq, int Tk, int causal, const float *__restrict__ S, int64_t ldS,
                  const float *__restrict__ lse, __nv_bfloat16 *__restrict__ P, int64_t ldP, int cols) {
  const int row = blockIdx.x;
  const int vis = attn_visible(row0 + row, Tq, Tk, causal);
  const float *s = S + (int64_t)row * ldS;
  __nv_bfloat16 *p = P + (int64_t)row * ldP;
  const float l = lse[row];
  for (int j = threadIdx.x; j < cols; j += ATTN_THREADS)
    p[j] = __float2bfloat16_rn(j < vis ? exp2f((s[j] - l) * ATTN_LOG2E) : 0.0f);
}

// delta[row] = sum_d dO[row, d] * O[row, d] for one head (warp per row)
__global__ void __launch_bounds__(ATTN_THREADS)
attn_delta_kernel(int Tq, int head_dim, const __nv_bfloat16 *__restrict__ dO, const __nv_bfloat16 *__restrict__ O, int64_t ld,
                  float *__restrict__ delta) {
  const int row = blockIdx.x * (ATTN_THREADS >> 5) + (threadIdx.x >> 5);
  if (row >= Tq) return;
  float acc = 0.0f;
  for (int c = threadIdx.x & 31; c < head_dim; c += 32)
    acc += __bfloat162float(dO[(int64_t)row * ld + c]) * __bfloat162float(O[(int64_t)row * ld + c]);
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) delta[row] = acc;
}

// dS = P * (dP - delta[row]) in place over P (bf16), dP fp32
__global__ void __launch_bounds__(ATTN_THREADS)
attn_ds_kernel(const float *__restrict__ dP, int64_t ld_dP, const float *__restrict__ delta,
               __nv_bfloat16 *__restrict__ P, int64_t ldP, int cols) {
  const int row = blockIdx.x;
  const float dl = delta[row];
  __nv_bfloat16 *p = P + (int64_t)row * ldP;
  const float *g = dP + (int64_t)row * ld_dP;
  for (int j = threadIdx.x; j < cols; j += ATTN_THREADS) {
    const float pv = __bfloat162float(p[j]);
    p[j] = __float2bfloat16_rn(pv == 0.0f ? 0.0f : pv * (g[j] - dl));
  }
}

// fp32 [rows][cols] (packed) -> bf16 [rows][ld]
__global__ void attn_cast_kernel(int rows, int cols, const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t ld) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (int64_t)r * cols);
  dst[(int64_t)r * ld + c] = __float2bfloat16_rn(src[i]);
}

}  // namespace b200

using namespace b200;

namespace {

struct AttnWorkspace {
  float *S;            // [max_q][ldS]   scores, then dP in the backward
  __nv_bfloat16 *P;    // [max_q][ldS]   probabilities, then dS
  float *delta;        // [max_q]
  float *dK, *dV;      // [max_k][head_dim] fp32 accumulators over the query heads of a group
  int64_t ldS;
};

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// The fused kernels serve head sizes 64 and 128 unless the environment variable B200_ATTN_FUSED is "0" (read once; it
// exists so that the two forms can be compared on the same inputs).
bool use_fused(int head_dim) {
  static int mode = -1;
  if (mode < 0) {
    const char *e = getenv("B200_ATTN_FUSED");
    mode = (e && e[0] == '0') ? 0 : 1;
  }
  return mode == 1 && attn_fused_supported(head_dim);
}

// query rows per pass: 4096 under a causal mask, else the whole sequence. Smaller chunks skip more of the upper triangle
// but the passes are then bound by the host's launch rate (measured at 8192 tokens, 16 heads: whole 4.3 ms, 2048-row
// chunks 5.5 ms at 29 us per launch).
constexpr int ATTN_CHUNK = 4096;
int chunk_rows(int is_causal, int Tq) { return (is_causal && Tq > ATTN_CHUNK) ? ATTN_CHUNK : (Tq > 0 ? Tq : 1); }

uint64_t attn_workspace_layout(int is_training, int max_seqlen_q, int max_seqlen_k, int head_dim, unsigned char *base,
                               AttnWorkspace *w) {
  const int64_t ldS = round_up(max_seqlen_k, 8);
  uint64_t at = 0;
  auto take = [&](uint64_t bytes) {
    uint64_t here = at;
    at = (uint64_t)round_up((int64_t)(at + bytes), 256);
    return here;
  };
  const uint64_t oS = take((uint64_t)max_seqlen_q * ldS * 4), oP = take((uint64_t)max_seqlen_q * ldS * 2);
  uint64_t oD = 0, oK = 0, oV = 0;
  if (is_training) {
    oD = take((uint64_t)max_seqlen_q * 4);
    oK = take((uint64_t)max_seqlen_k * head_dim * 4);
    oV = take((uint64_t)max_seqlen_k * head_dim * 4);
  }
  if (w) {
    w->S = reinterpret_cast<float *>(base + oS);
    w->P = reinterpret_cast<__nv_bfloat16 *>(base + oP);
    w->delta = reinterpret_cast<float *>(base + oD);
    w->dK = reinterpret_cast<float *>(base + oK);
    w->dV = reinterpret_cast<float *>(base + oV);
    w->ldS = ldS;
  }
  return at;
}

int attn_check(const char *op, int dt, int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len,
               const int *k_off, const int *k_len, int num_q_heads, int num_kv_heads, int head_dim, int max_q, int max_k) {
  B200_REQUIRE(dt == B200_DT_BF16, "%s: only bf16 is implemented (datatype code %d)", op, dt);
  B200_REQUIRE(num_seqs >= 0 && total_q >= 0 && total_k >= 0 && q_off && q_len && k_off && k_len, "%s: bad sequence description", op);
  B200_REQUIRE(num_q_heads >= 1 && num_kv_heads >= 1 && num_q_heads % num_kv_heads == 0 && head_dim >= 8 && head_dim % 8 == 0,
               "%s: query heads must be a multiple of the key/value heads and head_dim a multiple of 8 (%d, %d, %d)", op,
               num_q_heads, num_kv_heads, head_dim);
  for (int s = 0; s < num_seqs; s++) {
    B200_REQUIRE(q_len[s] >= 0 && k_len[s] >= q_len[s] && q_len[s] <= max_q && k_len[s] <= max_k && q_off[s] >= 0 &&
                     k_off[s] >= 0 && q_off[s] + q_len[s] <= total_q && k_off[s] + k_len[s] <= total_k,
                 "%s: sequence %d (q %d+%d of %d, k %d+%d of %d; at most %d / %d per sequence, keys >= queries)", op, s,
                 q_off[s], q_len[s], total_q, k_off[s], k_len[s], total_k, max_q, max_k);
  }
  return 0;
}

// what a call needs: nothing for the fused forward, the dQ accumulator and delta for the fused backward, the score
// matrices of one (sequence, head, chunk) for the unfused form
uint64_t workspace_need(int is_training, int num_q_heads, int head_dim, int total_q, int max_seqlen_q, int max_seqlen_k,
                        bool for_backward) {
  const bool fused_fwd = use_fused(head_dim), fused_bwd = fused_fwd && attn_fused_bwd_supported(head_dim);
  if (for_backward || is_training) {
    if (fused_bwd) return attn_fused_bwd_workspace(total_q, num_q_heads, head_dim);
    return attn_workspace_layout(1, max_seqlen_q, max_seqlen_k, head_dim, nullptr, nullptr);
  }
  return fused_fwd ? 0 : attn_workspace_layout(0, max_seqlen_q, max_seqlen_k, head_dim, nullptr, nullptr);
}

}  // namespace

extern "C" uint64_t b200_attention_workspace_bytes(int is_training, int num_q_heads, int num_kv_heads, int head_dim,
                                                   int max_total_q, int max_seqlen_q, int max_seqlen_k) {
  if (max_seqlen_q <= 0 || max_seqlen_k <= 0 || head_dim <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_total_q <= 0)
    return 0;
  return workspace_need(is_training, num_q_heads, head_dim, max_total_q, max_seqlen_q, max_seqlen_k, false);
}

#define ATTN_MM(...)                              \
  do {                                            \
    if (b200_matmul_strided(__VA_ARGS__)) return -1; \
  } while (0)

extern "C" int b200_attention_fwd(int fwd_dt, int num_seqs, int total_q, int total_k, const int *q_seq_offsets,
                                  const int *q_seq_lens, int max_seqlen_q, const int *k_seq_offsets, const int *k_seq_lens,
                                  int max_seqlen_k, int num_q_heads, int num_kv_heads, int head_dim, const void *x_q,
                                  const void *x_k, const void *x_v, void *x_attn_out, float *softmax_lse, int is_causal,
                                  uint64_t workspaceBytes, void *workspace, void *stream) {
  if (attn_check("attention_fwd", fwd_dt, num_seqs, total_q, total_k, q_seq_offsets, q_seq_lens, k_seq_offsets, k_seq_lens,
                 num_q_heads, num_kv_heads, head_dim, max_seqlen_q, max_seqlen_k))
    return -1;
  B200_REQUIRE(x_q && x_k && x_v && x_attn_out && softmax_lse, "attention_fwd: null tensor");
  if (num_seqs == 0 || total_q == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (use_fused(head_dim))  // needs no workspace
    return attn_fused_fwd(num_seqs, total_q, total_k, q_seq_offsets, q_seq_lens, k_seq_offsets, k_seq_lens, num_q_heads,
                          num_kv_heads, head_dim, x_q, x_k, x_v, x_attn_out, softmax_lse, is_causal, s);
  AttnWorkspace w;
  const uint64_t need = attn_workspace_layout(0, max_seqlen_q, max_seqlen_k, head_dim, (unsigned char *)workspace, &w);
  B200_REQUIRE(workspace != nullptr && b200_aligned16(workspace) && workspaceBytes >= need,
               "attention_fwd: the workspace holds %llu bytes, %llu are needed (b200_attention_workspace_bytes)",
               (unsigned long long)workspaceBytes, (unsigned long long)need);
  const int BF = B200_DT_BF16, F32 = B200_DT_FP32, NONE = B200_DT_NONE;
  const int64_t Dq = (int64_t)num_q_heads * head_dim, Dk = (int64_t)num_kv_heads * head_dim;
  const int group = num_q_heads / num_kv_heads;
  const float scale = 1.0f / sqrtf((float)head_dim);
  const __nv_bfloat16 *Q = (const __nv_bfloat16 *)x_q, *K = (const __nv_bfloat16 *)x_k, *V = (const __nv_bfloat16 *)x_v;
  __nv_bfloat16 *O = (__nv_bfloat16 *)x_attn_out;
  for (int sq = 0; sq < num_seqs; sq++) {
    const int Tq = q_seq_lens[sq], Tk = k_seq_lens[sq];
    if (Tq == 0) continue;
    const int Tk8 = (int)round_up(Tk, 8);
    const int k_extent = (int)std::min<int64_t>(Tk8, (int64_t)total_k - k_seq_offsets[sq]);
    for (int h = 0; h < num_q_heads; h++) {
      const __nv_bfloat16 *Qh = Q + (int64_t)q_seq_offsets[sq] * Dq + (int64_t)h * head_dim;
      const __nv_bfloat16 *Kg = K + (int64_t)k_seq_offsets[sq] * Dk + (int64_t)(h / group) * head_dim;
      const __nv_bfloat16 *Vg = V + (int64_t)k_seq_offsets[sq] * Dk + (int64_t)(h / group) * head_dim;
      __nv_bfloat16 *Oh = O + (int64_t)q_seq_offsets[sq] * Dq + (int64_t)h * head_dim;
      float *lse = softmax_lse + (int64_t)h * total_q + q_seq_offsets[sq];
      // Causal: the queries go in chunks of ATTN_CHUNK rows, each against the keys its last row may see, so that part of
      // the upper triangle is never computed.
      for (int r0 = 0; r0 < Tq; r0 += chunk_rows(is_causal, Tq)) {
        const int rows = std::min(chunk_rows(is_causal, Tq), Tq - r0);
        const int keys = is_causal ? std::min(Tk, r0 + rows + (Tk - Tq)) : Tk;
        const int keys8 = (int)round_up(keys, 8);
        // S[rows][keys8] = scale * Q_h K_g^T (fp32)
        ATTN_MM(BF, BF, NONE, F32, 1, 0, keys8, head_dim, rows, scale, 0.0f, Kg, Dk, std::min(keys8, k_extent), Qh + r0 * Dq,
                Dq, nullptr, w.S, w.ldS, stream);
        attn_softmax_kernel<<<rows, ATTN_THREADS, 0, s>>>(r0, Tq, Tk, is_causal, w.S, w.ldS, w.P, w.ldS, keys8, lse + r0);
        B200_CHECK_LAUNCH("attention_fwd (softmax)");
        // O_h[rows][hd] = P V_g
        ATTN_MM(BF, BF, NONE, BF, 0, 0, head_dim, keys, rows, 1.0f, 0.0f, Vg, Dk, head_dim, w.P, w.ldS, nullptr, Oh + r0 * Dq,
                Dq, stream);
      }
    }
  }
  return 0;
}

extern "C" int b200_attention_bwd(int bwd_dt, int num_seqs, int total_q, int total_k, const int *q_seq_offsets,
                                  const int *q_seq_lens, int max_seqlen_q, const int *k_seq_offsets, const int *k_seq_lens,
                                  int max_seqlen_k, int num_q_heads, int num_kv_heads, int head_dim, const void *x_q,
                                  const void *x_k, const void *x_v, const void *x_attn_out, const float *softmax_lse,
                                  const void *dx_out, void *dx_q, void *dx_k, void *dx_v, int is_causal,
                                  uint64_t workspaceBytes, void *workspace, void *stream) {
  if (attn_check("attention_bwd", bwd_dt, num_seqs, total_q, total_k, q_seq_offsets, q_seq_lens, k_seq_offsets, k_seq_lens,
                 num_q_heads, num_kv_heads, head_dim, max_seqlen_q, max_seqlen_k))
    return -1;
  B200_REQUIRE(x_q && x_k && x_v && x_attn_out && softmax_lse && dx_out && dx_q && dx_k && dx_v, "attention_bwd: null tensor");
  if (num_seqs == 0 || total_q == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (use_fused(head_dim) && attn_fused_bwd_supported(head_dim)) {
    const uint64_t need = attn_fused_bwd_workspace(total_q, num_q_heads, head_dim);
    B200_REQUIRE(workspace != nullptr && b200_aligned16(workspace) && workspaceBytes >= need,
                 "attention_bwd: the workspace holds %llu bytes, %llu are needed (b200_attention_workspace_bytes)",
                 (unsigned long long)workspaceBytes, (unsigned long long)need);
    return attn_fused_bwd(num_seqs, total_q, total_k, q_seq_offsets, q_seq_lens, k_seq_offsets, k_seq_lens, num_q_heads,
                          num_kv_heads, head_dim, x_q, x_k, x_v, x_attn_out, softmax_lse, dx_out, dx_q, dx_k, dx_v, is_causal,
                          workspace, s);
  }
  AttnWorkspace w;
  const uint64_t need = attn_workspace_layout(1, max_seqlen_q, max_seqlen_k, head_dim, (unsigned char *)workspace, &w);
  B200_REQUIRE(workspace != nullptr && b200_aligned16(workspace) && workspaceBytes >= need,
               "attention_bwd: the workspace holds %llu bytes, %llu are needed (b200_attention_workspace_bytes)",
               (unsigned long long)workspaceBytes, (unsigned long long)need);
  const int BF = B200_DT_BF16, F32 = B200_DT_FP32, NONE = B200_DT_NONE;
  const int64_t Dq = (int64_t)num_q_heads * head_dim, Dk = (int64_t)num_kv_heads * head_dim;
  const int group = num_q_heads / num_kv_heads;
  const float scale = 1.0f / sqrtf((float)head_dim);
  const __nv_bfloat16 *Q = (const __nv_bfloat16 *)x_q, *K = (const __nv_bfloat16 *)x_k, *V = (const __nv_bfloat16 *)x_v;
  const __nv_bfloat16 *O = (const __nv_bfloat16 *)x_attn_out, *dO = (const __nv_bfloat16 *)dx_out;
  __nv_bfloat16 *dQ = (__nv_bfloat16 *)dx_q, *dK = (__nv_bfloat16 *)dx_k, *dV = (__nv_bfloat16 *)dx_v;
  for (int sq = 0; sq < num_seqs; sq++) {
    const int Tq = q_seq_lens[sq], Tk = k_seq_lens[sq];
    if (Tk == 0) continue;
    const int Tk8 = (int)round_up(Tk, 8);
    const int k_extent = (int)std::min<int64_t>(Tk8, (int64_t)total_k - k_seq_offsets[sq]);
    for (int g = 0; g < num_kv_heads; g++) {
      const __nv_bfloat16 *Kg = K + (int64_t)k_seq_offsets[sq] * Dk + (int64_t)g * head_dim;
      const __nv_bfloat16 *Vg = V + (int64_t)k_seq_offsets[sq] * Dk + (int64_t)g * head_dim;
      B200_CUDA(cudaMemsetAsync(w.dK, 0, sizeof(float) * (size_t)Tk * head_dim, s));
      B200_CUDA(cudaMemsetAsync(w.dV, 0, sizeof(float) * (size_t)Tk * head_dim, s));
      for (int h = g * group; h < (g + 1) * group && Tq > 0; h++) {
        const int64_t qo = (int64_t)q_seq_offsets[sq] * Dq + (int64_t)h * head_dim;
        const __nv_bfloat16 *Qh = Q + qo, *Oh = O + qo, *dOh = dO + qo;
        const float *lse = softmax_lse + (int64_t)h * total_q + q_seq_offsets[sq];
        for (int r0 = 0; r0 < Tq; r0 += chunk_rows(is_causal, Tq)) {
          const int rows = std::min(chunk_rows(is_causal, Tq), Tq - r0);
          const int keys = is_causal ? std::min(Tk, r0 + rows + (Tk - Tq)) : Tk;
          const int keys8 = (int)round_up(keys, 8);
          const int kext = std::min(keys8, k_extent);
          const __nv_bfloat16 *Qc = Qh + r0 * Dq, *dOc = dOh + r0 * Dq;
          // the probabilities again: S = scale Q K^T, P = exp(S - lse)
          ATTN_MM(BF, BF, NONE, F32, 1, 0, keys8, head_dim, rows, scale, 0.0f, Kg, Dk, kext, Qc, Dq, nullptr, w.S, w.ldS, stream);
          attn_probs_kernel<<<rows, ATTN_THREADS, 0, s>>>(r0, Tq, Tk, is_causal, w.S, w.ldS, lse + r0, w.P, w.ldS, keys8);
          B200_CHECK_LAUNCH("attention_bwd (probabilities)");
          // dV_g[keys][hd] += P^T dO_h  (fp32 over the chunks and the heads of the group)
          ATTN_MM(BF, BF, F32, F32, 0, 1, head_dim, rows, keys, 1.0f, 1.0f, dOc, Dq, head_dim, w.P, w.ldS, w.dV, w.dV, head_dim,
                  stream);
          // dP[rows][keys8] = dO_h V_g^T (fp32, over the score buffer)
          ATTN_MM(BF, BF, NONE, F32, 1, 0, keys8, head_dim, rows, 1.0f, 0.0f, Vg, Dk, kext, dOc, Dq, nullptr, w.S, w.ldS, stream);
          attn_delta_kernel<<<(rows + 7) / 8, ATTN_THREADS, 0, s>>>(rows, head_dim, dOc, Oh + r0 * Dq, Dq, w.delta);
          B200_CHECK_LAUNCH("attention_bwd (delta)");
          attn_ds_kernel<<<rows, ATTN_THREADS, 0, s>>>(w.S, w.ldS, w.delta, w.P, w.ldS, keys8);
          B200_CHECK_LAUNCH("attention_bwd (dS)");
          // dQ_h[rows][hd] = scale dS K_g
          ATTN_MM(BF, BF, NONE, BF, 0, 0, head_dim, keys, rows, scale, 0.0f, Kg, Dk, head_dim, w.P, w.ldS, nullptr,
                  dQ + qo + r0 * Dq, Dq, stream);
          // dK_g[keys][hd] += scale dS^T Q_h
          ATTN_MM(BF, BF, F32, F32, 0, 1, head_dim, rows, keys, scale, 1.0f, Qc, Dq, head_dim, w.P, w.ldS, w.dK, w.dK, head_dim,
                  stream);
        }
      }
      const int64_t ko = (int64_t)k_seq_offsets[sq] * Dk + (int64_t)g * head_dim;
      const int64_t n = (int64_t)Tk * head_dim;
      attn_cast_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(Tk, head_dim, w.dK, dK + ko, Dk);
      attn_cast_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(Tk, head_dim, w.dV, dV + ko, Dk);
      B200_CHECK_LAUNCH("attention_bwd (cast)");
    }
  }
  return 0;
}
