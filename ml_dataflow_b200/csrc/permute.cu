// Bandwidth-bound row movers: gather into expert-contiguous order, weighted combine back to
// token order, the per-expert variants, router_bwd_x and the SwiGLU elementwise ops.
// All rows are bf16 and moved as 16-byte vectors (8 elements).
#include "common.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

constexpr int ROW_THREADS = 128;

// ---------------------------------------------------------------------------------------
// prepare_experts: zone[token_mapping[t,j], :] = X[t, :]   (moe/prepare_expert_zone.cu:69-117)
// One block per token. Each thread keeps up to VPT 16-byte pieces of the row in registers
// (all loads issued before the first store) and writes them to the k destination rows.
// ---------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(ROW_THREADS)
prepare_experts_kernel(int total_tokens, int dim_vec, int top_k, const uint4 *__restrict__ X,
                       const int *__restrict__ token_mapping, const float *__restrict__ weights,
                       uint4 *__restrict__ zone) {
  __shared__ int dst_rows[B200_MAX_TOP_K];
  __shared__ float dst_w[B200_MAX_TOP_K];
  for (int64_t token = blockIdx.x; token < total_tokens; token += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < top_k) {
      dst_rows[threadIdx.x] = token_mapping[token * top_k + threadIdx.x];
      if (weights) dst_w[threadIdx.x] = weights[token * top_k + threadIdx.x];
    }
    __syncthreads();
    const uint4 *src = X + token * dim_vec;
    for (int c0 = 0; c0 < dim_vec; c0 += ROW_THREADS * VPT) {
      uint4 v[VPT];
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        int c = c0 + i * ROW_THREADS + threadIdx.x;
        if (c < dim_vec) v[i] = ld_stream(src + c);
      }
      for (int j = 0; j < top_k; j++) {
        const int r = dst_rows[j];
        if (r < 0) continue;
        uint4 *dst = zone + (int64_t)r * dim_vec;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          int c = c0 + i * ROW_THREADS + threadIdx.x;
          if (c < dim_vec) {
            if (weights) {  // row scaled by its gate weight: fp32 product, one rounding
              float f[8];
              unpack8(v[i], f);
              const float w = dst_w[j];
#pragma unroll
              for (int q = 0; q < 8; q++) f[q] *= w;
              st_stream(dst + c, pack8(f));
            } else {
              st_stream(dst + c, v[i]);
            }
          }
        }
      }
    }
  }
}

// per-expert gather (moe/prepare_expert_zone.cu:28-67): one block per destination row
__global__ void __launch_bounds__(ROW_THREADS)
prepare_expert_zone_kernel(int dim_vec, const uint4 *__restrict__ X, int expert_id,
                           const int *__restrict__ expert_counts, const int *__restrict__ cumsum_incl,
                           const int *__restrict__ expert_mapping, uint4 *__restrict__ zone) {
  const int n = expert_counts[expert_id];
  const int base = cumsum_incl[expert_id] - n;
  for (int r = blockIdx.x; r < n; r += gridDim.x) {
    const int t = expert_mapping[base + r];
    const uint4 *src = X + (int64_t)t * dim_vec;
    uint4 *dst = zone + (int64_t)r * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += ROW_THREADS) st_stream(dst + c, ld_stream(src + c));
  }
}

// ---------------------------------------------------------------------------------------
// merge_experts (moe/merge_expert_result.cu:118-247): one block per token, each thread owns
// 16-byte column pieces; for every piece the k gathered loads are issued together, then
// accumulated in slot order in fp32 on top of the existing output row; one rounding.
// ---------------------------------------------------------------------------------------
// OVERWRITE: the output row starts from zero instead of being read (the un-permute of the backward, where the
// reference zeroes dX and then accumulates: same bits, a third fewer bytes and no memset)
template <int KU, bool OVERWRITE = false>
__global__ void __launch_bounds__(ROW_THREADS)
merge_experts_kernel(int num_tokens, int dim_vec, int top_k, const uint4 *__restrict__ zone,
                     const int *__restrict__ token_mapping, const float *__restrict__ weights,
                     uint4 *__restrict__ X_combined) {
  __shared__ int rows[B200_MAX_TOP_K];
  __shared__ float wts[B200_MAX_TOP_K];
  for (int64_t token = blockIdx.x; token < num_tokens; token += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < top_k) {
      rows[threadIdx.x] = token_mapping[token * top_k + threadIdx.x];
      wts[threadIdx.x] = weights ? weights[token * top_k + threadIdx.x] : 1.0f;
    }
    __syncthreads();
    uint4 *out = X_combined + token * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += ROW_THREADS) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (!OVERWRITE) unpack8(out[c], acc);
      for (int j0 = 0; j0 < top_k; j0 += KU) {
        uint4 v[KU];
#pragma unroll
        for (int u = 0; u < KU; u++) {
          const int j = j0 + u;
          const int r = (j < top_k) ? rows[j] : -1;
          v[u] = (r >= 0) ? ld_stream(zone + (int64_t)r * dim_vec + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < KU; u++) {
          const int j = j0 + u;
          if (j < top_k && rows[j] >= 0) {
            const float w = wts[j];
            float f[8];
            unpack8(v[u], f);
#pragma unroll
            for (int q = 0; q < 8; q++) acc[q] += w * f[q];
          }
        }
      }
      out[c] = pack8(acc);
    }
  }
}

// per-expert combine (moe/merge_expert_result.cu:3-115): one block per expert row
__global__ void __launch_bounds__(ROW_THREADS)
merge_expert_result_kernel(int n_rows, int dim_vec, int top_k, const uint4 *__restrict__ zone, int expert_id,
                           const int *__restrict__ cumsum_incl, const int *__restrict__ expert_mapping,
                           const float *__restrict__ weights, const uint16_t *__restrict__ chosen,
                           uint4 *__restrict__ X_combined) {
  const int base = cumsum_incl[expert_id] - n_rows;
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const int t = expert_mapping[base + r];
    float w = 1.0f;
    if (weights) {
      w = 0.0f;
      for (int j = 0; j < top_k; j++)
        if (chosen[(int64_t)t * top_k + j] == (uint16_t)expert_id) {
          w = weights[(int64_t)t * top_k + j];
          break;
        }
    }
    if (w == 0.0f) continue;
    const uint4 *src = zone + (int64_t)r * dim_vec;
    uint4 *out = X_combined + (int64_t)t * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += ROW_THREADS) {
      float a[8], f[8];
      unpack8(out[c], a);
      unpack8(ld_stream(src + c), f);
#pragma unroll
      for (int q = 0; q < 8; q++) a[q] += w * f[q];
      out[c] = pack8(a);
    }
  }
}

// ---------------------------------------------------------------------------------------
// router_bwd_x, one expert (moe/router_bwd_x.cu:4-92). One block per expert row:
// dot(expert_out[r,:], dOut[t,:]) -> dX_routed[t, e]; then the row is overwritten with
// dOut[t,:] * w. expert_out and dX_expert_out may alias: the row is read completely
// (block-wide reduction) before it is written.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
router_bwd_x_kernel(int n_rows, int dim_vec, int E, int top_k, int expert_id,
                    const int *__restrict__ cumsum_incl, const int *__restrict__ expert_mapping,
                    const uint16_t *__restrict__ chosen, const float *__restrict__ weights,
                    const uint4 *expert_out, const uint4 *__restrict__ upstream_dX,
                    __nv_bfloat16 *__restrict__ dX_routed, uint4 *dX_expert_out) {
  __shared__ float warp_part[8];
  const int base = cumsum_incl[expert_id] - n_rows;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const int t = expert_mapping[base + r];
    const uint4 *y = expert_out + (int64_t)r * dim_vec;
    const uint4 *g = upstream_dX + (int64_t)t * dim_vec;
    float part = 0.f;
    for (int c = threadIdx.x; c < dim_vec; c += 256) {
      float a[8], b[8];
      unpack8(y[c], a);
      unpack8(g[c], b);
#pragma unroll
      for (int q = 0; q < 8; q++) part += a[q] * b[q];
    }
    part = warp_sum(part);
    __syncthreads();  // previous iteration's readers of warp_part are done
    if (lane == 0) warp_part[warp] = part;
    __syncthreads();
    float w = 0.f;
    for (int j = 0; j < top_k; j++)
      if (chosen[(int64_t)t * top_k + j] == (uint16_t)expert_id) {
        w = weights[(int64_t)t * top_k + j];
        break;
      }
    if (threadIdx.x == 0) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) dot += warp_part[i];
      dX_routed[(int64_t)t * E + expert_id] = __float2bfloat16_rn(dot);
    }
    if (w != 0.f) {
      uint4 *o = dX_expert_out + (int64_t)r * dim_vec;
      for (int c = threadIdx.x; c < dim_vec; c += 256) {
        float b[8];
        unpack8(g[c], b);
#pragma unroll
        for (int q = 0; q < 8; q++) b[q] *= w;
        o[c] = pack8(b);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU forward / backward (activations/swiglu.cu:66-151, swiglu_bwd_x.cu:111-256)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_kernel(int64_t n_vec, const uint4 *x1, const uint4 *x3, uint4 *out) {  // out may alias an input
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    float a[8], b[8];
    unpack8(x1[i], a);
    unpack8(x3[i], b);
#pragma unroll
    for (int q = 0; q < 8; q++) a[q] = (a[q] / (1.0f + __expf(-a[q]))) * b[q];
    out[i] = pack8(a);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(int64_t n_vec, const uint4 *x1, const uint4 *x3, const uint4 *dy, uint4 *dx1,
                  uint4 *dx3) {  // outputs may alias inputs
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    float a[8], b[8], g[8], o1[8], o3[8];
    unpack8(x1[i], a);
    unpack8(x3[i], b);
    unpack8(dy[i], g);
#pragma unroll
    for (int q = 0; q < 8; q++) {
      const float s = 1.0f / (1.0f + __expf(-a[q]));
      o3[q] = g[q] * (a[q] * s);
      o1[q] = g[q] * b[q] * (s + a[q] * (s * (1.0f - s)));
    }
    dx1[i] = pack8(o1);
    dx3[i] = pack8(o3);
  }
}

}  // namespace b200

using namespace b200;

static int rows_ok(const char *op, int dim, const void *a, const void *b, const void *c = nullptr) {
  B200_REQUIRE(dim > 0 && dim % 8 == 0, "%s: row length must be a positive multiple of 8 (got %d)", op, dim);
  B200_REQUIRE(b200_aligned16(a) && b200_aligned16(b) && b200_aligned16(c), "%s: row buffers must be 16-byte aligned",
               op);
  return 0;
}

static int launch_prepare(int total_tokens, int model_dim, int top_k, const void *X, const int *token_mapping,
                          const float *weights, void *expert_zone, void *stream) {
  B200_REQUIRE(total_tokens >= 0 && top_k >= 1 && top_k <= B200_MAX_TOP_K, "prepare_experts: need 1 <= top_k <= %d",
               B200_MAX_TOP_K);
  B200_REQUIRE(X && token_mapping && expert_zone, "prepare_experts: null buffer");
  if (rows_ok("prepare_experts", model_dim, X, expert_zone)) return -1;
  if (total_tokens == 0) return 0;
  const int dv = model_dim / 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (dv <= ROW_THREADS * 2)
    prepare_experts_kernel<2><<<total_tokens, ROW_THREADS, 0, s>>>(total_tokens, dv, top_k, (const uint4 *)X,
                                                                   token_mapping, weights, (uint4 *)expert_zone);
  else
    prepare_experts_kernel<4><<<total_tokens, ROW_THREADS, 0, s>>>(total_tokens, dv, top_k, (const uint4 *)X,
                                                                   token_mapping, weights, (uint4 *)expert_zone);
  B200_CHECK_LAUNCH("prepare_experts");
  return 0;
}

extern "C" int b200_prepare_experts(int total_tokens, int model_dim, int num_selected_experts, const void *X,
                                    const int *token_mapping, void *expert_zone, void *stream) {
  return launch_prepare(total_tokens, model_dim, num_selected_experts, X, token_mapping, nullptr, expert_zone, stream);
}

extern "C" int b200_prepare_experts_weighted(int total_tokens, int model_dim, int num_selected_experts, const void *X,
                                             const int *token_mapping, const float *token_expert_weights,
                                             void *expert_zone, void *stream) {
  B200_REQUIRE(token_expert_weights, "prepare_experts_weighted: null weights");
  return launch_prepare(total_tokens, model_dim, num_selected_experts, X, token_mapping, token_expert_weights,
                        expert_zone, stream);
}

extern "C" int b200_prepare_expert_zone(int model_dim, const void *X, int expert_id, const int *expert_counts,
                                        const int *expert_counts_cumsum, const int *expert_mapping,
                                        void *expert_zone, void *stream) {
  B200_REQUIRE(expert_id >= 0 && X && expert_counts && expert_counts_cumsum && expert_mapping && expert_zone,
               "prepare_expert_zone: bad arguments");
  if (rows_ok("prepare_expert_zone", model_dim, X, expert_zone)) return -1;
  int sms = 148;
  b200_device_info(&sms, nullptr, nullptr);
  prepare_expert_zone_kernel<<<sms * 8, ROW_THREADS, 0, (cudaStream_t)stream>>>(
      model_dim / 8, (const uint4 *)X, expert_id, expert_counts, expert_counts_cumsum, expert_mapping,
      (uint4 *)expert_zone);
  B200_CHECK_LAUNCH("prepare_expert_zone");
  return 0;
}

template <bool OVERWRITE>
static int merge_experts_launch(const char *op, int num_tokens, int model_dim, int top_k_experts, const void *expert_zones,
                                const int *token_mapping, const float *token_expert_weights, void *X_combined,
                                void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k_experts >= 1 && top_k_experts <= B200_MAX_TOP_K, "%s: need 1 <= top_k <= %d", op,
               B200_MAX_TOP_K);
  B200_REQUIRE(expert_zones && token_mapping && X_combined, "%s: null buffer", op);
  if (rows_ok(op, model_dim, expert_zones, X_combined)) return -1;
  if (num_tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int dv = model_dim / 8;
  if (top_k_experts >= 8)
    merge_experts_kernel<8, OVERWRITE><<<num_tokens, ROW_THREADS, 0, s>>>(num_tokens, dv, top_k_experts, (const uint4 *)expert_zones,
                                                                          token_mapping, token_expert_weights, (uint4 *)X_combined);
  else if (top_k_experts >= 4)
    merge_experts_kernel<4, OVERWRITE><<<num_tokens, ROW_THREADS, 0, s>>>(num_tokens, dv, top_k_experts, (const uint4 *)expert_zones,
                                                                          token_mapping, token_expert_weights, (uint4 *)X_combined);
  else
    merge_experts_kernel<2, OVERWRITE><<<num_tokens, ROW_THREADS, 0, s>>>(num_tokens, dv, top_k_experts, (const uint4 *)expert_zones,
                                                                          token_mapping, token_expert_weights, (uint4 *)X_combined);
  B200_CHECK_LAUNCH(op);
  return 0;
}

extern "C" int b200_merge_experts(int num_tokens, int model_dim, int top_k_experts, const void *expert_zones,
                                  const int *token_mapping, const float *token_expert_weights, void *X_combined,
                                  void *stream) {
  return merge_experts_launch<false>("merge_experts", num_tokens, model_dim, top_k_experts, expert_zones, token_mapping,
                                     token_expert_weights, X_combined, stream);
}

extern "C" int b200_unpermute_experts(int num_tokens, int model_dim, int top_k_experts, const void *expert_zones,
                                      const int *token_mapping, void *X_out, void *stream) {
  return merge_experts_launch<true>("unpermute_experts", num_tokens, model_dim, top_k_experts, expert_zones, token_mapping,
                                    nullptr, X_out, stream);
}

extern "C" int b200_merge_expert_result(int num_tokens, int model_dim, int top_k_experts, const void *expert_zone,
                                        int expert_id, const int *expert_counts_cumsum, const int *expert_mapping,
                                        const float *token_expert_weights, const uint16_t *chosen_experts,
                                        void *X_combined, void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k_experts >= 1 && expert_id >= 0, "merge_expert_result: bad sizes");
  B200_REQUIRE(expert_zone && expert_counts_cumsum && expert_mapping && X_combined &&
                   (!token_expert_weights || chosen_experts),
               "merge_expert_result: null buffer");
  if (rows_ok("merge_expert_result", model_dim, expert_zone, X_combined)) return -1;
  if (num_tokens == 0) return 0;
  merge_expert_result_kernel<<<num_tokens, ROW_THREADS, 0, (cudaStream_t)stream>>>(
      num_tokens, model_dim / 8, top_k_experts, (const uint4 *)expert_zone, expert_id, expert_counts_cumsum,
      expert_mapping, token_expert_weights, chosen_experts, (uint4 *)X_combined);
  B200_CHECK_LAUNCH("merge_expert_result");
  return 0;
}

extern "C" int b200_router_bwd_x(int num_expert_tokens, int model_dim, int num_routed_experts, int top_k_active,
                                 int expert_id, const int *expert_counts_cumsum, const int *expert_mapping,
                                 const uint16_t *chosen_experts, const float *token_expert_weights,
                                 const void *expert_out, const void *upstream_dX, void *dX_routed,
                                 void *dX_expert_out, void *stream) {
  B200_REQUIRE(num_expert_tokens >= 0 && num_routed_experts >= 1 && top_k_active >= 1 && expert_id >= 0 &&
                   expert_id < num_routed_experts,
               "router_bwd_x: bad sizes");
  B200_REQUIRE(expert_counts_cumsum && expert_mapping && chosen_experts && token_expert_weights && expert_out &&
                   upstream_dX && dX_routed && dX_expert_out,
               "router_bwd_x: null buffer");
  if (rows_ok("router_bwd_x", model_dim, expert_out, upstream_dX, dX_expert_out)) return -1;
  if (num_expert_tokens == 0) return 0;
  router_bwd_x_kernel<<<num_expert_tokens, 256, 0, (cudaStream_t)stream>>>(
      num_expert_tokens, model_dim / 8, num_routed_experts, top_k_active, expert_id, expert_counts_cumsum,
      expert_mapping, chosen_experts, token_expert_weights, (const uint4 *)expert_out, (const uint4 *)upstream_dX,
      (__nv_bfloat16 *)dX_routed, (uint4 *)dX_expert_out);
  B200_CHECK_LAUNCH("router_bwd_x");
  return 0;
}

static int elementwise_grid(int64_t n_vec) {
  int64_t blocks = (n_vec + 255) / 256;
  const int64_t cap = 148 * 16;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

extern "C" int b200_swiglu(int num_rows, int num_cols, const void *x_w1, const void *x_w3, void *out, void *stream) {
  B200_REQUIRE(num_rows >= 0 && x_w1 && x_w3 && out, "swiglu: bad arguments");
  if (rows_ok("swiglu", num_cols, x_w1, x_w3, out)) return -1;
  const int64_t n_vec = (int64_t)num_rows * (num_cols / 8);
  if (n_vec == 0) return 0;
  swiglu_kernel<<<elementwise_grid(n_vec), 256, 0, (cudaStream_t)stream>>>(n_vec, (const uint4 *)x_w1,
                                                                           (const uint4 *)x_w3, (uint4 *)out);
  B200_CHECK_LAUNCH("swiglu");
  return 0;
}

extern "C" int b200_swiglu_bwd_x(int num_rows, int num_cols, const void *x_w1, const void *x_w3,
                                 const void *upstream_dX, void *dX_w1, void *dX_w3, void *stream) {
  B200_REQUIRE(num_rows >= 0 && x_w1 && x_w3 && upstream_dX && dX_w1 && dX_w3, "swiglu_bwd_x: bad arguments");
  if (rows_ok("swiglu_bwd_x", num_cols, x_w1, x_w3, upstream_dX) || rows_ok("swiglu_bwd_x", num_cols, dX_w1, dX_w3))
    return -1;
  const int64_t n_vec = (int64_t)num_rows * (num_cols / 8);
  if (n_vec == 0) return 0;
  swiglu_bwd_kernel<<<elementwise_grid(n_vec), 256, 0, (cudaStream_t)stream>>>(
      n_vec, (const uint4 *)x_w1, (const uint4 *)x_w3, (const uint4 *)upstream_dX, (uint4 *)dX_w1, (uint4 *)dX_w3);
  B200_CHECK_LAUNCH("swiglu_bwd_x");
  return 0;
}
