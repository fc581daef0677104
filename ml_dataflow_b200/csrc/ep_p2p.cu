// Expert-parallel row movement over NVLink peer memory: the gather that builds the expert zones writes every row
// straight into the buffer of the GPU that owns the expert (peer stores), and the combine reads every expert
// output row straight from its owner (peer loads). No staging buffer, no second copy, no collective on the data
// path; the callers order the phases with a stream-ordered barrier. Plain ld/st only: no TMA, no multicast.
//
// Addressing. Rank g owns experts [g*E_loc, (g+1)*E_loc). In the owner's buffer the rows of expert e are laid out
// source rank by source rank; dst_base[e] is the first row (in the OWNER's buffer) of the block that holds THIS
// rank's rows of expert e. A routed pair (t, j) with local zone row r = token_mapping[t, j] and expert
// e = chosen[t, j] therefore lives at row dst_base[e] + (r - first_local_row[e]) of rank e / E_loc.
#include "common.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

constexpr int P2P_THREADS = 128;
constexpr int P2P_MAX_RANKS = 16;

struct PeerTable {
  unsigned long long base[P2P_MAX_RANKS];  // device address of every rank's buffer, as mapped into this process
};

struct RouteView {
  const int *token_mapping;
  const uint16_t *chosen;
  const int *counts, *cumsum_incl, *dst_base;
  int num_experts, experts_per_rank;
  int local_begin, local_end;  // only pairs whose expert index inside its owner is in [local_begin, local_end)
  int64_t capacity_rows;       // rows every rank's buffer holds: a pair whose row would lie past it is skipped
};

__device__ __forceinline__ bool locate(const RouteView &rv, int64_t slot, int &owner, int64_t &row) {
  const int e = rv.chosen[slot];
  const int r = rv.token_mapping[slot];
  if (e >= rv.num_experts || r < 0) return false;
  owner = e / rv.experts_per_rank;
  const int le = e - owner * rv.experts_per_rank;
  if (le < rv.local_begin || le >= rv.local_end) return false;
  row = (int64_t)rv.dst_base[e] + (r - (rv.cumsum_incl[e] - rv.counts[e]));
  return row >= 0 && row < rv.capacity_rows;
}

// X[t, :] (optionally scaled by the gate weight) -> row (t, j) in its owner's buffer
template <int VPT>
__global__ void __launch_bounds__(P2P_THREADS)
dispatch_rows_kernel(int total_tokens, int dim_vec, int top_k, const uint4 *__restrict__ X,
                     const float *__restrict__ weights, RouteView rv, PeerTable peers) {
  __shared__ unsigned long long dst_ptr[B200_MAX_TOP_K];
  __shared__ float dst_w[B200_MAX_TOP_K];
  for (int64_t token = blockIdx.x; token < total_tokens; token += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < top_k) {
      int owner;
      int64_t row;
      const int64_t slot = token * top_k + threadIdx.x;
      dst_ptr[threadIdx.x] = locate(rv, slot, owner, row) ? peers.base[owner] + (unsigned long long)row * dim_vec * 16ull : 0ull;
      dst_w[threadIdx.x] = weights ? weights[slot] : 1.0f;
    }
    __syncthreads();
    const uint4 *src = X + token * dim_vec;
    for (int c0 = 0; c0 < dim_vec; c0 += P2P_THREADS * VPT) {
      uint4 v[VPT];
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int c = c0 + i * P2P_THREADS + threadIdx.x;
        if (c < dim_vec) v[i] = ld_stream(src + c);
      }
      for (int j = 0; j < top_k; j++) {
        if (dst_ptr[j] == 0ull) continue;
        uint4 *dst = reinterpret_cast<uint4 *>(dst_ptr[j]);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int c = c0 + i * P2P_THREADS + threadIdx.x;
          if (c < dim_vec) {
            if (weights) {
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

// X_combined[t,:] = bf16(f32(X_combined[t,:]) + sum_j w[t,j] * row(t,j) read from its owner)
template <int KU>
__global__ void __launch_bounds__(P2P_THREADS)
combine_rows_kernel(int num_tokens, int dim_vec, int top_k, const float *__restrict__ weights, RouteView rv,
                    PeerTable peers, uint4 *__restrict__ X_combined) {
  __shared__ unsigned long long src_ptr[B200_MAX_TOP_K];
  __shared__ float wts[B200_MAX_TOP_K];
  for (int64_t token = blockIdx.x; token < num_tokens; token += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < top_k) {
      int owner;
      int64_t row;
      const int64_t slot = token * top_k + threadIdx.x;
      src_ptr[threadIdx.x] = locate(rv, slot, owner, row) ? peers.base[owner] + (unsigned long long)row * dim_vec * 16ull : 0ull;
      wts[threadIdx.x] = weights ? weights[slot] : 1.0f;
    }
    __syncthreads();
    uint4 *out = X_combined + token * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += P2P_THREADS) {
      float acc[8];
      unpack8(out[c], acc);
      for (int j0 = 0; j0 < top_k; j0 += KU) {
        uint4 v[KU];
#pragma unroll
        for (int u = 0; u < KU; u++) {
          const int j = j0 + u;
          const unsigned long long sp = (j < top_k) ? src_ptr[j] : 0ull;
          v[u] = sp ? ld_stream(reinterpret_cast<const uint4 *>(sp) + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < KU; u++) {
          const int j = j0 + u;
          if (j < top_k && src_ptr[j]) {
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

// dX_routed[t, chosen[t,j]] = bf16(dP_owner[row(t,j)] / w[t,j]); dP holds w * <Y, dOut> per routed row
__global__ void router_grad_p2p_kernel(int64_t n, int top_k, const float *__restrict__ weights, RouteView rv,
                                       PeerTable peers, __nv_bfloat16 *__restrict__ dX_routed) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int owner;
  int64_t row;
  if (!locate(rv, i, owner, row)) return;
  const float w = weights[i];
  const float v = *(reinterpret_cast<const float *>(peers.base[owner]) + row);
  dX_routed[(i / top_k) * rv.num_experts + rv.chosen[i]] = __float2bfloat16_rn(w != 0.f ? v / w : 0.f);
}

// tags_owner[row(t,j)] = (my_rank << 40) | local zone row of (t, j): tells the owner's GEMM epilogue where the
// output row of that routed pair has to go (b200_moe_experts_fwd_scatter / _bwd_x_scatter)
__global__ void publish_row_tags_kernel(int64_t n, unsigned long long my_rank, RouteView rv, PeerTable peers) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int owner;
  int64_t row;
  if (!locate(rv, i, owner, row)) return;
  *(reinterpret_cast<unsigned long long *>(peers.base[owner]) + row) =
      (my_rank << 40) | (unsigned long long)rv.token_mapping[i];
}

}  // namespace b200

using namespace b200;

static int fill_views(const char *op, int num_experts, int experts_per_rank, int world, const int *token_mapping,
                      const uint16_t *chosen, const int *counts, const int *cumsum, const int *dst_base,
                      const unsigned long long *peer_ptrs, int64_t capacity_rows, RouteView &rv, PeerTable &pt) {
  B200_REQUIRE(capacity_rows >= 0, "%s: negative buffer capacity", op);
  B200_REQUIRE(num_experts >= 1 && experts_per_rank >= 1 && world >= 1 && world <= P2P_MAX_RANKS &&
                   experts_per_rank * world == num_experts,
               "%s: need experts_per_rank * world == num_experts and world <= %d (got %d, %d, %d)", op, P2P_MAX_RANKS,
               experts_per_rank, world, num_experts);
  B200_REQUIRE(token_mapping && chosen && counts && cumsum && dst_base && peer_ptrs, "%s: null routing table", op);
  rv.token_mapping = token_mapping;
  rv.chosen = chosen;
  rv.counts = counts;
  rv.cumsum_incl = cumsum;
  rv.dst_base = dst_base;
  rv.num_experts = num_experts;
  rv.experts_per_rank = experts_per_rank;
  rv.local_begin = 0;
  rv.local_end = experts_per_rank;
  rv.capacity_rows = capacity_rows;
  for (int i = 0; i < P2P_MAX_RANKS; i++) pt.base[i] = i < world ? peer_ptrs[i] : 0ull;
  for (int i = 0; i < world; i++) B200_REQUIRE(pt.base[i] != 0 && (pt.base[i] & 15ull) == 0, "%s: bad peer pointer %d", op, i);
  return 0;
}

extern "C" int b200_ep_dispatch_rows(int total_tokens, int model_dim, int top_k, const void *X,
                                     const float *token_expert_weights, const int *token_mapping,
                                     const uint16_t *chosen_experts, const int *expert_counts,
                                     const int *expert_counts_cumsum, const int *dst_base,
                                     const unsigned long long *peer_buffers, int world, int num_experts,
                                     int experts_per_rank, int64_t capacity_rows, int local_expert_begin,
                                     int local_expert_end, void *stream) {
  B200_REQUIRE(total_tokens >= 0 && top_k >= 1 && top_k <= B200_MAX_TOP_K && model_dim > 0 && model_dim % 8 == 0 && X &&
                   b200_aligned16(X),
               "ep_dispatch_rows: bad arguments");
  B200_REQUIRE(0 <= local_expert_begin && local_expert_begin <= local_expert_end && local_expert_end <= experts_per_rank,
               "ep_dispatch_rows: local expert range [%d, %d) outside [0, %d)", local_expert_begin, local_expert_end,
               experts_per_rank);
  RouteView rv;
  PeerTable pt;
  if (fill_views("ep_dispatch_rows", num_experts, experts_per_rank, world, token_mapping, chosen_experts, expert_counts,
                 expert_counts_cumsum, dst_base, peer_buffers, capacity_rows, rv, pt))
    return -1;
  rv.local_begin = local_expert_begin;
  rv.local_end = local_expert_end;
  if (total_tokens == 0 || local_expert_begin == local_expert_end) return 0;
  const int dv = model_dim / 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (dv <= P2P_THREADS * 2)
    dispatch_rows_kernel<2><<<total_tokens, P2P_THREADS, 0, s>>>(total_tokens, dv, top_k, (const uint4 *)X,
                                                                 token_expert_weights, rv, pt);
  else
    dispatch_rows_kernel<4><<<total_tokens, P2P_THREADS, 0, s>>>(total_tokens, dv, top_k, (const uint4 *)X,
                                                                 token_expert_weights, rv, pt);
  B200_CHECK_LAUNCH("ep_dispatch_rows");
  return 0;
}

extern "C" int b200_ep_combine_rows(int num_tokens, int model_dim, int top_k, const float *token_expert_weights,
                                    const int *token_mapping, const uint16_t *chosen_experts, const int *expert_counts,
                                    const int *expert_counts_cumsum, const int *dst_base,
                                    const unsigned long long *peer_buffers, int world, int num_experts,
                                    int experts_per_rank, int64_t capacity_rows, void *X_combined, void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k >= 1 && top_k <= B200_MAX_TOP_K && model_dim > 0 && model_dim % 8 == 0 &&
                   X_combined && b200_aligned16(X_combined),
               "ep_combine_rows: bad arguments");
  RouteView rv;
  PeerTable pt;
  if (fill_views("ep_combine_rows", num_experts, experts_per_rank, world, token_mapping, chosen_experts, expert_counts,
                 expert_counts_cumsum, dst_base, peer_buffers, capacity_rows, rv, pt))
    return -1;
  if (num_tokens == 0) return 0;
  const int dv = model_dim / 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (top_k >= 8)
    combine_rows_kernel<8><<<num_tokens, P2P_THREADS, 0, s>>>(num_tokens, dv, top_k, token_expert_weights, rv, pt, (uint4 *)X_combined);
  else if (top_k >= 4)
    combine_rows_kernel<4><<<num_tokens, P2P_THREADS, 0, s>>>(num_tokens, dv, top_k, token_expert_weights, rv, pt, (uint4 *)X_combined);
  else
    combine_rows_kernel<2><<<num_tokens, P2P_THREADS, 0, s>>>(num_tokens, dv, top_k, token_expert_weights, rv, pt, (uint4 *)X_combined);
  B200_CHECK_LAUNCH("ep_combine_rows");
  return 0;
}

extern "C" int b200_ep_gather_router_grad(int num_tokens, int top_k, const float *token_expert_weights,
                                          const int *token_mapping, const uint16_t *chosen_experts,
                                          const int *expert_counts, const int *expert_counts_cumsum, const int *dst_base,
                                          const unsigned long long *peer_dP_buffers, int world, int num_experts,
                                          int experts_per_rank, int64_t capacity_rows, void *dX_routed,
                                          void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k >= 1 && token_expert_weights && dX_routed, "ep_gather_router_grad: bad arguments");
  RouteView rv;
  PeerTable pt;
  if (fill_views("ep_gather_router_grad", num_experts, experts_per_rank, world, token_mapping, chosen_experts,
                 expert_counts, expert_counts_cumsum, dst_base, peer_dP_buffers, capacity_rows, rv, pt))
    return -1;
  const int64_t n = (int64_t)num_tokens * top_k;
  if (n == 0) return 0;
  router_grad_p2p_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      n, top_k, token_expert_weights, rv, pt, (__nv_bfloat16 *)dX_routed);
  B200_CHECK_LAUNCH("ep_gather_router_grad");
  return 0;
}

extern "C" int b200_ep_publish_row_tags(int num_tokens, int top_k, int my_rank, const int *token_mapping,
                                        const uint16_t *chosen_experts, const int *expert_counts,
                                        const int *expert_counts_cumsum, const int *dst_base,
                                        const unsigned long long *peer_tag_buffers, int world, int num_experts,
                                        int experts_per_rank, int64_t capacity_rows, void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k >= 1 && my_rank >= 0 && my_rank < world, "ep_publish_row_tags: bad arguments");
  RouteView rv;
  PeerTable pt;
  if (fill_views("ep_publish_row_tags", num_experts, experts_per_rank, world, token_mapping, chosen_experts,
                 expert_counts, expert_counts_cumsum, dst_base, peer_tag_buffers, capacity_rows, rv, pt))
    return -1;
  const int64_t n = (int64_t)num_tokens * top_k;
  if (n == 0) return 0;
  publish_row_tags_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, (unsigned long long)my_rank,
                                                                                        rv, pt);
  B200_CHECK_LAUNCH("ep_publish_row_tags");
  return 0;
}
