// Expert-parallel MoE layer driven from C: the op sequence of one rank, forward and backward, with no collective
// library on the path. Everything the ranks tell one another travels through buffers that are mapped into every
// rank over NVLink (the caller allocates them and hands in the peer addresses):
//   * the barrier between phases is a kernel: every rank stores a rising epoch number into its slot of every peer's
//     flag array and waits, with a time limit, until all its own slots have reached that epoch; a small payload (the
//     per-expert row counts) can ride on it, stored into the peers just before the flag;
//   * the exchange plan (per-expert receive counts and offsets) is one kernel over the gathered counts;
//   * rows go out through b200_ep_dispatch_rows and come home through the epilogue of the last GEMM of each pass;
//   * the router weight gradient is summed over the ranks by reading every peer's partial result in rank order.
// The reference is single-GPU (its MoE_Config.num_local_experts / local_expert_inds,
// libdataflowmodels/include/dataflow_models.h:51-67, are placeholders), so there is no reference sequence to follow
// beyond the per-token maths, which is that of b200_moe_block_fwd / _bwd.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

constexpr int EP_MAX_RANKS = 16;

struct EpPeers {
  unsigned long long p[EP_MAX_RANKS];
};

__device__ int g_ep_status = 0;  // 1 = a barrier wait ran out of time

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One block. flags[r] of every rank's flag array is written by rank r only. payload (optional): payload_ints ints of
// this rank go to offset rank * payload_ints of every peer's payload array before the flag is raised.
__global__ void __launch_bounds__(256)
ep_barrier_kernel(EpPeers flag_peers, int world, int rank, unsigned int *epoch, unsigned long long limit_ns,
                  const int *payload, int payload_ints, EpPeers payload_peers, int *status) {
  __shared__ unsigned int target;
  if (threadIdx.x == 0) target = *epoch + 1u;
  __syncthreads();
  const unsigned int e = target;
  if (payload != nullptr) {
    for (int i = threadIdx.x; i < world * payload_ints; i += blockDim.x) {
      const int r = i / payload_ints, j = i - r * payload_ints;
      reinterpret_cast<int *>(payload_peers.p[r])[(int64_t)rank * payload_ints + j] = payload[j];
    }
  }
  __threadfence_system();  // this rank's earlier stores (payload, and rows stored by earlier kernels) before the flag
  __syncthreads();
  if (threadIdx.x < world) {
    st_release_sys(reinterpret_cast<unsigned int *>(flag_peers.p[threadIdx.x]) + rank, e);
    const unsigned int *mine = reinterpret_cast<const unsigned int *>(flag_peers.p[rank]) + threadIdx.x;
    const unsigned long long t0 = ptx::globaltimer_ns();
    unsigned int polls = 0;
    // a peer may already be one barrier ahead, never behind: compare as a signed distance
    while ((int)(ld_acquire_sys(mine) - e) < 0) {
      if ((++polls & 255u) == 0 && ptx::globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, 1);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x == 0) *epoch = e;
}

// gathered[s][h][j]: rows rank s sends to local expert j of rank h. For this rank: counts of its local experts summed
// over the sources and their inclusive prefix sums, both clipped so that nothing reaches past the receive capacity;
// dst_base[e] = first row, in the owner's buffer, of THIS rank's rows of global expert e (source-major inside an
// expert); overflow[0] |= 1 when this rank's buffer would need more than the capacity.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int *__restrict__ gathered, int world, int rank, int experts_per_rank, long long capacity,
               int *__restrict__ local_counts, int *__restrict__ local_cumsum, int *__restrict__ dst_base,
               int *__restrict__ overflow) {
  const int E = world * experts_per_rank;
  // dst_base: one thread per global expert e = (h, j): sum over experts before j of owner h (all sources) + the
  // rows of lower source ranks for (h, j)
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int h = e / experts_per_rank, j = e - h * experts_per_rank;
    long long base = 0;
    for (int jj = 0; jj < j; jj++)
      for (int s = 0; s < world; s++) base += gathered[((int64_t)s * world + h) * experts_per_rank + jj];
    for (int s = 0; s < rank; s++) base += gathered[((int64_t)s * world + h) * experts_per_rank + j];
    dst_base[e] = (int)min(base, (long long)INT_MAX);
  }
  if (threadIdx.x == 0) {
    long long run = 0, prev = 0;
    for (int j = 0; j < experts_per_rank; j++) {
      for (int s = 0; s < world; s++) run += gathered[((int64_t)s * world + rank) * experts_per_rank + j];
      const long long clipped = min(run, capacity);
      local_cumsum[j] = (int)clipped;
      local_counts[j] = (int)(clipped - prev);
      prev = clipped;
    }
    if (run > capacity) overflow[0] = 1;
  }
}

// dWr[i] = bf16(f32(dWr[i]) + sum over ranks (in rank order) of peer_partial[r][i]); n a multiple of 8
__global__ void ep_reduce_router_grad_kernel(EpPeers partials, int world, int64_t n_vec, uint4 *__restrict__ dWr) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  float acc[8];
  unpack8(dWr[i], acc);
  for (int r = 0; r < world; r++) {
    float f[8];
    unpack8(ld_stream(reinterpret_cast<const uint4 *>(partials.p[r]) + i), f);
#pragma unroll
    for (int q = 0; q < 8; q++) acc[q] += f[q];
  }
  dWr[i] = pack8(acc);
}

}  // namespace b200

using namespace b200;

static unsigned long long g_ep_barrier_limit_ns = 2ull * 1000ull * 1000ull * 1000ull;

static int *ep_status_ptr() {
  static int *ptr[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev] && cudaGetSymbolAddress((void **)&ptr[dev], g_ep_status) != cudaSuccess) ptr[dev] = nullptr;
  return ptr[dev];
}

static int fill_peers(const char *op, const unsigned long long *host_table, int world, EpPeers &out, unsigned align) {
  B200_REQUIRE(host_table != nullptr && world >= 1 && world <= EP_MAX_RANKS, "%s: bad peer table (world %d, at most %d)",
               op, world, EP_MAX_RANKS);
  for (int i = 0; i < EP_MAX_RANKS; i++) out.p[i] = i < world ? host_table[i] : 0ull;
  for (int i = 0; i < world; i++)
    B200_REQUIRE(out.p[i] != 0 && (out.p[i] & (align - 1)) == 0, "%s: peer address %d missing or unaligned", op, i);
  return 0;
}

extern "C" int b200_ep_set_barrier_timeout_ms(int ms) {
  B200_REQUIRE(ms >= 1, "ep_set_barrier_timeout_ms: need at least 1 ms");
  g_ep_barrier_limit_ns = (unsigned long long)ms * 1000000ull;
  return 0;
}

extern "C" int b200_ep_status(int *status_out) {
  int v = 0;
  B200_CUDA(cudaDeviceSynchronize());
  B200_CUDA(cudaMemcpyFromSymbol(&v, g_ep_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    B200_CUDA(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(int)));
  }
  if (status_out) *status_out = v;
  return 0;
}

extern "C" int b200_ep_barrier(const unsigned long long *peer_flags, int world, int rank, unsigned int *epoch,
                               const int *payload, int payload_ints, const unsigned long long *peer_payload,
                               void *stream) {
  B200_REQUIRE(rank >= 0 && rank < world && epoch != nullptr, "ep_barrier: bad rank %d of %d, or no epoch word", rank, world);
  EpPeers flags, pay;
  memset(&pay, 0, sizeof(pay));
  if (fill_peers("ep_barrier", peer_flags, world, flags, 4)) return -1;
  if (payload != nullptr) {
    B200_REQUIRE(payload_ints >= 1 && payload_ints <= 65536, "ep_barrier: bad payload length %d", payload_ints);
    if (fill_peers("ep_barrier (payload)", peer_payload, world, pay, 4)) return -1;
  }
  int *status = ep_status_ptr();
  B200_REQUIRE(status != nullptr, "ep_barrier: status word unavailable");
  ep_barrier_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(flags, world, rank, epoch, g_ep_barrier_limit_ns, payload,
                                                        payload ? payload_ints : 0, pay, status);
  B200_CHECK_LAUNCH("ep_barrier");
  return 0;
}

extern "C" int b200_ep_plan(const int *gathered_counts, int world, int rank, int experts_per_rank,
                            int64_t capacity_rows, int *local_counts, int *local_cumsum, int *dst_base, int *overflow,
                            void *stream) {
  B200_REQUIRE(gathered_counts && local_counts && local_cumsum && dst_base && overflow, "ep_plan: null buffer");
  B200_REQUIRE(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world && experts_per_rank >= 1 &&
                   capacity_rows >= 0 && capacity_rows <= INT_MAX,
               "ep_plan: bad arguments (world %d, rank %d, %d experts per rank)", world, rank, experts_per_rank);
  ep_plan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(gathered_counts, world, rank, experts_per_rank,
                                                      (long long)capacity_rows, local_counts, local_cumsum, dst_base,
                                                      overflow);
  B200_CHECK_LAUNCH("ep_plan");
  return 0;
}

extern "C" int b200_ep_reduce_router_grad(const unsigned long long *peer_partials, int world, int64_t num_elements,
                                          void *dWr, void *stream) {
  B200_REQUIRE(dWr && b200_aligned16(dWr) && num_elements >= 0 && num_elements % 8 == 0,
               "ep_reduce_router_grad: dWr must be 16-byte aligned and hold a multiple of 8 elements");
  EpPeers parts;
  if (fill_peers("ep_reduce_router_grad", peer_partials, world, parts, 16)) return -1;
  const int64_t n_vec = num_elements / 8;
  if (n_vec == 0) return 0;
  ep_reduce_router_grad_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, (cudaStream_t)stream>>>(parts, world, n_vec,
                                                                                                (uint4 *)dWr);
  B200_CHECK_LAUNCH("ep_reduce_router_grad");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// The layer
// ---------------------------------------------------------------------------------------------------------------

static int check_ep_block(const char *op, const B200EpMoeBlock *b) {
  B200_REQUIRE(b != nullptr, "%s: null block description", op);
  B200_REQUIRE(b->world >= 1 && b->world <= EP_MAX_RANKS && b->rank >= 0 && b->rank < b->world,
               "%s: bad rank %d of %d (at most %d ranks)", op, b->rank, b->world, EP_MAX_RANKS);
  B200_REQUIRE(b->total_tokens >= 0 && b->model_dim > 0 && b->num_experts >= 1 && b->num_experts % b->world == 0 &&
                   b->top_k >= 1 && b->top_k <= b->num_experts && b->ffn_dim > 0 && b->capacity_rows >= 0,
               "%s: bad shape (T %d, d %d, E %d over %d ranks, k %d, f %d)", op, b->total_tokens, b->model_dim,
               b->num_experts, b->world, b->top_k, b->ffn_dim);
  B200_REQUIRE(b->Wr && b->W1 && b->W3 && b->W2, "%s: weight pointer missing", op);
  B200_REQUIRE(b->logits && b->token_expert_weights && b->chosen_experts && b->expert_counts && b->expert_counts_cumsum &&
                   b->expert_mapping && b->token_mapping && b->mapping_workspace,
               "%s: routing buffer missing", op);
  B200_REQUIRE(b->gathered_counts && b->local_counts && b->local_cumsum && b->dst_base && b->overflow && b->barrier_epoch,
               "%s: exchange-plan buffer missing", op);
  B200_REQUIRE(b->peer_flags && b->peer_counts && b->peer_zone && b->peer_tags && b->peer_Y_home, "%s: peer table missing", op);
  B200_REQUIRE(b->zone_recv && b->tags_recv && b->Y_home && b->x1 && b->x3 && b->h, "%s: activation buffer missing", op);
  return 0;
}

// a barrier of this block: advances the block's epoch word
static int ep_sync(const B200EpMoeBlock *b, const int *payload, int payload_ints, void *stream) {
  return b200_ep_barrier(b->peer_flags, b->world, b->rank, b->barrier_epoch, payload, payload_ints,
                         payload ? b->peer_counts : nullptr, stream);
}

extern "C" int b200_ep_moe_block_fwd(const B200EpMoeBlock *b, const void *Xn, void *X_combined, void *stream) {
  if (check_ep_block("ep_moe_block_fwd", b)) return -1;
  B200_REQUIRE(Xn && X_combined, "ep_moe_block_fwd: Xn / X_combined missing");
  const int T = b->total_tokens, d = b->model_dim, E = b->num_experts, k = b->top_k, f = b->ffn_dim;
  const int El = E / b->world;
  const int64_t cap = b->capacity_rows;
  cudaStream_t s = (cudaStream_t)stream;
  // route this rank's tokens over all E experts (global expert ids)
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_NONE, B200_DT_FP32, 1, 0, E, d, T, 1.0f, 0.0f, b->Wr, Xn, nullptr,
                  b->logits, b->matmul_workspace_bytes, b->matmul_workspace, stream))
    return -1;
  B200_CUDA(cudaMemsetAsync(b->expert_counts, 0, sizeof(int) * (size_t)(E + 1), s));
  B200_CUDA(cudaMemsetAsync(b->expert_counts_cumsum, 0, sizeof(int) * (size_t)E, s));
  if (b200_select_experts(B200_DT_FP32, T, E, k, b->logits, b->token_expert_weights, b->chosen_experts, b->expert_counts,
                          b->expert_counts_cumsum, nullptr, stream))
    return -1;
  if (b200_build_expert_mapping(T, E, k, b->chosen_experts, b->expert_counts_cumsum, b->expert_mapping, b->token_mapping,
                                b->mapping_workspace, b->mapping_workspace_bytes, stream))
    return -1;
  // counts to every rank; the same barrier orders this step after every rank's previous step (its buffers are free)
  if (ep_sync(b, b->expert_counts, E, stream)) return -1;
  if (b200_ep_plan(b->gathered_counts, b->world, b->rank, El, cap, b->local_counts, b->local_cumsum, b->dst_base,
                   b->overflow, stream))
    return -1;
  // rows (the gather IS the dispatch) and the tags that tell the owners' GEMM where each output row goes home
  if (b200_ep_dispatch_rows(T, d, k, Xn, nullptr, b->token_mapping, b->chosen_experts, b->expert_counts,
                            b->expert_counts_cumsum, b->dst_base, b->peer_zone, b->world, E, El, cap, 0, El, stream))
    return -1;
  if (b200_ep_publish_row_tags(T, k, b->rank, b->token_mapping, b->chosen_experts, b->expert_counts,
                               b->expert_counts_cumsum, b->dst_base, b->peer_tags, b->world, E, El, cap, stream))
    return -1;
  if (ep_sync(b, nullptr, 0, stream)) return -1;
  // this rank's experts over the rows of every rank; Y rows are stored straight into their home rank's buffer
  if (b200_moe_experts_fwd_scatter((int)cap, d, f, El, b->zone_recv, b->W1, b->W3, b->W2, b->w1_stride_elems,
                                   b->w3_stride_elems, b->w2_stride_elems, b->local_counts, b->local_cumsum, b->x1, b->x3,
                                   b->h, b->tags_recv, b->peer_Y_home, b->world, (int64_t)T * k, stream))
    return -1;
  if (ep_sync(b, nullptr, 0, stream)) return -1;
  return b200_merge_experts(T, d, k, b->Y_home, b->token_mapping, b->token_expert_weights, X_combined, stream);
}

extern "C" int b200_ep_moe_block_bwd(const B200EpMoeBlock *b, const void *Xn, const void *dOut, void *dXn, void *dWr,
                                     void *dW1, void *dW3, void *dW2, void *stream) {
  if (check_ep_block("ep_moe_block_bwd", b)) return -1;
  B200_REQUIRE(Xn && dOut && dXn && dWr, "ep_moe_block_bwd: Xn / dOut / dXn / dWr missing");
  B200_REQUIRE(b->peer_dY && b->peer_dP && b->peer_dZ_home && b->peer_dWr && b->dY_recv && b->dP_recv && b->dZ_home &&
                   b->dWr_partial && b->dx1 && b->dx3 && b->ones && b->dX_routed,
               "ep_moe_block_bwd: backward buffer missing");
  const int T = b->total_tokens, d = b->model_dim, E = b->num_experts, k = b->top_k, f = b->ffn_dim;
  const int El = E / b->world;
  const int64_t cap = b->capacity_rows;
  cudaStream_t s = (cudaStream_t)stream;
  B200_CUDA(cudaMemsetAsync(b->dP_recv, 0, sizeof(float) * (size_t)cap, s));
  // dY rows = w * dOut, stored straight into the owners' buffers
  if (b200_ep_dispatch_rows(T, d, k, dOut, b->token_expert_weights, b->token_mapping, b->chosen_experts, b->expert_counts,
                            b->expert_counts_cumsum, b->dst_base, b->peer_dY, b->world, E, El, cap, 0, El, stream))
    return -1;
  if (ep_sync(b, nullptr, 0, stream)) return -1;
  // the gate weight of a row lives on its home rank: accumulate w * <Y, dOut> here (row weight 1), divide there
  if (b200_moe_experts_bwd_x_scatter((int)cap, d, f, El, b->dY_recv, b->ones, b->x1, b->x3, b->W1, b->W3, b->W2,
                                     b->w1_stride_elems, b->w3_stride_elems, b->w2_stride_elems, b->local_counts,
                                     b->local_cumsum, b->dx1, b->dx3, nullptr, b->dP_recv, b->tags_recv, b->peer_dZ_home,
                                     b->world, (int64_t)T * k, stream))
    return -1;
  if (dW1 || dW3 || dW2) {
    if (b200_moe_experts_bwd_w((int)cap, d, f, El, b->dY_recv, b->h, b->zone_recv, b->dx1, b->dx3, dW1, dW3, dW2,
                               b->w1_stride_elems, b->w3_stride_elems, b->w2_stride_elems, b->local_counts, b->local_cumsum,
                               stream))
      return -1;
  }
  if (ep_sync(b, nullptr, 0, stream)) return -1;
  if (b200_unpermute_experts(T, d, k, b->dZ_home, b->token_mapping, dXn, stream)) return -1;
  B200_CUDA(cudaMemsetAsync(b->dX_routed, 0, 2 * (size_t)T * E, s));
  if (b200_ep_gather_router_grad(T, k, b->token_expert_weights, b->token_mapping, b->chosen_experts, b->expert_counts,
                                 b->expert_counts_cumsum, b->dst_base, b->peer_dP, b->world, E, El, cap, b->dX_routed,
                                 stream))
    return -1;
  if (b200_router_gate_bwd_x(T, E, k, b->chosen_experts, b->token_expert_weights, b->dX_routed, stream)) return -1;
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, B200_DT_BF16, 0, 0, d, E, T, 1.0f, 1.0f, b->Wr, b->dX_routed,
                  dXn, dXn, 0, nullptr, stream))
    return -1;
  // the replicated router weight sees every rank's tokens: this rank's partial sum, then the sum over the ranks
  if (b200_matmul(B200_DT_BF16, B200_DT_BF16, B200_DT_NONE, B200_DT_BF16, 0, 1, d, T, E, 1.0f, 0.0f, Xn, b->dX_routed,
                  nullptr, b->dWr_partial, b->matmul_workspace_bytes, b->matmul_workspace, stream))
    return -1;
  if (ep_sync(b, nullptr, 0, stream)) return -1;
  return b200_ep_reduce_router_grad(b->peer_dWr, b->world, (int64_t)E * d, dWr, stream);
}
