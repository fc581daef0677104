// Router kernels: top-k selection + softmax + histogram + exclusive scan, the
// deterministic expert/token mapping, and the gate backward.
#include "common.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

// ---------------------------------------------------------------------------------------
// select_experts
//
// One thread per token. A block stages a [32 tokens x 64 experts] logits tile in shared
// memory with coalesced loads (row pitch 65 floats so the per-thread row walk is bank
// conflict free), then every thread replays the reference's sequential insert/evict rule
// over its row so the slot order of chosen_experts is identical to the reference's
// (backends/nvidia/src/ops/src/native/src/moe/select_experts.cu:135-166).
// The k slots live in registers (KP = k rounded up to a power of two, loops unrolled).
// Histogram: shared-memory atomics, one global atomic per expert per block; the block that
// finishes last performs the exclusive scan and the host copy (select_experts.cu:207-294).
// ---------------------------------------------------------------------------------------

constexpr int SEL_TOKENS = 32;   // tokens per block = threads per block (one warp: 256 blocks at 8192 tokens)
constexpr int SEL_EC = 64;       // experts per staged chunk
static_assert(SEL_EC == 64, "the staging loop shifts by 6");
constexpr int SEL_PITCH = SEL_EC + 1;

template <typename T>
__device__ __forceinline__ float load_logit(const T *p);
template <>
__device__ __forceinline__ float load_logit<float>(const float *p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16 *p) {
  return __bfloat162float(*p);
}

template <int KP, typename T>
__global__ void __launch_bounds__(SEL_TOKENS)
select_experts_kernel(int total_tokens, int n_experts, int top_k, const T *__restrict__ X_routed,
                      float *__restrict__ token_expert_weights, uint16_t *__restrict__ chosen_experts,
                      int *expert_counts, int *expert_counts_cumsum, int *host_expert_counts) {
  extern __shared__ __align__(16) unsigned char sel_smem[];
  float *tile = reinterpret_cast<float *>(sel_smem);                       // [SEL_TOKENS][SEL_PITCH]
  int *block_counts = reinterpret_cast<int *>(tile + SEL_TOKENS * SEL_PITCH);  // [n_experts]
  __shared__ int completion;

  const int tid = threadIdx.x;
  const int64_t tok0 = (int64_t)blockIdx.x * SEL_TOKENS;
  const int64_t token = tok0 + tid;
  const bool active = token < total_tokens;

  for (int e = tid; e < n_experts; e += SEL_TOKENS) block_counts[e] = 0;

  float vals[KP];
  int inds[KP];
#pragma unroll
  for (int j = 0; j < KP; j++) {
    vals[j] = -INFINITY;
    inds[j] = 0xFFFF;
  }
  float max_val = -INFINITY, min_val = -INFINITY;
  int min_slot = 0;

  const int rows_here = (int)min((int64_t)SEL_TOKENS, (int64_t)total_tokens - tok0);
  for (int e0 = 0; e0 < n_experts; e0 += SEL_EC) {
    const int ec = min(SEL_EC, n_experts - e0);
    __syncthreads();  // previous chunk fully consumed (and block_counts zeroed on first pass)
    // sixteen independent loads in flight per thread before the first store (one load per trip leaves the whole
    // staging loop waiting on memory latency, trip after trip)
    const int n_stage = rows_here * ec;
    for (int i0 = tid; i0 < n_stage; i0 += SEL_TOKENS * 16) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; u++) {
        const int i = i0 + u * SEL_TOKENS;
        const int r = ec == SEL_EC ? i >> 6 : i / ec, c = i - r * ec;  // no division in the common 64-expert chunk
        v[u] = (i < n_stage) ? load_logit<T>(X_routed + (tok0 + r) * n_experts + e0 + c) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 16; u++) {
        const int i = i0 + u * SEL_TOKENS;
        const int r = ec == SEL_EC ? i >> 6 : i / ec, c = i - r * ec;
        if (i < n_stage) tile[r * SEL_PITCH + c] = v[u];
      }
    }
    __syncthreads();
    if (active) {
      const float *row = tile + tid * SEL_PITCH;
      for (int c = 0; c < ec; c++) {
        const float v = row[c];
        if (v > min_val) {
          if (v > max_val) max_val = v;
#pragma unroll
          for (int j = 0; j < KP; j++)
            if (j == min_slot) {
              vals[j] = v;
              inds[j] = e0 + c;
            }
          min_val = INFINITY;
          min_slot = 0;
          int min_exp = 0xFFFF;
#pragma unroll
          for (int j = 0; j < KP; j++) {
            if (j < top_k && (vals[j] < min_val || (vals[j] == min_val && inds[j] > min_exp))) {
              min_val = vals[j];
              min_slot = j;
              min_exp = inds[j];
            }
          }
        }
      }
    }
  }

  if (active) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < KP; j++)
      if (j < top_k) sum += expf(vals[j] - max_val);
    float *wout = token_expert_weights + token * top_k;
    uint16_t *cout = chosen_experts + token * top_k;
#pragma unroll
    for (int j = 0; j < KP; j++)
      if (j < top_k) {
        wout[j] = expf(vals[j] - max_val) / sum;
        cout[j] = (uint16_t)inds[j];
        if (inds[j] < n_experts) atomicAdd(&block_counts[inds[j]], 1);
      }
  }
  __syncthreads();
  for (int e = tid; e < n_experts; e += SEL_TOKENS) {
    int c = block_counts[e];
    if (c) atomicAdd(&expert_counts[e], c);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) completion = atomicAdd(&expert_counts[n_experts], 1);
  __syncthreads();
  if (completion != (int)gridDim.x - 1) return;
  __threadfence();
  if (tid >= 32) return;

  // last block, first warp: exclusive scan of the counts in chunks of 32, then host copy
  int running = 0;
  for (int e0 = 0; e0 < n_experts; e0 += 32) {
    const int e = e0 + tid;
    const int v = (e < n_experts) ? __ldcg(&expert_counts[e]) : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += t;
    }
    if (e < n_experts) {
      expert_counts_cumsum[e] = running + incl - v;
      if (host_expert_counts) host_expert_counts[e] = v;
    }
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
}

template <typename T>
static int launch_select(int T_, int E, int k, const T *X, float *w, uint16_t *ch, int *counts, int *cumsum,
                         int *host_counts, cudaStream_t s) {
  const int grid = (T_ + SEL_TOKENS - 1) / SEL_TOKENS;
  const size_t smem = sizeof(float) * SEL_TOKENS * SEL_PITCH + sizeof(int) * E;
#define SEL_LAUNCH(KP)                                                                                     \
  do {                                                                                                     \
    auto kern = select_experts_kernel<KP, T>;                                                              \
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));         \
    kern<<<grid, SEL_TOKENS, smem, s>>>(T_, E, k, X, w, ch, counts, cumsum, host_counts);                  \
  } while (0)
  if (k <= 1) SEL_LAUNCH(1);
  else if (k <= 2) SEL_LAUNCH(2);
  else if (k <= 4) SEL_LAUNCH(4);
  else if (k <= 8) SEL_LAUNCH(8);
  else if (k <= 16) SEL_LAUNCH(16);
  else SEL_LAUNCH(32);
#undef SEL_LAUNCH
  B200_CHECK_LAUNCH("select_experts");
  return 0;
}

// ---------------------------------------------------------------------------------------
// build_expert_mapping: deterministic stable counting sort in two launches.
//
// The T*k (token, slot) entries are cut into contiguous runs, one per warp. Launch 1 counts
// experts per warp run and per block into scratch. Launch 2: each block sums the block
// histograms before it (giving its base inside every expert's range), each warp adds the
// warp histograms before it inside the block, then walks its run 32 entries at a time and
// ranks equal experts with __match_any_sync, so rows are numbered tokens-ascending then
// slots-ascending. The block that owns the tail writes the inclusive cumsum the reference
// leaves behind (moe/build_expert_mapping.cu:63-67).
// scratch layout (ints): excl[E] | block_hist[nblocks][E] | warp_hist[nblocks*MAP_WARPS][E]
// ---------------------------------------------------------------------------------------

constexpr int MAP_WARPS = 8;
constexpr int MAP_THREADS = MAP_WARPS * 32;

struct MapPlan {
  int nblocks;
  int run;  // entries per warp, multiple of 32
};

static MapPlan map_plan(int64_t n_entries) {
  MapPlan p;
  int64_t max_blocks = 296;
  int64_t per_warp = (n_entries + max_blocks * MAP_WARPS - 1) / (max_blocks * MAP_WARPS);
  per_warp = ((per_warp + 31) / 32) * 32;
  if (per_warp < 32) per_warp = 32;
  p.run = (int)per_warp;
  p.nblocks = (int)((n_entries + per_warp * MAP_WARPS - 1) / (per_warp * MAP_WARPS));
  if (p.nblocks < 1) p.nblocks = 1;
  return p;
}

__global__ void __launch_bounds__(MAP_THREADS)
mapping_hist_kernel(int64_t n_entries, int E, int run, const uint16_t *__restrict__ chosen,
                    const int *__restrict__ cumsum_excl, int *__restrict__ scratch) {
  extern __shared__ int map_smem[];  // [MAP_WARPS][E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblocks = gridDim.x;
  int *excl_copy = scratch;
  int *block_hist = scratch + E;
  int *warp_hist = block_hist + (int64_t)nblocks * E;

  for (int i = tid; i < MAP_WARPS * E; i += MAP_THREADS) map_smem[i] = 0;
  if (blockIdx.x == 0)
    for (int e = tid; e < E; e += MAP_THREADS) excl_copy[e] = cumsum_excl[e];
  __syncthreads();

  int *mine = map_smem + warp * E;
  const int64_t begin = ((int64_t)blockIdx.x * MAP_WARPS + warp) * run;
  const int64_t end = min(begin + (int64_t)run, n_entries);
  for (int64_t i = begin + lane; i < end; i += 32) {
    int e = chosen[i];
    if (e < E) atomicAdd(&mine[e], 1);
  }
  __syncthreads();
  for (int e = tid; e < E; e += MAP_THREADS) {
    int s = 0;
#pragma unroll
    for (int w = 0; w < MAP_WARPS; w++) {
      int c = map_smem[w * E + e];
      warp_hist[((int64_t)blockIdx.x * MAP_WARPS + w) * E + e] = c;
      s += c;
    }
    block_hist[(int64_t)blockIdx.x * E + e] = s;
  }
}

__global__ void __launch_bounds__(MAP_THREADS)
mapping_scatter_kernel(int64_t n_entries, int E, int top_k, int run, const uint16_t *__restrict__ chosen,
                       const int *__restrict__ scratch, int *__restrict__ cumsum_out,
                       int *__restrict__ expert_mapping, int *__restrict__ token_mapping) {
  extern __shared__ int map_smem[];  // cursor[MAP_WARPS][E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblocks = gridDim.x;
  const int *excl_copy = scratch;
  const int *block_hist = scratch + E;
  const int *warp_hist = block_hist + (int64_t)nblocks * E;

  // base of this block inside every expert range
  for (int e = tid; e < E; e += MAP_THREADS) {
    int base = excl_copy[e];
    for (int b = 0; b < (int)blockIdx.x; b++) base += block_hist[(int64_t)b * E + e];
    int run_sum = base;
#pragma unroll
    for (int w = 0; w < MAP_WARPS; w++) {
      map_smem[w * E + e] = run_sum;
      run_sum += warp_hist[((int64_t)blockIdx.x * MAP_WARPS + w) * E + e];
    }
    if (blockIdx.x == nblocks - 1) cumsum_out[e] = run_sum;  // inclusive prefix sum
  }
  __syncthreads();

  int *cursor = map_smem + warp * E;
  const int64_t begin = ((int64_t)blockIdx.x * MAP_WARPS + warp) * run;
  const int64_t end = min(begin + (int64_t)run, n_entries);
  for (int64_t i0 = begin; i0 < end; i0 += 32) {
    const int64_t i = i0 + lane;
    const bool valid = i < end;
    int e = valid ? (int)chosen[i] : 0xFFFF;
    const bool routed = valid && e < E;
    // lanes that are not routed get a key no routed lane can have
    const unsigned peers = __match_any_sync(0xffffffffu, routed ? e : (0x10000 + lane));
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (routed) base = cursor[e];
    __syncwarp();
    if (routed && rank == 0) cursor[e] = base + __popc(peers);
    __syncwarp();
    if (routed) {
      const int pos = base + rank;
      expert_mapping[pos] = (int)(i / top_k);
      token_mapping[i] = pos;
    } else if (valid) {
      token_mapping[i] = -1;
    }
  }
}

// ---------------------------------------------------------------------------------------
// router_gate_bwd_x: one warp per token (moe/router_gate_bwd_x.cu:7-57).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
router_gate_bwd_kernel(int num_tokens, int E, int top_k, const uint16_t *__restrict__ chosen,
                       const float *__restrict__ weights, __nv_bfloat16 *__restrict__ dX_routed) {
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= num_tokens) return;
  __nv_bfloat16 *row = dX_routed + token * E;
  float part = 0.f;
  for (int j = lane; j < top_k; j += 32) {
    int e = chosen[token * top_k + j];
    if (e < E) part += __bfloat162float(row[e]) * weights[token * top_k + j];
  }
  const float avg = warp_sum(part);
  __syncwarp();
  for (int j = lane; j < top_k; j += 32) {
    int e = chosen[token * top_k + j];
    if (e < E) {
      float w = weights[token * top_k + j];
      row[e] = __float2bfloat16_rn(w * (__bfloat162float(row[e]) - avg));
    }
  }
}

// row_weights[token_mapping[t,j]] = w[t,j]
__global__ void scatter_row_weights_kernel(int64_t n, const int *__restrict__ token_mapping,
                                           const float *__restrict__ w, float *__restrict__ row_weights) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int r = token_mapping[i];
  if (r >= 0) row_weights[r] = w[i];
}

// dX_routed[t, chosen[t,j]] = bf16(dP[token_mapping[t,j]])
__global__ void gather_router_grad_kernel(int64_t n, int E, int top_k, const int *__restrict__ token_mapping,
                                          const uint16_t *__restrict__ chosen, const float *__restrict__ dP,
                                          __nv_bfloat16 *__restrict__ dX_routed) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int r = token_mapping[i];
  int e = chosen[i];
  if (r >= 0 && e < E) dX_routed[(i / top_k) * E + e] = __float2bfloat16_rn(dP[r]);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_device_info(int *sm_count, int *cc_major, int *cc_minor) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp p;
  B200_CUDA(cudaGetDeviceProperties(&p, dev));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return 0;
}

extern "C" int b200_select_experts(int x_dt, int total_tokens, int n_experts, int top_k_experts,
                                   const void *X_routed, float *token_expert_weights, uint16_t *chosen_experts,
                                   int *expert_counts, int *expert_counts_cumsum, int *host_expert_counts,
                                   void *stream) {
  B200_REQUIRE(x_dt == B200_DT_FP32 || x_dt == B200_DT_BF16, "select_experts: logits must be fp32 or bf16 (got %d)", x_dt);
  B200_REQUIRE(total_tokens >= 0 && n_experts >= 1 && n_experts <= B200_MAX_EXPERTS,
               "select_experts: need 1 <= n_experts <= %d (got %d)", B200_MAX_EXPERTS, n_experts);
  B200_REQUIRE(top_k_experts >= 1 && top_k_experts <= B200_MAX_TOP_K && top_k_experts <= n_experts,
               "select_experts: need 1 <= top_k <= min(%d, n_experts) (got %d)", B200_MAX_TOP_K, top_k_experts);
  B200_REQUIRE(X_routed && token_expert_weights && chosen_experts && expert_counts && expert_counts_cumsum,
               "select_experts: null buffer");
  if (total_tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dt == B200_DT_FP32)
    return launch_select<float>(total_tokens, n_experts, top_k_experts, (const float *)X_routed,
                                token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum,
                                host_expert_counts, s);
  return launch_select<__nv_bfloat16>(total_tokens, n_experts, top_k_experts, (const __nv_bfloat16 *)X_routed,
                                      token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum,
                                      host_expert_counts, s);
}

extern "C" size_t b200_build_expert_mapping_workspace_bytes(int total_tokens, int num_routed_experts,
                                                            int num_selected_experts) {
  if (total_tokens < 0 || num_routed_experts < 1 || num_selected_experts < 1) return 0;
  MapPlan p = map_plan((int64_t)total_tokens * num_selected_experts);
  size_t ints = (size_t)num_routed_experts * (1 + (size_t)p.nblocks * (1 + MAP_WARPS));
  return ints * sizeof(int);
}

extern "C" int b200_build_expert_mapping(int total_tokens, int num_routed_experts, int num_selected_experts,
                                         const uint16_t *chosen_experts, int *expert_counts_cumsum,
                                         int *expert_mapping, int *token_mapping, void *workspace,
                                         size_t workspace_bytes, void *stream) {
  B200_REQUIRE(total_tokens >= 0 && num_routed_experts >= 1 && num_routed_experts <= B200_MAX_EXPERTS,
               "build_expert_mapping: need 1 <= experts <= %d (got %d)", B200_MAX_EXPERTS, num_routed_experts);
  B200_REQUIRE(num_selected_experts >= 1, "build_expert_mapping: top_k must be >= 1");
  B200_REQUIRE(chosen_experts && expert_counts_cumsum && expert_mapping && token_mapping,
               "build_expert_mapping: null buffer");
  const size_t need = b200_build_expert_mapping_workspace_bytes(total_tokens, num_routed_experts, num_selected_experts);
  B200_REQUIRE(workspace && workspace_bytes >= need, "build_expert_mapping: workspace too small (%zu < %zu)",
               workspace_bytes, need);
  if (total_tokens == 0) return 0;
  const int64_t n = (int64_t)total_tokens * num_selected_experts;
  MapPlan p = map_plan(n);
  const size_t smem = sizeof(int) * MAP_WARPS * num_routed_experts;
  cudaStream_t s = (cudaStream_t)stream;
  B200_CUDA(cudaFuncSetAttribute(mapping_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  B200_CUDA(cudaFuncSetAttribute(mapping_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mapping_hist_kernel<<<p.nblocks, MAP_THREADS, smem, s>>>(n, num_routed_experts, p.run, chosen_experts,
                                                           expert_counts_cumsum, (int *)workspace);
  B200_CHECK_LAUNCH("build_expert_mapping(hist)");
  mapping_scatter_kernel<<<p.nblocks, MAP_THREADS, smem, s>>>(n, num_routed_experts, num_selected_experts, p.run,
                                                              chosen_experts, (const int *)workspace,
                                                              expert_counts_cumsum, expert_mapping, token_mapping);
  B200_CHECK_LAUNCH("build_expert_mapping(scatter)");
  return 0;
}

// ---------------------------------------------------------------------------------------
// build_expert_mapping without caller-provided scratch.
//
// Some hosts of this library cannot hand over device scratch: a backend op slot whose
// argument list is fixed by the framework's op signature (build_expert_mapping has exactly
// seven arguments there) and which runs at submit time, when the framework forbids device
// allocation because all device memory was carved up front. For them the histogram tables
// live in this fixed array inside the library image. Every GPU that loads the library keeps
// the array (4 MiB) until the process exits.
// ---------------------------------------------------------------------------------------
constexpr size_t STATIC_MAP_SCRATCH_INTS = 1u << 20;  // 4 MiB
static __device__ __align__(256) int g_static_map_scratch[STATIC_MAP_SCRATCH_INTS];

constexpr int STATIC_MAX_DEVICES = 64;
static int *g_static_map_scratch_addr[STATIC_MAX_DEVICES];  // device address of the array, per device ordinal

extern "C" size_t b200_build_expert_mapping_static_capacity_bytes(void) {
  return STATIC_MAP_SCRATCH_INTS * sizeof(int);
}

extern "C" int b200_build_expert_mapping_static(int total_tokens, int num_routed_experts, int num_selected_experts,
                                                const uint16_t *chosen_experts, int *expert_counts_cumsum,
                                                int *expert_mapping, int *token_mapping, void *stream) {
  const size_t need =
      b200_build_expert_mapping_workspace_bytes(total_tokens, num_routed_experts, num_selected_experts);
  B200_REQUIRE(need != 0, "build_expert_mapping_static: bad sizes (tokens %d, experts %d, top_k %d)", total_tokens,
               num_routed_experts, num_selected_experts);
  B200_REQUIRE(need <= STATIC_MAP_SCRATCH_INTS * sizeof(int),
               "build_expert_mapping_static: this problem needs %zu bytes of scratch but the built-in array holds %zu; "
               "use b200_build_expert_mapping with caller scratch",
               need, STATIC_MAP_SCRATCH_INTS * sizeof(int));
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, "build_expert_mapping_static: device ordinal %d out of range", dev);
  if (g_static_map_scratch_addr[dev] == nullptr) {
    // In host code the array's name is only a handle; the kernels need its address on the current device.
    int *addr = nullptr;
    B200_CUDA(cudaGetSymbolAddress((void **)&addr, g_static_map_scratch));
    B200_REQUIRE(addr != nullptr, "build_expert_mapping_static: no device address for the built-in scratch");
    g_static_map_scratch_addr[dev] = addr;
  }
  return b200_build_expert_mapping(total_tokens, num_routed_experts, num_selected_experts, chosen_experts,
                                   expert_counts_cumsum, expert_mapping, token_mapping, g_static_map_scratch_addr[dev],
                                   STATIC_MAP_SCRATCH_INTS * sizeof(int), stream);
}

extern "C" int b200_router_gate_bwd_x(int num_tokens, int num_routed_experts, int top_k_active,
                                      const uint16_t *chosen_experts, const float *token_expert_weights,
                                      void *dX_routed, void *stream) {
  B200_REQUIRE(num_tokens >= 0 && num_routed_experts >= 1 && top_k_active >= 1, "router_gate_bwd_x: bad sizes");
  B200_REQUIRE(chosen_experts && token_expert_weights && dX_routed, "router_gate_bwd_x: null buffer");
  if (num_tokens == 0) return 0;
  const int warps = 8;
  router_gate_bwd_kernel<<<(num_tokens + warps - 1) / warps, warps * 32, 0, (cudaStream_t)stream>>>(
      num_tokens, num_routed_experts, top_k_active, chosen_experts, token_expert_weights,
      (__nv_bfloat16 *)dX_routed);
  B200_CHECK_LAUNCH("router_gate_bwd_x");
  return 0;
}

extern "C" int b200_scatter_row_weights(int num_tokens, int top_k, const int *token_mapping,
                                        const float *token_expert_weights, float *row_weights, void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k >= 1 && token_mapping && token_expert_weights && row_weights,
               "scatter_row_weights: bad arguments");
  const int64_t n = (int64_t)num_tokens * top_k;
  if (n == 0) return 0;
  scatter_row_weights_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      n, token_mapping, token_expert_weights, row_weights);
  B200_CHECK_LAUNCH("scatter_row_weights");
  return 0;
}

extern "C" int b200_gather_router_grad(int num_tokens, int num_routed_experts, int top_k, const int *token_mapping,
                                       const uint16_t *chosen_experts, const float *dP, void *dX_routed,
                                       void *stream) {
  B200_REQUIRE(num_tokens >= 0 && top_k >= 1 && num_routed_experts >= 1 && token_mapping && chosen_experts && dP &&
                   dX_routed,
               "gather_router_grad: bad arguments");
  const int64_t n = (int64_t)num_tokens * top_k;
  if (n == 0) return 0;
  gather_router_grad_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      n, num_routed_experts, top_k, token_mapping, chosen_experts, dP, (__nv_bfloat16 *)dX_routed);
  B200_CHECK_LAUNCH("gather_router_grad");
  return 0;
}
