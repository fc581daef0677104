// Micro-benchmark behind the design of gemm_sm100.cu: what one thread issuing tcgen05.mma can and cannot hide.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o /tmp/mma_queue_probe mma_queue_probe.cu && /tmp/mma_queue_probe
// Every wait is bounded (sm100_ptx.cuh); operands are zeros resident in shared memory; nothing is loaded or stored.
// Depth of the tcgen05.mma queue and cost of tcgen05.commit, measured from one issuing thread.
//  exp 0: groups of G MMAs separated by a busy delay of D cycles (no commits)
//  exp 1: a commit (to a rotating dummy barrier) after every G MMAs, no delay
//  exp 2: latency: one MMA, commit, cycles until the barrier flips (repeated)
//  exp 3: commit after every G MMAs + wait for the commit issued two groups earlier (as a pipeline's consumer release)
#include <cstdio>
#include <cuda_runtime.h>
#include "../sm100_ptx.cuh"
using namespace b200;

struct Res { long long cycles, aux; int mmas; };

template <bool PAIR>
__global__ void __launch_bounds__(384, 1) k(int exp, int groups, int G, int D, int mc, int pollers, Res *res) {
  extern __shared__ unsigned char raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar, cbar[8];
  __shared__ uint32_t tmem_base_s;
  __shared__ int ab_s, st_s;
  __shared__ volatile int done_s;
  __shared__ uint64_t never;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
  for (int i = tid; i < 128 * 1024 / 16; i += 384) ((uint4 *)smem)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    ab_s = 0; st_s = 0; done_s = 0;
    ptx::mbar_init(ptx::smem_u32(&never), 1);
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    for (int i = 0; i < 8; i++) ptx::mbar_init(ptx::smem_u32(&cbar[i]), 1);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    if (PAIR) { ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_s), 512); ptx::tmem_relinquish_pair(); }
    else { ptx::tmem_alloc(ptx::smem_u32(&tmem_base_s), 512); ptx::tmem_relinquish(); }
  }
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync_all(); else __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tb = tmem_base_s;
  const uint32_t sbase = ptx::smem_u32(smem);
  auto commit = [&](uint32_t b) {
    if (PAIR && mc) ptx::umma_commit_pair(b);
    else if (PAIR) asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(b) : "memory");
    else ptx::umma_commit(b);
  };
  if (warp == 0 && tid == 0 && rank == 0) {
    const uint32_t idesc = ptx::make_idesc_bf16(PAIR ? 256 : 128, 256, 0, 0);
    auto mma = [&](int i) {
      const uint32_t sA = sbase + (i & 1) * 32768 + (i & 3) * 32, sB = sA + 16384;
      const uint64_t ad = ptx::make_smem_desc(sA, 0, 1024), bd = ptx::make_smem_desc(sB, 0, 1024);
      if (PAIR) ptx::umma_bf16_pair(tb, ad, bd, idesc, 1u); else ptx::umma_bf16(tb, ad, bd, idesc, 1u);
    };
    long long t0 = clock64(), aux = 0;
    int cnt = 0;
    uint32_t par[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (exp == 2) {
      for (int g = 0; g < groups; g++) {
        const long long a = clock64();
        mma(0); cnt++;
        commit(ptx::smem_u32(&cbar[0]));
        ptx::mbar_wait<PAIR>(ptx::smem_u32(&cbar[0]), par[0], &ab_s, &st_s, 3);
        par[0] ^= 1u;
        aux += clock64() - a;
      }
    } else {
      for (int g = 0; g < groups; g++) {
        for (int i = 0; i < G; i++) { mma(i); cnt++; }
        if (exp == 0 && D > 0) { const long long a = clock64(); while (clock64() - a < D) {} }
        if (exp == 1 || exp == 3) commit(ptx::smem_u32(&cbar[g & 7]));
        if (exp == 3 && g >= 2) {
          const long long a = clock64();
          const int s = (g - 2) & 7;
          ptx::mbar_wait<PAIR>(ptx::smem_u32(&cbar[s]), par[s], &ab_s, &st_s, 3);
          par[s] ^= 1u;
          aux += clock64() - a;
        }
      }
    }
    if (PAIR) ptx::umma_commit_pair(ptx::smem_u32(&bar)); else ptx::umma_commit(ptx::smem_u32(&bar));
    ptx::mbar_wait<PAIR>(ptx::smem_u32(&bar), 0, &ab_s, &st_s, 1);
    long long t1 = clock64();
    if (blockIdx.x == 0) { res->cycles = t1 - t0; res->mmas = cnt; res->aux = aux; }
    done_s = 1;
  } else if (PAIR && warp == 0 && tid == 0) {
    ptx::mbar_wait<PAIR>(ptx::smem_u32(&bar), 0, &ab_s, &st_s, 1);
    done_s = 1;
  }
  if (warp >= 2 && warp < 2 + (pollers & 15)) {
    // like the epilogue warps of the GEMM while they wait for an accumulator: every lane (bit 4 clear) or lane 0 only
    // (bit 4 set) polls a barrier that does not complete, and looks at a flag in shared memory between polls
    const bool lane0_only = (pollers & 16) != 0;
    if (!lane0_only || (tid & 31) == 0) {
      unsigned long long guard = 0;
      while (!done_s && guard < 200000000ull) {
        if (ptx::mbar_try_wait(ptx::smem_u32(&never), 0)) break;
        guard++;
      }
    }
    __syncwarp();
  }
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    if (PAIR) ptx::tmem_dealloc_pair(tb, 512); else ptx::tmem_dealloc(tb, 512);
  }
}

template <bool PAIR>
void run(int exp, int groups, int G, int D, int mc, int pollers = 0) {
  Res *d; cudaMalloc(&d, sizeof(Res)); cudaMemset(d, 0, sizeof(Res));
  const int smem = 140 * 1024;
  cudaFuncSetAttribute(k<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(148); cfg.blockDim = dim3(384); cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = PAIR ? 2 : 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  for (int rep = 0; rep < 2; rep++) {
    cudaError_t rc = cudaLaunchKernelEx(&cfg, k<PAIR>, exp, groups, G, D, mc, pollers, d);
    cudaError_t rs = cudaDeviceSynchronize();
    Res h; cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
    if (rep == 1)
      printf("%s exp=%d G=%2d D=%4d mc=%d pollers=%2d: %.1f cycles/MMA, %.0f cycles/group, aux %.0f cycles/group  rc=%d/%d\n", PAIR ? "pair  " : "single",
             exp, G, D, mc, pollers, (double)h.cycles / h.mmas, (double)h.cycles / groups, (double)h.aux / groups, (int)rc, (int)rs);
  }
  cudaFree(d);
}

int main() {
  // exp 0: how long may the issuing thread pause between groups of eight MMAs before the pipe idles
  for (int D : {0, 100, 200, 400, 800, 1600}) run<true>(0, 1000, 8, D, 1);
  for (int D : {0, 400, 1600}) run<false>(0, 1000, 8, D, 1);
  // exp 1: cost of a commit every G MMAs (multicast to both CTAs of a pair, to the issuing CTA only, single CTA)
  for (int G : {4, 8, 16, 32}) { run<true>(1, 1000, G, 0, 1); run<true>(1, 1000, G, 0, 0); run<false>(1, 1000, G, 0, 0); }
  // exp 2: one MMA, commit, cycles until the barrier flips
  run<true>(2, 200, 1, 0, 1); run<true>(2, 200, 1, 0, 0); run<false>(2, 200, 1, 0, 0);
  // exp 3: commit every G MMAs and a wait on a barrier that completed two groups ago (aux = cycles inside the wait)
  for (int G : {4, 8, 16}) { run<true>(3, 1000, G, 0, 1); run<false>(3, 1000, G, 0, 0); }
  // eight warps polling a barrier that never completes (all lanes / lane 0 only) beside the issuing thread
  for (int pl : {0, 8, 16 + 8}) run<true>(1, 1000, 8, 0, 1, pl);
  return 0;
}
