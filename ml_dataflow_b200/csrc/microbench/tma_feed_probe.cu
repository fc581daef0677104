// Micro-benchmark behind the design of gemm_sm100.cu: how many bytes per clock TMA can feed an SM from L2 / HBM, by box
// size and number of issuing threads, with and without a thread issuing tcgen05.mma on other shared-memory stages.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o /tmp/tma_feed_probe tma_feed_probe.cu && /tmp/tma_feed_probe
// Loads and MMAs are independent (no pipeline between them); every wait is bounded; plain per-CTA TMA loads only.
// MMA rate with concurrent, INDEPENDENT TMA traffic into other shared-memory stages (no dependency between the two):
// isolates shared-memory / fabric contention from the pipeline protocol.
//   mode bits: 1 = TMA producer runs, 2 = MMA thread runs
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../sm100_ptx.cuh"
using namespace b200;

struct Res { long long mma_cycles, prod_cycles; int mmas, slabs; };

template <bool PAIR>
__global__ void __launch_bounds__(256, 1)
k(const __grid_constant__ CUtensorMap tm, int iters, int mode, int box_rows, int boxes_per_slab, int inflight, int mma_stages,
  int rows_total, int nprod, int commit_every, int fence_wait, Res *res) {
  extern __shared__ unsigned char raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar, pbar[32], cbar[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int ab_s, st_s;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
  for (int i = tid; i < 208 * 1024 / 16; i += 256) ((uint4 *)smem)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    ab_s = 0; st_s = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    for (int i = 0; i < 32; i++) ptx::mbar_init(ptx::smem_u32(&pbar[i]), 1);
    for (int i = 0; i < 4; i++) ptx::mbar_init(ptx::smem_u32(&cbar[i]), 1);
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
  // MMA operands: stages [0, mma_stages) of 32 KB; TMA ring: the 32 KB stages after them
  if (warp == 0 && tid == 0 && rank == 0 && (mode & 2)) {
    const uint32_t idesc = ptx::make_idesc_bf16(PAIR ? 256 : 128, 256, 0, 0);
    long long t0 = clock64();
    int cnt = 0;
    for (int it = 0; it < iters; it++) {
      const uint32_t sA = sbase + (it % mma_stages) * 32768;
      const uint32_t sB = sA + 16384;
#pragma unroll
      for (int k16 = 0; k16 < 4; k16++) {
        const uint64_t ad = ptx::make_smem_desc(sA + k16 * 32, 0, 1024);
        const uint64_t bd = ptx::make_smem_desc(sB + k16 * 32, 0, 1024);
        if (PAIR) ptx::umma_bf16_pair(tb + (it & 1) * 256, ad, bd, idesc, 1u);
        else ptx::umma_bf16(tb + (it & 1) * 256, ad, bd, idesc, 1u);
        cnt++;
      }
      if (commit_every > 0 && (it + 1) % commit_every == 0) {
        if (PAIR) ptx::umma_commit_pair(ptx::smem_u32(&cbar[(it / commit_every) & 3]));
        else ptx::umma_commit(ptx::smem_u32(&cbar[(it / commit_every) & 3]));
        if (fence_wait) {
          // a wait on a barrier that completed long ago (the first commit's), then the fence the real loop uses
          if (it >= 64) ptx::mbar_wait<PAIR>(ptx::smem_u32(&pbar[31]), 1, &ab_s, &st_s, 3);
          ptx::tc_fence_after();
        }
      }
    }
    if (PAIR) ptx::umma_commit_pair(ptx::smem_u32(&bar)); else ptx::umma_commit(ptx::smem_u32(&bar));
    ptx::mbar_wait<PAIR>(ptx::smem_u32(&bar), 0, &ab_s, &st_s, 1);
    long long t1 = clock64();
    if (blockIdx.x == 0) { res->mma_cycles = t1 - t0; res->mmas = cnt; }
  } else if (PAIR && warp == 0 && tid == 0 && (mode & 2)) {
    ptx::mbar_wait<PAIR>(ptx::smem_u32(&bar), 0, &ab_s, &st_s, 1);
  }
  if (warp >= 2 && warp < 2 + nprod && (tid & 31) == 0 && (mode & 1)) {
    // producer p streams 32768 / nprod bytes per iteration into its own ring of `inflight` slots
    const int pidx = warp - 2;
    long long t0 = clock64();
    const int part_bytes = 32768 / nprod;
    const uint32_t ring = sbase + mma_stages * 32768 + pidx * (4 * part_bytes);
    const int box_bytes = box_rows * 128;
    const int nbox = part_bytes / box_bytes;
    uint64_t *mybar = &pbar[pidx * 8];
    uint32_t par[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    bool alive = true;
    for (int s = 0; s < iters && alive; s++) {
      const int slot = s % inflight;
      if (s >= inflight) {
        alive = ptx::mbar_wait<false>(ptx::smem_u32(&mybar[slot]), par[slot], &ab_s, &st_s, 2);
        par[slot] ^= 1u;
      }
      ptx::mbar_arrive_expect_tx(ptx::smem_u32(&mybar[slot]), (uint32_t)(nbox * box_bytes));
      const long long r0 = ((long long)blockIdx.x * 9973 + (long long)s * 131 + pidx * 57) * 256;
      for (int b = 0; b < nbox; b++) {
        const int row = (int)((r0 + (long long)b * box_rows) % (rows_total - box_rows));
        ptx::tma_load_2d(ring + slot * part_bytes + b * box_bytes, &tm, ptx::smem_u32(&mybar[slot]), (s & 63) * 64, row & ~7);
      }
    }
    for (int s = max(0, iters - inflight); s < iters && alive; s++) {
      const int slot = s % inflight;
      alive = ptx::mbar_wait<false>(ptx::smem_u32(&mybar[slot]), par[slot], &ab_s, &st_s, 2);
      par[slot] ^= 1u;
    }
    if (blockIdx.x == 0 && pidx == 0) { res->prod_cycles = clock64() - t0; res->slabs = iters; }
  }
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    if (PAIR) ptx::tmem_dealloc_pair(tb, 512); else ptx::tmem_dealloc(tb, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <bool PAIR>
void run(const char *name, void *buf, int rows_total, int mode, int box_rows, int inflight, int mma_stages, int nprod, int commit_every, int fence_wait) {
  void *sym = nullptr; cudaDriverEntryPointQueryResult q;
  cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
  EncodeTiledFn fn = (EncodeTiledFn)sym;
  CUtensorMap tm;
  cuuint64_t dims[2] = {4096, (cuuint64_t)rows_total};
  cuuint64_t strides[1] = {8192};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, buf, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return; }
  Res *d; cudaMalloc(&d, sizeof(Res)); cudaMemset(d, 0, sizeof(Res));
  const int smem = 220 * 1024;
  cudaFuncSetAttribute(k<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(148); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = PAIR ? 2 : 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  const int iters = 4000;
  const int boxes_per_slab = 32768 / (box_rows * 128);
  for (int rep = 0; rep < 2; rep++) {
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0);
    cudaError_t rc = cudaLaunchKernelEx(&cfg, k<PAIR>, tm, iters, mode, box_rows, boxes_per_slab, inflight, mma_stages, rows_total, nprod, commit_every, fence_wait, d);
    cudaEventRecord(e1);
    cudaError_t rs = cudaDeviceSynchronize();
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    Res h; cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
    if (rep == 1)
      printf("%-8s mode=%d box_rows=%3d nprod=%d commit_every=%d fw=%d: %.1f cycles/MMA, %.0f cycles/slab TMA (%.1f B/clk/SM), %.3f ms rc=%d/%d\n",
             name, mode, box_rows, nprod, commit_every, fence_wait, h.mmas ? (double)h.mma_cycles / h.mmas : 0.0,
             h.slabs ? (double)h.prod_cycles / h.slabs : 0.0, h.slabs ? 32768.0 * h.slabs / h.prod_cycles : 0.0, ms, (int)rc, (int)rs);
  }
  cudaFree(d);
}

int main() {
  const int rows_big = 32768;
  void *buf; cudaMalloc(&buf, (size_t)rows_big * 8192);
  cudaMemset(buf, 0, (size_t)rows_big * 8192);
  for (int rows_total : {4096, 32768}) {   // 32 MB (stays in L2) and 256 MB
    printf("--- CTA pairs, %d rows (%d MB)\n", rows_total, rows_total / 128);
    run<true>("pair", buf, rows_total, 2, 64, 4, 2, 1, 0, 0);   // MMAs alone
    for (int nprod : {1, 2, 4})
      for (int box_rows : {64, 128, 256}) {
        if (box_rows * 128 > 32768 / nprod) continue;
        run<true>("pair", buf, rows_total, 1, box_rows, 4, 2, nprod, 0, 0);   // loads alone
        run<true>("pair", buf, rows_total, 3, box_rows, 4, 2, nprod, 0, 0);   // both
      }
  }
  run<false>("single", buf, 4096, 3, 128, 4, 2, 2, 0, 0);
  return 0;
}
