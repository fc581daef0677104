// Fused softmax attention for sm_100a (head_dim 64 or 128, bf16): the scores and the probabilities never leave the SM.
// It serves b200_attention_fwd / _bwd (attention.cu), which keep the GEMM-by-GEMM form for every other head size (the
// backward kernel here is for head_dim 128).
//
// Forward, one CTA per (query head, 256 query rows of one sequence): Q (two 128-row tiles) is fetched once by TMA; the
// key and value tiles of 128 keys pass through a three-slot ring. One thread issues the tcgen05 MMAs
//     S_g = Q_g K_j^T  (fp32, tensor memory)        O_g += P_g V_j  (fp32, tensor memory)
// and two groups of four warps (one per query tile, a thread per query row = per tensor-memory lane) turn S_g into
// P_g = exp2((S_g - m) * scale * log2 e), keep the row's sum, and write P_g as bf16 into shared memory in the layout
// the second MMA reads (128-byte swizzle, keys contiguous). The offset m is the row maximum of the first key block; it
// is raised - and the sum and O_g rescaled in tensor memory - only when a later block's maximum exceeds it by more than
// 2^8, so the common step never touches O_g. While one group works on its scores the tensor pipe runs the other
// group's P V and next Q K^T. At the end O_g is divided by the sum and stored. Rounding points: scores, maximum, sum and
// the output in fp32; P to bf16 (unnormalised, relative to m) before it multiplies V; one rounding of the output.
//
// Every wait is bounded (two seconds); a wait that runs out raises the status word that b200_attention_status reads,
// and the CTA leaves through the common teardown.
#include <cuda.h>
#include <math.h>
#include <stddef.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "../../include/b200_moe.h"

namespace b200 {
namespace fa {

constexpr int BM = 128;         // query rows per accumulator tile (tensor-memory lanes)
constexpr int BN = 128;         // keys per step
constexpr int QT = 2;           // query tiles per CTA
constexpr int SLAB = 16384;     // 128 rows x 64 bf16, one swizzled slab
constexpr int KV_SLOTS = 3;
constexpr int FWD_THREADS = 32 * (2 + 4 * QT);  // warp 0 loads, warp 1 issues the MMAs, 8 softmax warps
constexpr float LOG2E = 1.4426950408889634f;

enum { ST_ATTN_Q = 21, ST_ATTN_KV_EMPTY = 22, ST_ATTN_KV_FULL = 23, ST_ATTN_P = 24, ST_ATTN_S = 25, ST_ATTN_PV = 26 };

__device__ int g_attn_status = 0;

// The sequences one launch covers: work units (forward: tiles of 256 query rows; backward: blocks of 128 keys) are
// numbered through the sequences, first[s] being the first unit of sequence s and first[n] their number.
constexpr int MAX_SEQS = 48;
struct SeqTable {
  int n;
  int q_off[MAX_SEQS], Tq[MAX_SEQS], k_off[MAX_SEQS], Tk[MAX_SEQS], first[MAX_SEQS + 1];
};

struct FwdParams {
  CUtensorMap tmQ, tmK, tmV;  // [rows][heads * HD] bf16, boxes of 64 columns x 128 rows, 128-byte swizzle
  __nv_bfloat16 *O;
  float *lse;  // [heads][total_q]
  SeqTable seqs;
  int causal, group, total_q, num_q_heads;
  int64_t ldO;
  float scale;
  int *status;
};

struct FwdTail {
  uint64_t q_full, kv_full[KV_SLOTS], kv_empty[KV_SLOTS], s_full[QT], p_ready[QT], pv_full[QT];
  uint32_t tmem_base;
  int abort_flag;
};

template <int HD>
constexpr size_t fwd_smem_bytes() {
  // Q tiles, P tiles, the K / V ring, bookkeeping, and the slack that aligns the tiles to 1024 bytes
  return 1024 + (size_t)QT * BM * HD * 2 + (size_t)QT * BM * BN * 2 + (size_t)KV_SLOTS * BN * HD * 2 + sizeof(FwdTail);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// shared-memory accesses by 32-bit shared address (kept in program order among themselves)
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1) attn_fwd_sm100_kernel(const __grid_constant__ FwdParams p) {
  constexpr int KSL = HD / 64;               // 64-column slabs of a Q / K tile
  constexpr int Q_TILE = BM * HD * 2;        // bytes
  constexpr int P_TILE = BM * BN * 2;
  constexpr int KV_TILE = BN * HD * 2;
  constexpr uint32_t TMEM_COLS = 512;        // S_0, S_1 (BN columns each), then O'_0, O'_1 (HD columns each)
  extern __shared__ unsigned char attn_smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char *sQ = smem, *sP = sQ + QT * Q_TILE, *sKV = sP + QT * P_TILE;
  FwdTail *st = reinterpret_cast<FwdTail *>(sKV + KV_SLOTS * KV_TILE);
  volatile int *abort_flag = &st->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](uint64_t *b) { return ptx::smem_u32(b); };
  auto wait = [&](uint64_t *b, uint32_t par, int code) { return ptx::mbar_wait<false>(bar(b), par, abort_flag, p.status, code); };

  if (tid == 0) {
    ptx::mbar_init(bar(&st->q_full), 1);
    for (int s = 0; s < KV_SLOTS; s++) {
      ptx::mbar_init(bar(&st->kv_full[s]), 1);
      ptx::mbar_init(bar(&st->kv_empty[s]), 1);
    }
    for (int g = 0; g < QT; g++) {
      ptx::mbar_init(bar(&st->s_full[g]), 1);
      ptx::mbar_init(bar(&st->p_ready[g]), BM);
      ptx::mbar_init(bar(&st->pv_full[g]), 1);
    }
    st->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&st->tmem_base), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::tma_prefetch_desc(&p.tmQ);
    ptx::tma_prefetch_desc(&p.tmK);
    ptx::tma_prefetch_desc(&p.tmV);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;

  // one-dimensional grid, query tile major: the tiles with the most keys to visit (the last query rows under a causal
  // mask) start first on every head; neighbouring CTAs are the heads of one group and share their K / V tiles in L2
  const int unit = (int)blockIdx.x / p.num_q_heads, h = (int)blockIdx.x % p.num_q_heads, kvh = h / p.group;
  int sq = 0;
  while (unit >= p.seqs.first[sq + 1]) sq++;
  const int q_off = p.seqs.q_off[sq], Tq = p.seqs.Tq[sq], k_off = p.seqs.k_off[sq], Tk = p.seqs.Tk[sq];
  const int qt = p.seqs.first[sq + 1] - 1 - unit;  // of this sequence, the last tile first
  const int r0 = qt * QT * BM;
  const int shift = Tk - Tq;  // the last query is aligned with the last key
  int nkb[QT], nkb_max = 0;
#pragma unroll
  for (int g = 0; g < QT; g++) {
    const int first = r0 + g * BM;
    if (first >= Tq) {
      nkb[g] = 0;
    } else {
      const int last = min(first + BM - 1, Tq - 1);
      const int vis = p.causal ? min(Tk, last + 1 + shift) : Tk;
      nkb[g] = (vis + BN - 1) / BN;
    }
    nkb_max = max(nkb_max, nkb[g]);
  }

  if (warp == 0) {
    // ================= loads =================
    if (lane == 0) {
      int nq = 0;
      for (int g = 0; g < QT; g++) nq += nkb[g] > 0;
      ptx::mbar_arrive_expect_tx(bar(&st->q_full), (uint32_t)(nq * Q_TILE));
      for (int g = 0; g < QT; g++) {
        if (nkb[g] == 0) continue;
        for (int s = 0; s < KSL; s++)
          ptx::tma_load_2d(ptx::smem_u32(sQ + g * Q_TILE + s * SLAB), &p.tmQ, bar(&st->q_full), h * HD + s * 64,
                           q_off + r0 + g * BM);
      }
      for (int n = 0; n < 2 * nkb_max; n++) {  // K_0, V_0, K_1, V_1, ...
        const int slot = n % KV_SLOTS;
        const uint32_t par = (uint32_t)((n / KV_SLOTS) & 1);
        if (!wait(&st->kv_empty[slot], par ^ 1u, ST_ATTN_KV_EMPTY)) break;
        ptx::mbar_arrive_expect_tx(bar(&st->kv_full[slot]), (uint32_t)KV_TILE);
        const CUtensorMap *m = (n & 1) ? &p.tmV : &p.tmK;
        for (int s = 0; s < KSL; s++)
          ptx::tma_load_2d(ptx::smem_u32(sKV + slot * KV_TILE + s * SLAB), m, bar(&st->kv_full[slot]), kvh * HD + s * 64,
                           k_off + (n >> 1) * BN);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issue =================
    if (lane == 0 && nkb_max > 0) {
      const uint32_t idesc_s = ptx::make_idesc_bf16(BM, BN, 0, 0);
      const uint32_t idesc_pv = ptx::make_idesc_bf16(BM, HD, 0, 1);  // V is read with its head dimension contiguous
      const uint32_t q_base = ptx::smem_u32(sQ), p_base = ptx::smem_u32(sP), kv_base = ptx::smem_u32(sKV);
      auto issue_s = [&](int g, int slot) {
#pragma unroll
        for (int k16 = 0; k16 < HD / 16; k16++) {
          const uint32_t off = (uint32_t)((k16 >> 2) * SLAB + (k16 & 3) * 32);
          ptx::umma_bf16(tmem_base + (uint32_t)(g * BN), ptx::make_smem_desc(q_base + g * Q_TILE + off, 0, 1024),
                         ptx::make_smem_desc(kv_base + slot * KV_TILE + off, 0, 1024), idesc_s, k16 > 0);
        }
        ptx::umma_commit(bar(&st->s_full[g]));
      };
      auto issue_pv = [&](int g, int slot, bool first) {
#pragma unroll
        for (int k16 = 0; k16 < BN / 16; k16++) {
          const uint32_t a_off = (uint32_t)((k16 >> 2) * SLAB + (k16 & 3) * 32);
          ptx::umma_bf16(tmem_base + (uint32_t)(QT * BN + g * HD), ptx::make_smem_desc(p_base + g * P_TILE + a_off, 0, 1024),
                         ptx::make_smem_desc(kv_base + slot * KV_TILE + k16 * 2048, SLAB, 1024), idesc_pv, !first || k16 > 0);
        }
        ptx::umma_commit(bar(&st->pv_full[g]));
      };
      bool alive = wait(&st->q_full, 0, ST_ATTN_Q) && wait(&st->kv_full[0], 0, ST_ATTN_KV_FULL);
      if (alive) {
        ptx::tc_fence_after();
        for (int g = 0; g < QT; g++)
          if (nkb[g] > 0) issue_s(g, 0);
        ptx::umma_commit(bar(&st->kv_empty[0]));
      }
      for (int j = 0; alive && j < nkb_max; j++) {
        const int nv = 2 * j + 1, nk = 2 * j + 2;
        const bool has_next = j + 1 < nkb_max;
        if (!wait(&st->kv_full[nv % KV_SLOTS], (uint32_t)((nv / KV_SLOTS) & 1), ST_ATTN_KV_FULL)) break;
        if (has_next && !wait(&st->kv_full[nk % KV_SLOTS], (uint32_t)((nk / KV_SLOTS) & 1), ST_ATTN_KV_FULL)) break;
        for (int g = 0; g < QT; g++) {
          if (j >= nkb[g]) continue;
          // P_g of this step is in shared memory, the group has read all of S_g and, if the row maxima grew, rescaled O_g
          if (!wait(&st->p_ready[g], (uint32_t)(j & 1), ST_ATTN_P)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          issue_pv(g, nv % KV_SLOTS, j == 0);
          if (j + 1 < nkb[g]) issue_s(g, nk % KV_SLOTS);
        }
        if (!alive) break;
        ptx::umma_commit(bar(&st->kv_empty[nv % KV_SLOTS]));
        if (has_next) ptx::umma_commit(bar(&st->kv_empty[nk % KV_SLOTS]));
      }
    }
    __syncwarp();
  } else {
    // ================= softmax and output (a thread per query row) =================
    const int g = (warp - 2) >> 2, quarter = warp & 3;  // tensor-memory lanes a warp may read: 32 * (warp % 4) ...
    const int trow = quarter * 32 + lane;
    const int row = r0 + g * BM + trow;  // position of the query in its sequence
    const int limit = p.causal ? min(Tk, row + 1 + shift) : Tk;  // keys this row sees
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)(g * BN), o_addr = lane_addr + (uint32_t)(QT * BN + g * HD);
    const uint32_t p_addr = ptx::smem_u32(sP + g * P_TILE + trow * 128);
    const float c = p.scale * LOG2E;
    // m is the score the probabilities are taken against: the row maximum of the first key block, raised (with the sum
    // and the output in tensor memory rescaled) only when a later block's maximum exceeds it by more than 2^8
    float m = -INFINITY, l = 0.0f;
    for (int j = 0; j < nkb[g]; j++) {
      if (!wait(&st->s_full[g], (uint32_t)(j & 1), ST_ATTN_S)) goto teardown;
      ptx::tc_fence_after();
      const int lim = limit - j * BN;  // columns below lim are visible
      // first pass over the scores: the row maximum (two chunks of 32 columns in flight)
      uint32_t ra[32], rb[32];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto max32 = [&](const uint32_t *v, int c4) {
        if (lim >= (c4 + 1) * 32) {
#pragma unroll
          for (int i = 0; i < 32; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) mx4[i & 3] = fmaxf(mx4[i & 3], c4 * 32 + i < lim ? __uint_as_float(v[i]) : -INFINITY);
        }
      };
      ptx::tmem_ld32(s_addr, ra);
      ptx::tmem_ld32(s_addr + 32, rb);
      ptx::tmem_ld_wait();
      max32(ra, 0);
      ptx::tmem_ld32(s_addr + 64, ra);
      max32(rb, 1);
      ptx::tmem_ld32(s_addr + 96, rb);
      ptx::tmem_ld_wait();
      max32(ra, 2);
      max32(rb, 3);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      if (j == 0) {
        m = mx;
      } else {
        const bool grow = (mx - m) * c > 8.0f;
        if (__any_sync(0xffffffffu, grow)) {  // tensor-memory accesses are warp-wide: every lane takes part
          const float m_new = grow ? mx : m;
          const float alpha = ex2((m - m_new) * c);  // 1 for the lanes that keep their offset
          if (!wait(&st->pv_full[g], (uint32_t)((j - 1) & 1), ST_ATTN_PV)) goto teardown;
          ptx::tc_fence_after();
#pragma unroll
          for (int c4 = 0; c4 < HD / 32; c4++) {
            ptx::tmem_ld32(o_addr + c4 * 32, ra);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
            ptx::tmem_st32(o_addr + c4 * 32, ra);
          }
          ptx::tmem_st_wait();
          l *= alpha;
          m = m_new;
        }
      }
      // a row that has seen no key yet keeps m = -inf: its probabilities are exp2(-inf) = 0 against a zero offset
      const float mc = (m == -INFINITY) ? 0.0f : m * c;
      // second pass: the probabilities, their sum, and P as bf16 in the layout the P V product reads
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      auto probs32 = [&](const uint32_t *v, int c4) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          float pr[8];
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float e = ex2(fmaf(__uint_as_float(v[q * 8 + i]), c, -mc));
            pr[i] = (c4 * 32 + q * 8 + i < lim) ? e : 0.0f;
            sum4[i & 3] += pr[i];
          }
          // keys c4*32 + q*8 .. +7 of this row: slab c4 / 2, 16-byte chunk (c4 % 2) * 4 + q, swizzled with the row
          sts128(p_addr + (uint32_t)((c4 >> 1) * SLAB + ((((c4 & 1) * 4 + q) ^ (trow & 7)) * 16)), pack8(pr));
        }
      };
      ptx::tmem_ld32(s_addr, ra);
      ptx::tmem_ld32(s_addr + 32, rb);
      ptx::tmem_ld_wait();
      probs32(ra, 0);
      ptx::tmem_ld32(s_addr + 64, ra);
      probs32(rb, 1);
      ptx::tmem_ld32(s_addr + 96, rb);
      ptx::tmem_ld_wait();
      probs32(ra, 2);
      probs32(rb, 3);
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(&st->p_ready[g]));
    }
    if (nkb[g] > 0) {
      if (!wait(&st->pv_full[g], (uint32_t)((nkb[g] - 1) & 1), ST_ATTN_PV)) goto teardown;
      ptx::tc_fence_after();
      const float inv = l > 0.0f ? __fdividef(1.0f, l) : 0.0f;
      __nv_bfloat16 *o = p.O + (int64_t)(q_off + row) * p.ldO + (int64_t)h * HD;
#pragma unroll
      for (int c4 = 0; c4 < HD / 32; c4++) {
        uint32_t r[32];
        ptx::tmem_ld32(o_addr + c4 * 32, r);
        ptx::tmem_ld_wait();
        if (row < Tq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float v[8];
#pragma unroll
            for (int t = 0; t < 8; t++) v[t] = __uint_as_float(r[i + t]) * inv;
            *reinterpret_cast<uint4 *>(o + c4 * 32 + i) = pack8(v);
          }
        }
      }
      if (row < Tq) p.lse[(int64_t)h * p.total_q + q_off + row] = l > 0.0f ? m * p.scale + logf(l) : -INFINITY;
    }
  }

teardown:
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------
// Backward (head_dim 128). One CTA per (block of 128 keys, key/value head) of one sequence; it walks the query heads of
// the group and the 128-row query blocks that see its keys. K and V stay in shared memory; Q and dO tiles pass through
// a three-slot ring. Per step, with the key rows on the tensor-memory lanes:
//     S^T = K Q^T,  dP^T = V dO^T                       (fp32, tensor memory)
//     P^T = exp2(S^T * scale * log2 e - lse * log2 e),  dS^T = P^T o (dP^T - delta)   (threads; bf16 into shared memory)
//     dV += P^T dO,  dK += dS^T Q                       (accumulated in tensor memory over all steps of the CTA)
//     dQ^T = K^T dS^T                                   (tensor memory, over the columns S^T occupied)
// dQ^T is staged in shared memory and added to an fp32 accumulator in global memory by two tiled bulk reductions per
// step (cp.reduce.async.bulk.tensor, 64 queries x 128 dims fp32 each) that a cast kernel rounds once; dK (times the softmax scale) and dV are rounded once at the end of the CTA. The Q and dO tiles are
// read by the tensor core both ways round - as [queries x dims] for S^T / dP^T and as [dims x queries] for dK / dV -
// from the same swizzled bytes, and so are K and dS^T for dQ^T.
// ---------------------------------------------------------------------------------------
constexpr int BWD_THREADS = 32 * 10;  // warp 0 loads, warp 1 issues the MMAs, 8 warps for the element-wise work
constexpr int BWD_HD = 128;
constexpr int BWD_TILE = 128 * BWD_HD * 2;
constexpr int RING = 3;

enum { ST_BWD_KV = 31, ST_BWD_RING_EMPTY = 32, ST_BWD_RING_FULL = 33, ST_BWD_S = 34, ST_BWD_DP = 35, ST_BWD_P = 36,
       ST_BWD_DS = 37, ST_BWD_DQ = 38, ST_BWD_DQ_EMPTY = 39, ST_BWD_ACC = 40, ST_BWD_STATS = 41, ST_BWD_STAGE = 42 };

struct BwdParams {
  CUtensorMap tmQ, tmK, tmV, tmdO;
  CUtensorMap tmdQ;  // the fp32 dQ accumulator [total_q][heads * 128], boxes of 128 x 64 rows, no swizzle
  const float *lse, *delta;  // [heads][total_q]
  float *dQacc;              // [total_q][heads * 128] fp32, zeroed by the caller
  __nv_bfloat16 *dK, *dV;
  SeqTable seqs;
  int causal, group, total_q, num_kv_heads;
  int64_t ldQ, ldK;
  float scale;
  int *status;
};

struct BwdTail {
  uint64_t kv_full, ring_full[RING], ring_empty[RING], s_full, dp_full, p_ready, ds_ready, dq_full, dq_read, dk_done, stage_ready, dq_empty, dq_empty_b, acc_full,
      stats0;
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) float stats[2][128];  // lse * log2 e and delta of the step's 128 queries (read 16 bytes at a time)
};

constexpr size_t bwd_smem_bytes() { return 1024 + (size_t)(4 + RING) * BWD_TILE + sizeof(BwdTail); }
static_assert(bwd_smem_bytes() <= 232448, "the backward kernel's shared memory exceeds what one CTA can be given");
static_assert(offsetof(BwdTail, stats) % 16 == 0, "the statistics are read with 16-byte loads");

__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_sm100_kernel(const __grid_constant__ BwdParams p) {
  constexpr int HD = BWD_HD;
  constexpr uint32_t TMEM_COLS = 512;  // S^T / dQ^T, dP^T, dK, dV: 128 columns each
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DK = 256, COL_DV = 384;
  extern __shared__ unsigned char attn_smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char *sK = smem, *sV = sK + BWD_TILE, *sPT = sV + BWD_TILE, *sDST = sPT + BWD_TILE, *sRing = sDST + BWD_TILE;
  BwdTail *st = reinterpret_cast<BwdTail *>(sRing + RING * BWD_TILE);
  volatile int *abort_flag = &st->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](uint64_t *b) { return ptx::smem_u32(b); };
  auto wait = [&](uint64_t *b, uint32_t par, int code) { return ptx::mbar_wait<false>(bar(b), par, abort_flag, p.status, code); };

  if (tid == 0) {
    ptx::mbar_init(bar(&st->kv_full), 1);
    for (int s = 0; s < RING; s++) {
      ptx::mbar_init(bar(&st->ring_full[s]), 1);
      ptx::mbar_init(bar(&st->ring_empty[s]), 1);
    }
    ptx::mbar_init(bar(&st->s_full), 1);
    ptx::mbar_init(bar(&st->dp_full), 1);
    ptx::mbar_init(bar(&st->p_ready), 256);
    ptx::mbar_init(bar(&st->ds_ready), 256);
    ptx::mbar_init(bar(&st->dq_full), 1);
    ptx::mbar_init(bar(&st->dq_read), 256);
    ptx::mbar_init(bar(&st->dk_done), 1);
    ptx::mbar_init(bar(&st->stage_ready), 256);
    ptx::mbar_init(bar(&st->dq_empty), 1);
    ptx::mbar_init(bar(&st->dq_empty_b), 1);
    ptx::mbar_init(bar(&st->acc_full), 1);
    ptx::mbar_init(bar(&st->stats0), 256);
    st->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&st->tmem_base), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::tma_prefetch_desc(&p.tmQ);
    ptx::tma_prefetch_desc(&p.tmK);
    ptx::tma_prefetch_desc(&p.tmV);
    ptx::tma_prefetch_desc(&p.tmdO);
    ptx::tma_prefetch_desc(&p.tmdQ);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;

  // one-dimensional grid, key block major: the key blocks most queries see (the first ones, under a causal mask) start
  // first on every key/value head, the short ones fill in behind them
  const int unit = (int)blockIdx.x / p.num_kv_heads, kvh = (int)blockIdx.x % p.num_kv_heads;
  int sq = 0;
  while (unit >= p.seqs.first[sq + 1]) sq++;
  const int q_off = p.seqs.q_off[sq], Tq = p.seqs.Tq[sq], k_off = p.seqs.k_off[sq], Tk = p.seqs.Tk[sq];
  const int kb = unit - p.seqs.first[sq];
  const int shift = Tk - Tq;
  const int nqb = (Tq + BM - 1) / BM;
  const int qb_start = p.causal ? max(0, kb * BN - shift) / BM : 0;
  const int per_head = nqb - qb_start;
  const int n_steps = per_head > 0 ? per_head * p.group : 0;

  if (warp == 0) {
    // ================= loads =================
    if (lane == 0 && n_steps > 0) {
      ptx::mbar_arrive_expect_tx(bar(&st->kv_full), (uint32_t)(2 * BWD_TILE));
      for (int s = 0; s < HD / 64; s++) {
        ptx::tma_load_2d(ptx::smem_u32(sK + s * SLAB), &p.tmK, bar(&st->kv_full), kvh * HD + s * 64, k_off + kb * BN);
        ptx::tma_load_2d(ptx::smem_u32(sV + s * SLAB), &p.tmV, bar(&st->kv_full), kvh * HD + s * 64, k_off + kb * BN);
      }
      for (int n = 0; n < 2 * n_steps; n++) {  // Q_0, dO_0, Q_1, dO_1, ...
        const int i = n >> 1, h = kvh * p.group + i / per_head, qb = qb_start + i % per_head;
        const int slot = n % RING;
        const uint32_t par = (uint32_t)((n / RING) & 1);
        if (!wait(&st->ring_empty[slot], par ^ 1u, ST_BWD_RING_EMPTY)) break;
        ptx::mbar_arrive_expect_tx(bar(&st->ring_full[slot]), (uint32_t)BWD_TILE);
        const CUtensorMap *m = (n & 1) ? &p.tmdO : &p.tmQ;
        for (int s = 0; s < HD / 64; s++)
          ptx::tma_load_2d(ptx::smem_u32(sRing + slot * BWD_TILE + s * SLAB), m, bar(&st->ring_full[slot]), h * HD + s * 64,
                           q_off + qb * BM);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issue =================
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_kk = ptx::make_idesc_bf16(128, 128, 0, 0);  // both operands with the reduction contiguous
      const uint32_t idesc_km = ptx::make_idesc_bf16(128, 128, 0, 1);  // B read the other way round
      const uint32_t idesc_mm = ptx::make_idesc_bf16(128, 128, 1, 1);  // both
      const uint32_t k_base = ptx::smem_u32(sK), v_base = ptx::smem_u32(sV), pt_base = ptx::smem_u32(sPT),
                     dst_base = ptx::smem_u32(sDST), ring_base = ptx::smem_u32(sRing);
      // operand with the reduction index contiguous (rows = M or N), 16 reduction elements per step
      auto kmaj = [&](uint32_t base, int k16) { return ptx::make_smem_desc(base + (uint32_t)((k16 >> 2) * SLAB + (k16 & 3) * 32), 0, 1024); };
      // the same bytes read with the rows as the reduction index
      auto mnmaj = [&](uint32_t base, int k16) { return ptx::make_smem_desc(base + (uint32_t)(k16 * 2048), SLAB, 1024); };
      bool alive = wait(&st->kv_full, 0, ST_BWD_KV);
      for (int i = 0; alive && i < n_steps; i++) {
        const int nq = 2 * i, nd = 2 * i + 1;
        const uint32_t q_tile = ring_base + (uint32_t)((nq % RING) * BWD_TILE), do_tile = ring_base + (uint32_t)((nd % RING) * BWD_TILE);
        const uint32_t par = (uint32_t)(i & 1);
        if (!wait(&st->ring_full[nq % RING], (uint32_t)((nq / RING) & 1), ST_BWD_RING_FULL)) break;
        if (i > 0 && !wait(&st->dq_read, par ^ 1u, ST_BWD_DQ_EMPTY)) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < HD / 16; k16++)
          ptx::umma_bf16(tmem_base + COL_S, kmaj(k_base, k16), kmaj(q_tile, k16), idesc_kk, k16 > 0);
        ptx::umma_commit(bar(&st->s_full));
        if (!wait(&st->ring_full[nd % RING], (uint32_t)((nd / RING) & 1), ST_BWD_RING_FULL)) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < HD / 16; k16++)
          ptx::umma_bf16(tmem_base + COL_DP, kmaj(v_base, k16), kmaj(do_tile, k16), idesc_kk, k16 > 0);
        ptx::umma_commit(bar(&st->dp_full));
        if (!wait(&st->p_ready, par, ST_BWD_P)) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < BM / 16; k16++)
          ptx::umma_bf16(tmem_base + COL_DV, kmaj(pt_base, k16), mnmaj(do_tile, k16), idesc_km, (i > 0 || k16 > 0));
        ptx::umma_commit(bar(&st->ring_empty[nd % RING]));
        if (!wait(&st->ds_ready, par, ST_BWD_DS)) break;
        ptx::tc_fence_after();
        // dQ^T first: the threads fetch it from tensor memory (and release those columns for the next S^T) while dK
        // runs; dk_done then says that dS^T and P^T are done with - the dQ staging lies over them
#pragma unroll
        for (int k16 = 0; k16 < BN / 16; k16++)
          ptx::umma_bf16(tmem_base + COL_S, mnmaj(k_base, k16), mnmaj(dst_base, k16), idesc_mm, k16 > 0);
        ptx::umma_commit(bar(&st->dq_full));
#pragma unroll
        for (int k16 = 0; k16 < BM / 16; k16++)
          ptx::umma_bf16(tmem_base + COL_DK, kmaj(dst_base, k16), mnmaj(q_tile, k16), idesc_km, (i > 0 || k16 > 0));
        ptx::umma_commit(bar(&st->ring_empty[nq % RING]));
        ptx::umma_commit(bar(&st->dk_done));
        if (i == n_steps - 1) ptx::umma_commit(bar(&st->acc_full));
      }
    }
    __syncwarp();
  } else if (n_steps > 0) {
    // ================= element-wise work: a thread per (tensor-memory lane, half of the columns) =================
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int trow = quarter * 32 + lane;
    const int key = kb * BN + trow;  // position of this lane's key in its sequence (steps 1-2 and the end)
    const bool key_ok = key < Tk;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 64);
    const uint32_t pt_addr = ptx::smem_u32(sPT + half * SLAB + trow * 128), dst_addr = ptx::smem_u32(sDST + half * SLAB + trow * 128);
    const uint32_t stats_addr = ptx::smem_u32(&st->stats[0][0]), stage_addr = ptx::smem_u32(sPT);
    const float c = p.scale * LOG2E;
    const int st_t = tid - 64;  // 0 .. 255
    // lse * log2 e (threads 0-127) or delta (128-255) of query st_t % 128 of step `step`: fetched a step ahead
    auto stat_load = [&](int step) {
      const int hh = kvh * p.group + step / per_head, qa = (qb_start + step % per_head) * BM + (st_t & 127);
      if (step >= n_steps || qa >= Tq) return 0.0f;
      const int64_t at = (int64_t)hh * p.total_q + q_off + qa;
      return st_t < 128 ? p.lse[at] * LOG2E : p.delta[at];
    };
    st->stats[st_t >> 7][st_t & 127] = stat_load(0);
    ptx::mbar_arrive(bar(&st->stats0));
    if (!wait(&st->stats0, 0, ST_BWD_STATS)) goto teardown;
    for (int i = 0; i < n_steps; i++) {
      const int h = kvh * p.group + i / per_head, qb = qb_start + i % per_head;
      const uint32_t par = (uint32_t)(i & 1);
      const int q0 = qb * BM;
      // every thread has left the step before: its statistics for this step are written
      if (i > 0 && !wait(&st->stage_ready, par ^ 1u, ST_BWD_STAGE)) goto teardown;
      const float stat_next = stat_load(i + 1);  // in flight while this step computes
      // queries of this step the lane's key is visible to: columns lo_rel <= col < hi_rel
      const int lo_rel = (key_ok ? (p.causal ? key - shift : 0) : (1 << 30)) - q0, hi_rel = Tq - q0;
      float prob[64];
      uint32_t r[32];
      if (!wait(&st->s_full, par, ST_BWD_S)) goto teardown;
      ptx::tc_fence_after();
#pragma unroll
      for (int c2 = 0; c2 < 2; c2++) {
        ptx::tmem_ld32(lane_addr + COL_S + c2 * 32, r);
        float4 l4[8];
#pragma unroll
        for (int q = 0; q < 8; q++) l4[q] = lds128(stats_addr + (uint32_t)((half * 64 + c2 * 32 + q * 4) * 4));
        ptx::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t++) {
          const int col = half * 64 + c2 * 32 + t;
          const float l2 = (t & 3) == 0 ? l4[t >> 2].x : (t & 3) == 1 ? l4[t >> 2].y : (t & 3) == 2 ? l4[t >> 2].z : l4[t >> 2].w;
          const float pv = ex2(fmaf(__uint_as_float(r[t]), c, -l2));
          prob[c2 * 32 + t] = (col >= lo_rel && col < hi_rel) ? pv : 0.0f;
        }
      }
      // P^T goes where the first half of the dQ staging area lies: the bulk reduction of the step before has to have
      // read it (it drained while the probabilities above were formed)
      if (i > 0) {
        if (st_t == 0) {
          ptx::bulk_wait_group_read1();
          ptx::mbar_arrive(bar(&st->dq_empty));
        }
        if (!wait(&st->dq_empty, par ^ 1u, ST_BWD_DQ_EMPTY)) goto teardown;
      }
#pragma unroll
      for (int q = 0; q < 8; q++) sts128(pt_addr + (uint32_t)(((q ^ (trow & 7))) * 16), pack8(prob + q * 8));
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(&st->p_ready));
      // the second half of the staging area lies over dS^T: its reduction of the step before has to have read it
      if (i > 0) {
        if (st_t == 0) {
          ptx::bulk_wait_group_read0();
          ptx::mbar_arrive(bar(&st->dq_empty_b));
        }
        if (!wait(&st->dq_empty_b, par ^ 1u, ST_BWD_DQ_EMPTY)) goto teardown;
      }
      if (!wait(&st->dp_full, par, ST_BWD_DP)) goto teardown;
      ptx::tc_fence_after();
#pragma unroll
      for (int c2 = 0; c2 < 2; c2++) {
        ptx::tmem_ld32(lane_addr + COL_DP + c2 * 32, r);
        float4 d4[8];
#pragma unroll
        for (int q = 0; q < 8; q++) d4[q] = lds128(stats_addr + (uint32_t)((128 + half * 64 + c2 * 32 + q * 4) * 4));
        ptx::tmem_ld_wait();
        float ds[32];
#pragma unroll
        for (int t = 0; t < 32; t++) {
          const float dl = (t & 3) == 0 ? d4[t >> 2].x : (t & 3) == 1 ? d4[t >> 2].y : (t & 3) == 2 ? d4[t >> 2].z : d4[t >> 2].w;
          // the probability as the tensor core saw it (bf16); zero where masked, whatever dP holds there
          const float pb = bf16_round(prob[c2 * 32 + t]);
          ds[t] = pb == 0.0f ? 0.0f : pb * (__uint_as_float(r[t]) - dl);
        }
#pragma unroll
        for (int q = 0; q < 4; q++) sts128(dst_addr + (uint32_t)((((c2 * 4 + q) ^ (trow & 7))) * 16), pack8(ds + q * 8));
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(&st->ds_ready));
      // once every thread is past its last read of this step's statistics, the next step's take their place
      if (!wait(&st->ds_ready, par, ST_BWD_DS)) goto teardown;
      st->stats[st_t >> 7][st_t & 127] = stat_next;
      // dQ^T: this lane is head dimension trow, the columns are the step's queries. It is staged as [query][dim] fp32
      // in shared memory (once dk_done says that the MMAs reading P^T and dS^T are finished) and added to the
      // accumulator in global memory by tiled bulk reductions.
      if (!wait(&st->dq_full, par, ST_BWD_DQ)) goto teardown;
      ptx::tc_fence_after();
      uint32_t r2[32];
      ptx::tmem_ld32(lane_addr + COL_S, r);
      ptx::tmem_ld32(lane_addr + COL_S + 32, r2);
      ptx::tmem_ld_wait();
      // the tensor core may overwrite these columns with the next S^T from here on
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(&st->dq_read));
      if (!wait(&st->dk_done, par, ST_BWD_DQ)) goto teardown;
#pragma unroll
      for (int t = 0; t < 32; t++) {
        sts32(stage_addr + (uint32_t)(((half * 64 + t) * HD + trow) * 4), __uint_as_float(r[t]) * p.scale);
        sts32(stage_addr + (uint32_t)(((half * 64 + 32 + t) * HD + trow) * 4), __uint_as_float(r2[t]) * p.scale);
      }
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(bar(&st->stage_ready));
      if (st_t == 0) {
        // two tiled reductions add the [128 queries][128 dims] block, 64 queries each (rows past the end of the sequence
        // hold zeros: their dS is masked; rows past the end of the array are clipped). Neither is waited for here: the
        // first half has to be read before the next step's P^T is stored, the second before its dS^T, and both drain
        // while that step's probabilities are formed.
        if (!wait(&st->stage_ready, par, ST_BWD_STAGE)) goto teardown;
        ptx::tma_reduce_add_2d(&p.tmdQ, stage_addr, h * HD, q_off + q0);
        ptx::bulk_commit_group();
        ptx::tma_reduce_add_2d(&p.tmdQ, stage_addr + 64 * HD * 4, h * HD, q_off + q0 + 64);
        ptx::bulk_commit_group();
      }
    }
    ptx::bulk_wait_group0();
    // dK and dV of this key block: one rounding
    if (!wait(&st->acc_full, 0, ST_BWD_ACC)) goto teardown;
    ptx::tc_fence_after();
    {
      uint32_t r[32];
      __nv_bfloat16 *dk = p.dK + (int64_t)(k_off + key) * p.ldK + (int64_t)kvh * HD + half * 64;
      __nv_bfloat16 *dv = p.dV + (int64_t)(k_off + key) * p.ldK + (int64_t)kvh * HD + half * 64;
#pragma unroll
      for (int c2 = 0; c2 < 2; c2++) {
        float v[32];
        ptx::tmem_ld32(lane_addr + COL_DK + c2 * 32, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t++) v[t] = __uint_as_float(r[t]) * p.scale;
        if (key_ok) {
#pragma unroll
          for (int q = 0; q < 4; q++) *reinterpret_cast<uint4 *>(dk + c2 * 32 + q * 8) = pack8(v + q * 8);
        }
        ptx::tmem_ld32(lane_addr + COL_DV + c2 * 32, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t++) v[t] = __uint_as_float(r[t]);
        if (key_ok) {
#pragma unroll
          for (int q = 0; q < 4; q++) *reinterpret_cast<uint4 *>(dv + c2 * 32 + q * 8) = pack8(v + q * 8);
        }
      }
    }
  }

teardown:
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// delta[h][row] = sum_d dO[row, h, d] * O[row, h, d]; a warp per (row, head)
__global__ void __launch_bounds__(256) attn_delta_all_kernel(int total_q, int heads, int head_dim,
                                                             const __nv_bfloat16 *__restrict__ dO,
                                                             const __nv_bfloat16 *__restrict__ O, float *__restrict__ delta) {
  const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= (int64_t)total_q * heads) return;
  const int row = (int)(w / heads), h = (int)(w - (int64_t)row * heads);
  const int64_t at = ((int64_t)row * heads + h) * head_dim;
  float acc = 0.0f;
  for (int c = (threadIdx.x & 31) * 4; c < head_dim; c += 128) {
    const uint2 a = *reinterpret_cast<const uint2 *>(dO + at + c), b = *reinterpret_cast<const uint2 *>(O + at + c);
    acc += bf16lo(a.x) * bf16lo(b.x) + bf16hi(a.x) * bf16hi(b.x) + bf16lo(a.y) * bf16lo(b.y) + bf16hi(a.y) * bf16hi(b.y);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) delta[(int64_t)h * total_q + row] = acc;
}

// fp32 -> bf16, eight elements per thread
__global__ void __launch_bounds__(256) attn_round_kernel(int64_t n8, const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4 *>(src)[2 * i], b = reinterpret_cast<const float4 *>(src)[2 * i + 1];
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  reinterpret_cast<uint4 *>(dst)[i] = pack8(v);
}

}  // namespace fa
}  // namespace b200

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
using namespace b200;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// bf16 [rows][cols] with a row pitch of `cols` elements; boxes of 64 columns x 128 rows, 128-byte swizzle, rows past
// the end read as zeros
int rows_map(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "attention: cuTensorMapEncodeTiled is not available from this driver");
  B200_REQUIRE(b200_aligned16(base) && (cols * 2) % 16 == 0, "attention: tensors must be 16-byte aligned with a 16-byte row pitch");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "attention: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

constexpr int MAX_DEVICES = 64;

int *attn_status_ptr() {
  static int *ptr[MAX_DEVICES];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  if (!ptr[dev] && cudaGetSymbolAddress((void **)&ptr[dev], fa::g_attn_status) != cudaSuccess) ptr[dev] = nullptr;
  return ptr[dev];
}

template <int HD>
int launch_fwd(const fa::FwdParams &p, int units, int num_q_heads, cudaStream_t s) {
  static bool attr_set[MAX_DEVICES];
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "attention: device ordinal %d is out of range", dev);
  constexpr size_t smem = fa::fwd_smem_bytes<HD>();
  if (!attr_set[dev]) {
    B200_CUDA(cudaFuncSetAttribute(fa::attn_fwd_sm100_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev] = true;
  }
  fa::attn_fwd_sm100_kernel<HD><<<(unsigned)(units * num_q_heads), fa::FWD_THREADS, smem, s>>>(p);
  B200_CHECK_LAUNCH("attention_fwd (fused)");
  return 0;
}

// Fills the table with the next sequences that have work (at most MAX_SEQS), starting at *next; units_of gives a
// sequence's number of work units. Returns the units in the table.
template <typename F>
int fill_table(fa::SeqTable &t, int *next, int num_seqs, const int *q_off, const int *q_len, const int *k_off,
               const int *k_len, F units_of) {
  t.n = 0;
  t.first[0] = 0;
  while (*next < num_seqs && t.n < fa::MAX_SEQS) {
    const int sq = (*next)++;
    const int u = units_of(sq);
    if (u == 0) continue;
    t.q_off[t.n] = q_off[sq];
    t.Tq[t.n] = q_len[sq];
    t.k_off[t.n] = k_off[sq];
    t.Tk[t.n] = k_len[sq];
    t.first[t.n + 1] = t.first[t.n] + u;
    t.n++;
  }
  for (int i = t.n + 1; i <= fa::MAX_SEQS; i++) t.first[i] = t.first[t.n];
  return t.first[t.n];
}

}  // namespace

namespace b200 {

bool attn_fused_supported(int head_dim) { return head_dim == 64 || head_dim == 128; }

// Forward over every sequence of the packed batch (one launch per 48 sequences); arguments as b200_attention_fwd.
int attn_fused_fwd(int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len, const int *k_off,
                   const int *k_len, int num_q_heads, int num_kv_heads, int head_dim, const void *Q, const void *K,
                   const void *V, void *O, float *lse, int is_causal, cudaStream_t s) {
  fa::FwdParams p;
  const uint64_t Dq = (uint64_t)num_q_heads * head_dim, Dk = (uint64_t)num_kv_heads * head_dim;
  if (rows_map(&p.tmQ, Q, (uint64_t)total_q, Dq) || rows_map(&p.tmK, K, (uint64_t)total_k, Dk) ||
      rows_map(&p.tmV, V, (uint64_t)total_k, Dk))
    return -1;
  p.O = (__nv_bfloat16 *)O;
  p.lse = lse;
  p.causal = is_causal;
  p.group = num_q_heads / num_kv_heads;
  p.total_q = total_q;
  p.ldO = (int64_t)Dq;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.status = attn_status_ptr();
  B200_REQUIRE(p.status != nullptr, "attention: the status word of this device is not reachable");
  p.num_q_heads = num_q_heads;
  // one launch per MAX_SEQS sequences of the packed batch
  for (int next = 0; next < num_seqs;) {
    const int units = fill_table(p.seqs, &next, num_seqs, q_off, q_len, k_off, k_len,
                                 [&](int sq) { return (q_len[sq] + fa::QT * fa::BM - 1) / (fa::QT * fa::BM); });
    if (units == 0) continue;
    if ((head_dim == 128 ? launch_fwd<128>(p, units, num_q_heads, s) : launch_fwd<64>(p, units, num_q_heads, s)) != 0) return -1;
  }
  return 0;
}

bool attn_fused_bwd_supported(int head_dim) { return head_dim == fa::BWD_HD; }

// bytes of workspace the fused backward needs: the fp32 dQ accumulator and delta
uint64_t attn_fused_bwd_workspace(int total_q, int num_q_heads, int head_dim) {
  auto up = [](uint64_t v) { return (v + 255) / 256 * 256; };
  return up((uint64_t)total_q * num_q_heads * head_dim * 4) + up((uint64_t)total_q * num_q_heads * 4);
}

// Backward over every sequence of the packed batch; arguments as b200_attention_bwd, the workspace sized by
// attn_fused_bwd_workspace. dQ, dK and dV are overwritten.
int attn_fused_bwd(int num_seqs, int total_q, int total_k, const int *q_off, const int *q_len, const int *k_off,
                   const int *k_len, int num_q_heads, int num_kv_heads, int head_dim, const void *Q, const void *K,
                   const void *V, const void *O, const float *lse, const void *dO, void *dQ, void *dK, void *dV,
                   int is_causal, void *workspace, cudaStream_t s) {
  fa::BwdParams p;
  const uint64_t Dq = (uint64_t)num_q_heads * head_dim, Dk = (uint64_t)num_kv_heads * head_dim;
  if (rows_map(&p.tmQ, Q, (uint64_t)total_q, Dq) || rows_map(&p.tmdO, dO, (uint64_t)total_q, Dq) ||
      rows_map(&p.tmK, K, (uint64_t)total_k, Dk) || rows_map(&p.tmV, V, (uint64_t)total_k, Dk))
    return -1;
  const uint64_t acc_bytes = ((uint64_t)total_q * Dq * 4 + 255) / 256 * 256;
  p.dQacc = (float *)workspace;
  {
    EncodeTiledFn fn = encode_fn();
    B200_REQUIRE(fn != nullptr, "attention: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {Dq, (cuuint64_t)total_q};
    cuuint64_t strides[1] = {Dq * 4};
    cuuint32_t box[2] = {128, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&p.tmdQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, workspace, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(r == CUDA_SUCCESS, "attention: cuTensorMapEncodeTiled (dQ accumulator) failed with code %d", (int)r);
  }
  float *delta = (float *)((unsigned char *)workspace + acc_bytes);
  p.delta = delta;
  p.lse = lse;
  p.dK = (__nv_bfloat16 *)dK;
  p.dV = (__nv_bfloat16 *)dV;
  p.causal = is_causal;
  p.group = num_q_heads / num_kv_heads;
  p.num_kv_heads = num_kv_heads;
  p.total_q = total_q;
  p.ldQ = (int64_t)Dq;
  p.ldK = (int64_t)Dk;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.status = attn_status_ptr();
  B200_REQUIRE(p.status != nullptr, "attention: the status word of this device is not reachable");
  static bool attr_set[MAX_DEVICES];
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "attention: device ordinal %d is out of range", dev);
  if (!attr_set[dev]) {
    B200_CUDA(cudaFuncSetAttribute(fa::attn_bwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)fa::bwd_smem_bytes()));
    attr_set[dev] = true;
  }
  B200_CUDA(cudaMemsetAsync(p.dQacc, 0, (size_t)total_q * Dq * 4, s));
  const int64_t warps = (int64_t)total_q * num_q_heads;
  fa::attn_delta_all_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(total_q, num_q_heads, head_dim,
                                                                         (const __nv_bfloat16 *)dO, (const __nv_bfloat16 *)O, delta);
  B200_CHECK_LAUNCH("attention_bwd (delta)");
  for (int sq = 0; sq < num_seqs; sq++) {
    if (k_len[sq] == 0 || q_len[sq] != 0) continue;
    // keys that no query of the batch reads
    B200_CUDA(cudaMemsetAsync((__nv_bfloat16 *)dK + (int64_t)k_off[sq] * Dk, 0, (size_t)k_len[sq] * Dk * 2, s));
    B200_CUDA(cudaMemsetAsync((__nv_bfloat16 *)dV + (int64_t)k_off[sq] * Dk, 0, (size_t)k_len[sq] * Dk * 2, s));
  }
  for (int next = 0; next < num_seqs;) {
    const int units = fill_table(p.seqs, &next, num_seqs, q_off, q_len, k_off, k_len, [&](int sq) {
      return (q_len[sq] == 0 || k_len[sq] == 0) ? 0 : (k_len[sq] + fa::BN - 1) / fa::BN;
    });
    if (units == 0) continue;
    fa::attn_bwd_sm100_kernel<<<(unsigned)(units * num_kv_heads), fa::BWD_THREADS, fa::bwd_smem_bytes(), s>>>(p);
    B200_CHECK_LAUNCH("attention_bwd (fused)");
  }
  const int64_t n8 = (int64_t)total_q * Dq / 8;
  fa::attn_round_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>(n8, p.dQacc, (__nv_bfloat16 *)dQ);
  B200_CHECK_LAUNCH("attention_bwd (dQ rounding)");
  return 0;
}

}  // namespace b200

extern "C" int b200_attention_status(int *status_out) {
  int v = 0;
  B200_CUDA(cudaDeviceSynchronize());
  B200_CUDA(cudaMemcpyFromSymbol(&v, fa::g_attn_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    B200_CUDA(cudaMemcpyToSymbol(fa::g_attn_status, &zero, sizeof(int)));
  }
  if (status_out) *status_out = v;
  return 0;
}
