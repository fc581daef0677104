// bf16 GEMM for sm_100a on tcgen05 tensor cores: operands staged in shared memory by TMA (128-byte swizzle,
// 64x64 boxes), fp32 accumulators in tensor memory, one persistent CTA per SM of twelve warps with these roles:
//   warp 0            one thread issues the TMA loads of operand A
//   warp 1            one thread issues the MMAs (in a pair: the even CTA; the odd CTA's thread hands its slabs over)
//   warps 2..9        epilogue: tcgen05.ld, convert, fused SwiGLU forward / backward or plain store / accumulate
//   warp 10           grouped weight gradients only: clears the reduction tail of an expert's last slab
//   warp 11           one thread issues the TMA loads of operand B
// The producer and MMA loops run on a single thread each, with no warp-wide operation between two stages.
//
// One kernel body serves
//   * the dense matmul op (any combination of K-major / MN-major operands), optionally with the reduction cut into
//     ranges whose fp32 partial results a second kernel adds (few output tiles, long reduction: the router GEMMs),
//   * the expert-grouped forward / dgrad GEMMs (groups along the rows, weights picked by the third TMA coordinate),
//     with fused SwiGLU forward or backward epilogues and, for expert parallelism, output rows stored wherever a
//     per-row tag says (another GPU's buffer included),
//   * the expert-grouped wgrad GEMMs (groups along the reduction).
//
// Tile per CTA: 128 rows x up to 256 columns; two 256-column accumulator buffers in tensor memory so the epilogue
// of one tile overlaps the next tile's MMAs. Two variants of the same body:
//   single (cta_group::1): 4 stages of one 64-deep slab, 48 KiB each (A 128x64 + B 256x64);
//   pair   (cta_group::2): two CTAs of a cluster share one 256 x 256 MMA; each loads its 128 rows of A and HALF
//           the columns of B; a stage holds two 64-deep slabs (64 KiB, 3 stages), so one barrier round trip covers
//           eight MMAs. No TMA multicast is used: every CTA fetches its own boxes, the odd CTA reports its slabs
//           with a remote arrive on the even CTA's full barrier, and tcgen05.commit (multicast to both CTAs) says
//           when a stage or an accumulator is done.
// Every wait on a barrier is bounded; a wait that runs out raises a status word and the CTA leaves in order.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

constexpr int BM = 128;                 // rows of A / of the accumulator per CTA
constexpr int BK = 64;
constexpr int BLK_BYTES = 64 * 64 * 2;  // one TMA box: 64 rows of 128 bytes
constexpr int A_BLKS = 2;
constexpr int ACC_COLS = 256;
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 8;
#ifndef B200_TWO_PRODUCERS
#define B200_TWO_PRODUCERS 1
#endif
constexpr int TAIL_WARP = 2 + EPI_WARPS;                // clears the reduction tail of grouped weight-gradient slabs
constexpr int PRODUCER_B_WARP = 3 + EPI_WARPS;          // second TMA thread: the B operand (warp 0 keeps A)
constexpr int NUM_PRODUCERS = B200_TWO_PRODUCERS ? 2 : 1;
constexpr int GEMM_THREADS = (3 + EPI_WARPS + (B200_TWO_PRODUCERS ? 1 : 0)) * 32;
constexpr int MAX_GROUPS = 1024;
constexpr int MAX_STAGES = 6;

#ifndef B200_PAIR_STAGES
#define B200_PAIR_STAGES 6
#endif
#ifndef B200_SINGLE_STAGES
#define B200_SINGLE_STAGES 4
#endif
#ifndef B200_PAIR_KSLABS
#define B200_PAIR_KSLABS 2
#endif

template <bool PAIR, int SUP>
struct Cfg {
  static_assert(SUP == 1 || (SUP == 2 && PAIR), "two column tiles per row tile exist for CTA pairs only");
  static constexpr int B_BLKS_SUB = PAIR ? 2 : 4;                   // 64-column boxes of B per column tile and CTA
  static constexpr int B_BLKS = B_BLKS_SUB * SUP;
  static constexpr int SLAB_BYTES = (A_BLKS + B_BLKS) * BLK_BYTES;  // one 64-deep slice of both operands
  // slices per pipeline stage (one barrier round trip): a stage always feeds eight MMAs in pair mode
  static constexpr int KSLABS = (PAIR && SUP == 1) ? B200_PAIR_KSLABS : 1;
  static constexpr int STAGE_BYTES = KSLABS * SLAB_BYTES;
  static constexpr int STAGES = PAIR ? (SUP == 2 ? 4 : B200_PAIR_STAGES / KSLABS) : B200_SINGLE_STAGES;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;
};

enum GroupMode { DENSE = 0, GROUPED_M = 1, GROUPED_K = 2 };
enum Epilogue { EPI_STORE = 0, EPI_SWIGLU_FWD = 1, EPI_SWIGLU_BWD = 2 };
constexpr int SCATTER_MAX_RANKS = 16;
constexpr int TAG_RANK_SHIFT = 40;
constexpr unsigned long long TAG_ROW_MASK = (1ull << TAG_RANK_SHIFT) - 1ull;

enum StatusCode {
  ST_OK = 0,
  ST_PRODUCER_TIMEOUT = 1,
  ST_MMA_TIMEOUT = 2,
  ST_EPILOGUE_TIMEOUT = 3,
  ST_PEER_TIMEOUT = 4,
  ST_TAIL_TIMEOUT = 6,
  ST_BAD_ROW_TAG = 5  // a scatter tag named a rank or row outside the destination buffers; the row was not stored
};

__device__ int g_gemm_status = 0;

struct GemmParams {
  CUtensorMap tmA, tmA2, tmB, tmB2;
  int group_mode, num_groups;
  int M, N, K;
  int a_mn_major, b_mn_major;
  int dual_b, k_segments;
  const int *counts, *cumsum_incl;
  float alpha, beta;
  int out_fp32, c_fp32;
  void *D;
  const void *C;
  int64_t ldd, d_group_stride;
  // fused SwiGLU forward outputs ([rows, N] bf16)
  void *x1_out, *x3_out, *h_out;
  // fused SwiGLU backward
  const void *x1_in, *x3_in;
  const float *row_w;
  void *dx1, *dx3, *hs;
  float *dP;
  int *status;
  int wide;  // every bf16 row the epilogue touches is 32-byte aligned: use 256-bit global accesses
  // Row scatter (EPI_STORE, bf16, no C): output row r goes to row (tag & ROW_MASK) of the buffer of rank
  // (tag >> RANK_SHIFT), tag = row_tags[r]; the buffers may be peer memory mapped over NVLink (plain stores).
  const unsigned long long *row_tags;
  unsigned long long scatter_base[SCATTER_MAX_RANKS];
  int scatter_world;
  int64_t scatter_rows;
  // scattered rows are first transposed through shared memory so that eight lanes store 128 contiguous bytes of one
  // row (32-byte pieces of 32 different rows per instruction use a peer link poorly); set when the block fits
  int stage_out;
  // DENSE only: the reduction is cut into k_splits ranges of k_split_len (a multiple of 64); range i is one more
  // tile whose fp32 result goes to D + i * d_group_stride, summed afterwards by splitk_reduce_kernel
  int k_splits, k_split_len;
  int k_hint;  // host only, GROUPED_K: average reduction length per group (rows / groups), for choosing the unit shape
};

struct Tile {
  int group;     // expert (0 for dense)
  int a_row0;    // first row of the tile in A (GROUPED_K: first column of the [R, M] array)
  int out_row0;  // first output row of the tile
  int m_valid;   // valid rows in the tile (up to TILE_M)
  int nt0, nsub;        // first column tile and how many column tiles share these rows (1 or 2)
  int n0, n_valid, nw;  // of the column tile picked by Sched::set_sub: first column, valid columns, columns rounded
                        // up to the load granule
  int k_row0, k_len;    // GROUPED_K: reduction range inside the [R, *] arrays
};

// Work units are row tiles times groups of `sup` adjacent column tiles: with sup == 2 one fetch of the A rows feeds
// two accumulators (a 256 x 512 output block per CTA pair), which cuts the bytes staged per flop by a quarter.
struct Sched {
  int mode, tiles_n, stiles_n, sup, tiles_m, n_tile_w, n_round, tile_m, total_tiles, M, N, K, k_splits, k_split_len;
  const int *s_cnt, *s_base, *s_tpre;
  int cursor;

  // s_cnt[g] rows of group g, s_base[g] its first row, s_tpre[g] row tiles of the groups before it (GROUPED_M)
  __host__ __device__ __forceinline__ void init(int group_mode, int M_, int N_, int K_, int dual_b, bool pair,
                                                int tile_rows, int sup_, int splits, int split_len, const int *cnt,
                                                const int *base, const int *tpre, int groups) {
    mode = group_mode;
    M = M_;
    N = N_;
    K = K_;
    tile_m = tile_rows;
    sup = sup_;
    n_tile_w = dual_b ? 128 : 256;
    n_round = (pair && !dual_b) ? 128 : 64;
    tiles_n = (N + n_tile_w - 1) / n_tile_w;
    stiles_n = (tiles_n + sup - 1) / sup;
    tiles_m = (M + tile_m - 1) / tile_m;
    s_cnt = cnt;
    s_base = base;
    s_tpre = tpre;
    cursor = 0;
    k_splits = splits;
    k_split_len = split_len;
    if (mode == DENSE) total_tiles = tiles_m * stiles_n * (splits > 1 ? splits : 1);
    else if (mode == GROUPED_M) total_tiles = tpre[groups] * stiles_n;
    else total_tiles = groups * tiles_m * stiles_n;
  }

  // column tile `sub` (0 .. t.nsub - 1) of the unit
  __host__ __device__ __forceinline__ void set_sub(Tile &t, int sub) const {
    t.n0 = (t.nt0 + sub) * n_tile_w;
    t.n_valid = min(n_tile_w, N - t.n0);
    t.nw = (t.n_valid + n_round - 1) & ~(n_round - 1);
  }

  __host__ __device__ __forceinline__ bool get(int tile_id, Tile &t) {
    if (tile_id >= total_tiles) return false;
    int snt;
    if (mode == DENSE) {
      const int per = tiles_m * stiles_n;
      const int split = tile_id / per;  // 0 unless the reduction is split
      const int rem = tile_id - split * per;
      const int mt = rem / stiles_n;
      snt = rem - mt * stiles_n;
      t.group = split;
      t.a_row0 = t.out_row0 = mt * tile_m;
      t.m_valid = min(tile_m, M - mt * tile_m);
      t.k_row0 = split * k_split_len;
      t.k_len = (k_splits > 1) ? min(k_split_len, K - t.k_row0) : K;
    } else if (mode == GROUPED_M) {
      const int mtg = tile_id / stiles_n;
      snt = tile_id - mtg * stiles_n;
      while (s_tpre[cursor + 1] <= mtg) cursor++;
      const int ml = mtg - s_tpre[cursor];
      t.group = cursor;
      t.a_row0 = t.out_row0 = s_base[cursor] + ml * tile_m;
      t.m_valid = min(tile_m, s_cnt[cursor] - ml * tile_m);
      t.k_row0 = 0;
      t.k_len = K;
    } else {
      const int per = tiles_m * stiles_n;
      const int e = tile_id / per;
      const int rem = tile_id - e * per;
      const int mt = rem / stiles_n;
      snt = rem - mt * stiles_n;
      t.group = e;
      t.a_row0 = t.out_row0 = mt * tile_m;
      t.m_valid = min(tile_m, M - mt * tile_m);
      t.k_row0 = s_base[e];
      t.k_len = s_cnt[e];
    }
    t.nt0 = snt * sup;
    t.nsub = min(sup, tiles_n - t.nt0);
    set_sub(t, 0);
    return true;
  }
};

// The quotients of the SwiGLU epilogues use the hardware reciprocal (2 ulp): an IEEE division is a subroutine of some
// forty instructions, and 64 of them per thread made the gate-up epilogue take 25 k cycles per 128 x 256 tile where
// 7 k suffice (measured); the eight epilogue warps share their schedulers with the MMA and TMA threads.
__device__ __forceinline__ float sigmoid_f(float a) { return __fdividef(1.0f, 1.0f + __expf(-a)); }
__device__ __forceinline__ float silu_f(float a) { return __fdividef(a, 1.0f + __expf(-a)); }

// shared-memory bookkeeping that follows the stage buffers
struct GemmSmemTail {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], tail_done[MAX_STAGES], tfull[2], tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];  // keeps what follows 16-byte aligned
  // followed in shared memory by the group tables (cnt[G], base[G], tpre[G + 1]; table_ints(G) ints) and, when
  // GemmParams::stage_out is set, by one 4 KiB staging block per epilogue warp
};

static_assert(sizeof(GemmSmemTail) % 16 == 0, "the staging blocks after the tables need 16-byte alignment");

__host__ __device__ constexpr int table_ints(int groups) { return ((3 * groups + 1) + 3) & ~3; }
constexpr int STAGE_OUT_BYTES_PER_WARP = 32 * 128;  // 32 rows x 64 bf16 columns

template <int EPI, bool PAIR, int SUP>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  using CF = Cfg<PAIR, SUP>;
  constexpr int STAGES = CF::STAGES;
  constexpr int STAGE_BYTES = CF::STAGE_BYTES;
  extern __shared__ unsigned char gemm_smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  GemmSmemTail *st = reinterpret_cast<GemmSmemTail *>(smem + STAGES * STAGE_BYTES);
  int *const tab_cnt = reinterpret_cast<int *>(st + 1);
  int *const tab_base = tab_cnt + p.num_groups;
  int *const tab_tpre = tab_base + p.num_groups;
  uint4 *const stage_out = reinterpret_cast<uint4 *>(tab_cnt + table_ints(p.num_groups));
  volatile int *abort_flag = &st->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const uint32_t smem_base = ptx::smem_u32(smem);
  auto full_bar = [&](int s) { return ptx::smem_u32(&st->full[s]); };
  auto empty_bar = [&](int s) { return ptx::smem_u32(&st->empty[s]); };
  auto tail_bar = [&](int s) { return ptx::smem_u32(&st->tail_done[s]); };
  auto tfull_bar = [&](int s) { return ptx::smem_u32(&st->tfull[s]); };
  auto tempty_bar = [&](int s) { return ptx::smem_u32(&st->tempty[s]); };

  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(full_bar(s), NUM_PRODUCERS + ((PAIR && leader) ? 1 : 0));  // own loads (+ the odd CTA's hand-over)
      ptx::mbar_init(empty_bar(s), p.group_mode == GROUPED_K ? 2 : 1);  // MMA commit (+ the tail warp)
      ptx::mbar_init(tail_bar(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      ptx::mbar_init(tfull_bar(s), 1);
      ptx::mbar_init(tempty_bar(s), PAIR ? 2 * EPI_WARPS : EPI_WARPS);
    }
    st->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&st->tmem_base), TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&st->tmem_base), TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    ptx::tma_prefetch_desc(&p.tmA);
    ptx::tma_prefetch_desc(&p.tmB);
    if (p.k_segments > 1) ptx::tma_prefetch_desc(&p.tmA2);
    if (p.k_segments > 1 || p.dual_b) ptx::tma_prefetch_desc(&p.tmB2);
  }

  // group tables
  const int G = p.num_groups;
  if (p.group_mode != DENSE) {
    for (int e = tid; e < G; e += GEMM_THREADS) {
      const int c = p.counts[e];
      tab_cnt[e] = c;
      tab_base[e] = p.cumsum_incl[e] - c;
    }
  }
  __syncthreads();
  if (p.group_mode == GROUPED_M && warp == 2) {
    int running = 0;
    for (int e0 = 0; e0 < G; e0 += 32) {
      const int e = e0 + lane;
      const int v = (e < G) ? (tab_cnt[e] + CF::TILE_M - 1) / CF::TILE_M : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (e < G) tab_tpre[e] = running + incl - v;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tab_tpre[G] = running;
  }
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;

  Sched sched;
  sched.init(p.group_mode, p.M, p.N, p.K, p.dual_b, PAIR, CF::TILE_M, SUP, p.k_splits, p.k_split_len, tab_cnt, tab_base,
             tab_tpre, G);
  const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int row_off = (int)cta_rank * BM;  // this CTA's rows inside a pair tile

  // barriers that the other CTA of a pair arrives on are polled with a cluster-scope acquire
  auto xwait = [&](uint32_t bar, uint32_t par, int code) -> bool {
    return ptx::mbar_wait<PAIR>(bar, par, abort_flag, p.status, code);
  };
  auto wait_local = [&](uint32_t bar, uint32_t par, int code) -> bool {
    return ptx::mbar_wait<false>(bar, par, abort_flag, p.status, code);
  };
  // 16 bf16 columns of a row at `ptr` (n_left valid columns remain, a multiple of 8): one 32-byte access when
  // the launch allows it, else one or two 16-byte accesses
  auto ld16 = [&](const __nv_bfloat16 *ptr, int n_left, uint4 &lo, uint4 &hi) {
    if (p.wide && n_left >= 16) {
      ld_global_256(ptr, lo, hi);
    } else {
      lo = *reinterpret_cast<const uint4 *>(ptr);
      if (n_left > 8) hi = *reinterpret_cast<const uint4 *>(ptr + 8);
    }
  };
  auto st16 = [&](__nv_bfloat16 *ptr, int n_left, const uint4 &lo, const uint4 &hi) {
    if (p.wide && n_left >= 16) {
      st_global_256(ptr, lo, hi);
    } else {
      *reinterpret_cast<uint4 *>(ptr) = lo;
      if (n_left > 8) *reinterpret_cast<uint4 *>(ptr + 8) = hi;
    }
  };
  // 64-column boxes of B that ONE CTA fetches per slab for a column tile of (rounded) width nw
  auto b_boxes = [&](int nw) { return p.dual_b ? ((PAIR ? 1 : 2) * (nw >> 6)) : (PAIR ? (nw >> 7) : (nw >> 6)); };
  Tile t;
  if (warp == 0 || (NUM_PRODUCERS == 2 && warp == PRODUCER_B_WARP)) {
    // ================= TMA producers (every CTA loads its own boxes) =================
    // Two threads issue the loads, warp 0 those of A and PRODUCER_B_WARP those of B: one thread issuing all the
    // boxes of a stage spends 85 % of its time inside cp.async.bulk.tensor.
    const bool do_a = (NUM_PRODUCERS == 1) || warp == 0;
    const bool do_b = (NUM_PRODUCERS == 1) || warp != 0;
    // issue the loads of one slab into (sA, sB), counted on `bar`; sB holds the B boxes of column tile 0, then
    // (at the fixed offset B_BLKS_SUB boxes) those of column tile 1
    auto slab = [&](Tile &tt, int ks, uint32_t sA, uint32_t sB, uint32_t bar) {
      const int ksteps_seg = (tt.k_len + BK - 1) / BK;
      const int seg = ks / ksteps_seg;
      const int kk = (ks - seg * ksteps_seg) * BK;
      const CUtensorMap *mA = seg ? &p.tmA2 : &p.tmA;
      const CUtensorMap *mB = seg ? &p.tmB2 : &p.tmB;
      const int a_row = tt.a_row0 + row_off;
      const int g3 = (p.group_mode == GROUPED_M) ? tt.group : 0;
      auto ld2 = [&](uint32_t dst, const CUtensorMap *m, int c0, int c1) { ptx::tma_load_2d(dst, m, bar, c0, c1); };
      auto ld3 = [&](uint32_t dst, const CUtensorMap *m, int c0, int c1, int c2) {
        ptx::tma_load_3d(dst, m, bar, c0, c1, c2);
      };
      if (do_a) {
        if (!p.a_mn_major) {
          ld2(sA, mA, tt.k_row0 + kk, a_row);
          ld2(sA + BLK_BYTES, mA, tt.k_row0 + kk, a_row + 64);
        } else {
          ld2(sA, mA, a_row, tt.k_row0 + kk);
          ld2(sA + BLK_BYTES, mA, a_row + 64, tt.k_row0 + kk);
        }
      }
      if (!do_b) return;
      for (int sub = 0; sub < tt.nsub; sub++) {
        sched.set_sub(tt, sub);
        const uint32_t sBs = sB + sub * CF::B_BLKS_SUB * BLK_BYTES;
        // boxes of one map, and where this CTA's columns start
        const int nb = p.dual_b ? (tt.nw >> 6) : (PAIR ? (tt.nw >> 7) : (tt.nw >> 6));
        const int n_start = tt.n0 + ((PAIR && !p.dual_b) ? (int)cta_rank * (tt.nw >> 1) : 0);
        if (p.dual_b) {
          if (PAIR) {  // even CTA holds the W1 columns, odd CTA the W3 columns
            const CUtensorMap *mine = cta_rank ? &p.tmB2 : &p.tmB;
            for (int i = 0; i < nb; i++) ld3(sBs + i * BLK_BYTES, mine, kk, tt.n0 + 64 * i, g3);
          } else {
            for (int i = 0; i < nb; i++) ld3(sBs + i * BLK_BYTES, &p.tmB, kk, tt.n0 + 64 * i, g3);
            for (int i = 0; i < nb; i++) ld3(sBs + (nb + i) * BLK_BYTES, &p.tmB2, kk, tt.n0 + 64 * i, g3);
          }
        } else if (!p.b_mn_major) {
          for (int i = 0; i < nb; i++) ld3(sBs + i * BLK_BYTES, mB, tt.k_row0 + kk, n_start + 64 * i, g3);
        } else {
          for (int i = 0; i < nb; i++) ld3(sBs + i * BLK_BYTES, mB, n_start + 64 * i, tt.k_row0 + kk, g3);
        }
      }
    };
    // one thread runs the whole loop: no warp-wide operation sits between two stages
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = first_tile; alive && sched.get(tile, t); tile += tile_step) {
        const int ksteps = ((t.k_len + BK - 1) / BK) * p.k_segments;
        int b_loaded = 0;
        for (int sub = 0; sub < t.nsub; sub++) {
          sched.set_sub(t, sub);
          b_loaded += b_boxes(t.nw);
        }
        const int my_blks = (do_a ? A_BLKS : 0) + (do_b ? b_loaded : 0);
        for (int ks = 0; ks < ksteps; ks += CF::KSLABS) {
          if (!xwait(empty_bar(stage), phase ^ 1u, ST_PRODUCER_TIMEOUT)) {
            alive = false;
            break;
          }
          const int nsl = min(CF::KSLABS, ksteps - ks);
          ptx::mbar_arrive_expect_tx(full_bar(stage), (uint32_t)(nsl * my_blks * BLK_BYTES));
          for (int j = 0; j < nsl; j++) {
            const uint32_t sA = smem_base + stage * STAGE_BYTES + j * CF::SLAB_BYTES;
            slab(t, ks + j, sA, sA + A_BLKS * BLK_BYTES, full_bar(stage));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer (even CTA) / slab forwarder (odd CTA of a pair) =================
    // again a single thread: wait, fence, issue, commit
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_par = 0;  // bit a: parity of the next completion of accumulator a (as seen by the epilogue)
      int seq = 0;
      uint32_t tail_par = 0;  // parity of tail_done[stage], one bit per stage
      bool alive = true;
      for (int tile = first_tile; alive && sched.get(tile, t); tile += tile_step) {
        const int ksteps_seg = (t.k_len + BK - 1) / BK;
        const int ksteps = ksteps_seg * p.k_segments;
        if (ksteps == 0) continue;
        // per column tile: its accumulator and its instruction descriptor
        uint32_t idesc[SUP], d_tmem[SUP];
        int accs[SUP];
#pragma unroll
        for (int sub = 0; sub < SUP; sub++) {
          if (sub < t.nsub) sched.set_sub(t, sub);
          accs[sub] = (SUP == 2) ? sub : (seq & 1);
          idesc[sub] = ptx::make_idesc_bf16(CF::TILE_M, p.dual_b ? 2 * t.nw : t.nw, p.a_mn_major, p.b_mn_major);
          d_tmem[sub] = tmem_base + (uint32_t)(accs[sub] * ACC_COLS);
        }
        if (SUP == 1 && leader) {
          // one column tile per unit: its accumulator is waited for once, before the first stage. (Waiting inside the
          // issue loop, as the two-tile units must, costs 7 % of a whole layer step: the tensor pipe queues only about
          // two MMAs behind the one it runs, so whatever this thread does between two MMAs beyond ~170 cycles idles it.)
          if (!xwait(tempty_bar(accs[0]), ((acc_par >> accs[0]) & 1u) ^ 1u, ST_MMA_TIMEOUT)) break;
          ptx::tc_fence_after();
        }
        for (int ks = 0; ks < ksteps; ks += CF::KSLABS) {
          const int nsl = min(CF::KSLABS, ksteps - ks);
          const bool last = ks + nsl == ksteps;
          // 16-row groups of the stage's last slab that hold rows of this expert (all four except at the ragged
          // end of a grouped weight gradient)
          int last_k16 = BK / 16;
          if (p.group_mode == GROUPED_K && last && (t.k_len & (BK - 1)) != 0) last_k16 = ((t.k_len & (BK - 1)) + 15) >> 4;
          // every CTA watches its own slabs land; a stage whose last slab straddles the end of the expert's rows is
          // handed over by the tail warp instead, once it has cleared the rows past the end
          bool ok;
          if (p.group_mode == GROUPED_K && last && (t.k_len & 15) != 0) {
            ok = wait_local(tail_bar(stage), (tail_par >> stage) & 1u, ST_MMA_TIMEOUT);
            tail_par ^= 1u << stage;
          } else if (!(PAIR && leader)) {
            ok = wait_local(full_bar(stage), phase, ST_MMA_TIMEOUT);
          } else {
            ok = true;
          }
          // in a pair the even CTA's barrier also counts the odd CTA's hand-over: one cluster-scope wait covers both
          if (ok && PAIR && leader) ok = xwait(full_bar(stage), phase, ST_PEER_TIMEOUT);
          if (!ok) {
            alive = false;
            break;
          }
          if (PAIR && !leader) {
            // ... the odd CTA then tells the even one that its half is in place
            ptx::mbar_arrive_remote(full_bar(stage), 0);
          } else {
            ptx::tc_fence_after();
            for (int j = 0; j < nsl && alive; j++) {
              const uint32_t sA = smem_base + stage * STAGE_BYTES + j * CF::SLAB_BYTES;
              const int n16 = (j == nsl - 1) ? last_k16 : BK / 16;
#pragma unroll
              for (int sub = 0; sub < SUP; sub++) {
                if (sub >= t.nsub) break;
                if (SUP == 2 && ks + j == 0) {
                  // the accumulator must have been drained by the epilogue of the unit before; column tile 1 is
                  // waited for only now, after the first MMAs of column tile 0 are on their way
                  if (!xwait(tempty_bar(accs[sub]), ((acc_par >> accs[sub]) & 1u) ^ 1u, ST_MMA_TIMEOUT)) {
                    alive = false;
                    break;
                  }
                  ptx::tc_fence_after();
                }
                const uint32_t sB = sA + (A_BLKS + sub * CF::B_BLKS_SUB) * BLK_BYTES;
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; k16++) {
                  if (k16 >= n16) break;
                  const uint64_t adesc = p.a_mn_major ? ptx::make_smem_desc(sA + k16 * 2048, BLK_BYTES, 1024)
                                                      : ptx::make_smem_desc(sA + k16 * 32, 0, 1024);
                  const uint64_t bdesc = p.b_mn_major ? ptx::make_smem_desc(sB + k16 * 2048, BLK_BYTES, 1024)
                                                      : ptx::make_smem_desc(sB + k16 * 32, 0, 1024);
                  const uint32_t accum = (ks + j > 0 || k16 > 0) ? 1u : 0u;
                  if (PAIR) ptx::umma_bf16_pair(d_tmem[sub], adesc, bdesc, idesc[sub], accum);
                  else ptx::umma_bf16(d_tmem[sub], adesc, bdesc, idesc[sub], accum);
                }
              }
            }
            if (!alive) break;
            if (PAIR) ptx::umma_commit_pair(empty_bar(stage));
            else ptx::umma_commit(empty_bar(stage));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
#pragma unroll
        for (int sub = 0; sub < SUP; sub++) {
          if (sub >= t.nsub) break;
          if (leader) {
            if (PAIR) ptx::umma_commit_pair(tfull_bar(accs[sub]));
            else ptx::umma_commit(tfull_bar(accs[sub]));
          }
          acc_par ^= 1u << accs[sub];
        }
        seq++;
      }
    }
    __syncwarp();
  } else if (warp == TAIL_WARP) {
    // ================= tail warp (grouped weight gradients) =================
    // The last 64-row slab of an expert's reduction range also holds rows of the next expert (or rows past the
    // end). This warp follows the producer's schedule, waits for such a slab to land, clears the rows past the end
    // in every 64x64 block of both operands (a row is 128 contiguous bytes in the swizzled layout) and passes the
    // stage on through tail_done, so the clearing is off the MMA warp's issue path.
    if (p.group_mode == GROUPED_K) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = first_tile; sched.get(tile, t); tile += tile_step) {
        const int ksteps = (t.k_len + BK - 1) / BK;
        int nbs[SUP];
#pragma unroll
        for (int sub = 0; sub < SUP; sub++) {
          nbs[sub] = 0;
          if (sub < t.nsub) {
            sched.set_sub(t, sub);
            nbs[sub] = PAIR ? (t.nw >> 7) : (t.nw >> 6);
          }
        }
        const int kv = t.k_len & (BK - 1);
        for (int ks = 0; ks < ksteps; ks += CF::KSLABS) {
          const int nsl = min(CF::KSLABS, ksteps - ks);
          // every use of a stage is observed, and the stage is not refilled before that (this warp is the second
          // arrival on the empty barrier), so the parity this warp waits for always names the right fill
          const bool ok = wait_local(full_bar(stage), phase, ST_TAIL_TIMEOUT);
          if (!__all_sync(0xffffffffu, ok)) goto teardown;
          if (ks + nsl == ksteps && (kv & 15) != 0) {
            // only the 16-row group that straddles the end is multiplied at all (the MMA warp skips the groups past
            // it), so rows kv .. roundup(kv, 16) - 1 of every block are all there is to clear
            unsigned char *stA = smem + stage * STAGE_BYTES + (nsl - 1) * CF::SLAB_BYTES;
            const int chunks_per_blk = (16 - (kv & 15)) * 8;
            auto clear_blocks = [&](unsigned char *first, int blocks) {
              for (int b = 0; b < blocks; b++)
                for (int c = lane; c < chunks_per_blk; c += 32)
                  *reinterpret_cast<uint4 *>(first + b * BLK_BYTES + kv * 128 + c * 16) = make_uint4(0, 0, 0, 0);
            };
            clear_blocks(stA, A_BLKS);
#pragma unroll
            for (int sub = 0; sub < SUP; sub++)
              clear_blocks(stA + (A_BLKS + sub * CF::B_BLKS_SUB) * BLK_BYTES, nbs[sub]);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tail_bar(stage));
          }
          if (lane == 0) ptx::mbar_arrive(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ================= epilogue (warps 2..9) =================
    // TMEM lanes a warp may read are fixed by warp_id % 4; two warps share a lane quarter and split the columns.
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    uint32_t acc_par = 0;  // bit a: parity of the next completion of accumulator a
    int seq = 0;
    for (int tile = first_tile; sched.get(tile, t); tile += tile_step) {
      const int row_in_cta = quarter * 32 + lane;
      const bool row_ok = row_in_cta + row_off < t.m_valid;
      const int64_t orow = (int64_t)t.out_row0 + row_off + row_in_cta;
      if (t.k_len == 0) {
        // An expert without rows: nothing to add. When the weight gradient is written rather than accumulated (no C),
        // its tiles are zeros - no MMA runs for them, so no accumulator is involved.
        if (EPI == EPI_STORE && p.group_mode == GROUPED_K && p.C == nullptr && !p.out_fp32 && row_ok) {
          for (int sub = 0; sub < t.nsub; sub++) {
            sched.set_sub(t, sub);
            __nv_bfloat16 *drow = static_cast<__nv_bfloat16 *>(p.D) + (int64_t)t.group * p.d_group_stride + orow * p.ldd + t.n0;
            const int cbeg = chalf * (t.nw >> 1), cend = min(cbeg + (t.nw >> 1), t.n_valid);
            for (int col = cbeg; col < cend; col += 8) *reinterpret_cast<uint4 *>(drow + col) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      for (int sub = 0; sub < t.nsub; sub++) {
        // the column tiles of a unit finish together; they are drained in order, each freeing its accumulator
        sched.set_sub(t, sub);
        const int acc = (SUP == 2) ? sub : (seq & 1);
        const uint32_t acc_phase = (acc_par >> acc) & 1u;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * ACC_COLS);
        // t.nw is the logical width (per part when the accumulator holds x1 | x3); each warp takes half of it
        const int cbeg = chalf * (t.nw >> 1), cend = cbeg + (t.nw >> 1);

        if (EPI == EPI_STORE) {
          const int64_t goff = (p.group_mode == GROUPED_K || p.k_splits > 1) ? (int64_t)t.group * p.d_group_stride : 0;
          const int64_t base = goff + orow * p.ldd + t.n0;
          const bool use_c = (p.C != nullptr) && (p.beta != 0.0f);
          // destination of this thread's row: D itself, or (row scatter) the row its tag names in some rank's buffer
          __nv_bfloat16 *drow = static_cast<__nv_bfloat16 *>(p.D) + base;
          bool store_ok = row_ok;
          if (p.row_tags != nullptr && row_ok) {
            const unsigned long long tag = p.row_tags[orow];
            const unsigned long long rk = tag >> TAG_RANK_SHIFT, rr = tag & TAG_ROW_MASK;
            if (rk < (unsigned long long)p.scatter_world && rr < (unsigned long long)p.scatter_rows) {
              drow = reinterpret_cast<__nv_bfloat16 *>(p.scatter_base[rk]) + (int64_t)rr * p.ldd + t.n0;
            } else {
              store_ok = false;
              atomicCAS(p.status, 0, (int)ST_BAD_ROW_TAG);
            }
          }
          // the bf16 C segment of this thread (up to 128 columns) is fetched before waiting on the MMAs
          uint4 cpre[16];
          if (use_c && !p.c_fp32 && row_ok) {
#pragma unroll
            for (int vv = 0; vv < 8; vv++) {
              const int col = cbeg + vv * 16;
              if (col < cend && col < t.n_valid)
                ld16(static_cast<const __nv_bfloat16 *>(p.C) + base + col, t.n_valid - col, cpre[2 * vv], cpre[2 * vv + 1]);
            }
          }
          bool ok = xwait(tfull_bar(acc), acc_phase, ST_EPILOGUE_TIMEOUT);
          if (!__all_sync(0xffffffffu, ok)) goto teardown;
          ptx::tc_fence_after();
#pragma unroll
          for (int ch = 0; ch < 2; ch++) {  // 64 accumulator columns per TMEM round trip
            const int c0 = cbeg + ch * 64;
            if (c0 < cend) {
              uint32_t r[64];
              ptx::tmem_ld32(taddr + c0, r);
              if (c0 + 32 < cend) ptx::tmem_ld32(taddr + c0 + 32, r + 32);
              ptx::tmem_ld_wait();
              if (p.stage_out) {
                // lane = row writes its 64 columns as eight 16-byte chunks (XOR-swizzled: conflict-free both ways), then
                // lanes 8i..8i+7 read back row 4*it + i and store its 128 bytes side by side
                uint4 *sb = stage_out + (warp - 2) * (STAGE_OUT_BYTES_PER_WARP / 16);
#pragma unroll
                for (int vv = 0; vv < 4; vv++) {
                  if (c0 + vv * 16 < cend) {
                    float f[16];
#pragma unroll
                    for (int q = 0; q < 16; q++) f[q] = p.alpha * __uint_as_float(r[vv * 16 + q]);
                    sb[lane * 8 + ((2 * vv) ^ (lane & 7))] = pack8(f);
                    sb[lane * 8 + ((2 * vv + 1) ^ (lane & 7))] = pack8(f + 8);
                  }
                }
                __syncwarp();
                const unsigned long long dptr = reinterpret_cast<unsigned long long>(drow);
                const int chunk = lane & 7;
                const int col = c0 + chunk * 8;
#pragma unroll
                for (int it = 0; it < 8; it++) {
                  const int rr = it * 4 + (lane >> 3);
                  const unsigned long long rp = __shfl_sync(0xffffffffu, dptr, rr);
                  const int rok = __shfl_sync(0xffffffffu, (int)store_ok, rr);
                  const uint4 v = sb[rr * 8 + (chunk ^ (rr & 7))];
                  if (rok && col < cend && col < t.n_valid) *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(rp) + col) = v;
                }
                __syncwarp();
              } else if (store_ok) {
#pragma unroll
                for (int vv = 0; vv < 4; vv++) {
                  const int col = c0 + vv * 16;
                  if (col < cend && col < t.n_valid) {
                    float f[16];
#pragma unroll
                    for (int q = 0; q < 16; q++) f[q] = p.alpha * __uint_as_float(r[vv * 16 + q]);
                    if (use_c) {
                      if (p.c_fp32) {
                        const float *cp = static_cast<const float *>(p.C) + base + col;
#pragma unroll
                        for (int q = 0; q < 16; q++)
                          if (col + q < t.n_valid) f[q] += p.beta * cp[q];
                      } else {
                        float cf[16];
                        unpack8(cpre[ch * 8 + 2 * vv], cf);
                        unpack8(cpre[ch * 8 + 2 * vv + 1], cf + 8);
#pragma unroll
                        for (int q = 0; q < 16; q++) f[q] += p.beta * cf[q];
                      }
                    }
                    if (p.out_fp32) {
                      float4 *dp = reinterpret_cast<float4 *>(static_cast<float *>(p.D) + base + col);
                      dp[0] = make_float4(f[0], f[1], f[2], f[3]);
                      dp[1] = make_float4(f[4], f[5], f[6], f[7]);
                      if (col + 8 < t.n_valid) {
                        dp[2] = make_float4(f[8], f[9], f[10], f[11]);
                        dp[3] = make_float4(f[12], f[13], f[14], f[15]);
                      }
                    } else {
                      st16(drow + col, t.n_valid - col, pack8(f), pack8(f + 8));
                    }
                  }
                }
              }
            }
          }
        } else if (EPI == EPI_SWIGLU_FWD) {
          // accumulator columns [0, nw) = x1 tile, [nw, 2 nw) = x3 tile
          bool ok = xwait(tfull_bar(acc), acc_phase, ST_EPILOGUE_TIMEOUT);
          if (!__all_sync(0xffffffffu, ok)) goto teardown;
          ptx::tc_fence_after();
          const int64_t base = orow * (int64_t)p.N + t.n0;
          // 32 columns of x1 and of x3 per TMEM round trip: 64 live accumulator registers leave the compiler room to
          // interleave the sixteen independent SwiGLU chains of a store group
          for (int c0 = cbeg; c0 < cend; c0 += 32) {
            uint32_t r1[32], r3[32];
            ptx::tmem_ld32(taddr + c0, r1);
            ptx::tmem_ld32(taddr + t.nw + c0, r3);
            ptx::tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int vv = 0; vv < 2; vv++) {
                const int col = c0 + vv * 16;
                if (col < cend && col < t.n_valid) {
                  float a[16], b[16], h[16];
#pragma unroll
                  for (int q = 0; q < 16; q++) {
                    a[q] = bf16_round(__uint_as_float(r1[vv * 16 + q]));
                    b[q] = bf16_round(__uint_as_float(r3[vv * 16 + q]));
                    h[q] = silu_f(a[q]) * b[q];
                  }
                  const int left = t.n_valid - col;
                  st16(static_cast<__nv_bfloat16 *>(p.x1_out) + base + col, left, pack8(a), pack8(a + 8));
                  st16(static_cast<__nv_bfloat16 *>(p.x3_out) + base + col, left, pack8(b), pack8(b + 8));
                  st16(static_cast<__nv_bfloat16 *>(p.h_out) + base + col, left, pack8(h), pack8(h + 8));
                }
              }
            }
          }
        } else {
          // EPI_SWIGLU_BWD: accumulator = dh = (w * dOut) W2 for this row
          const int64_t base = orow * (int64_t)p.N + t.n0;
          // x1 / x3 of the first 64 columns are requested before waiting on the MMAs, those of the second 64
          // together with the second TMEM read
          uint4 xa[8], xb[8];
          auto load_x = [&](int c0) {
            if (row_ok) {
#pragma unroll
              for (int vv = 0; vv < 4; vv++) {
                const int col = c0 + vv * 16;
                if (col < cend && col < t.n_valid) {
                  ld16(static_cast<const __nv_bfloat16 *>(p.x1_in) + base + col, t.n_valid - col, xa[2 * vv], xa[2 * vv + 1]);
                  ld16(static_cast<const __nv_bfloat16 *>(p.x3_in) + base + col, t.n_valid - col, xb[2 * vv], xb[2 * vv + 1]);
                }
              }
            }
          };
          load_x(cbeg);
          bool ok = xwait(tfull_bar(acc), acc_phase, ST_EPILOGUE_TIMEOUT);
          if (!__all_sync(0xffffffffu, ok)) goto teardown;
          ptx::tc_fence_after();
          float dp_part = 0.f;
#pragma unroll
          for (int ch = 0; ch < 2; ch++) {
            const int c0 = cbeg + ch * 64;
            if (c0 < cend) {
              uint32_t r[64];
              ptx::tmem_ld32(taddr + c0, r);
              if (c0 + 32 < cend) ptx::tmem_ld32(taddr + c0 + 32, r + 32);
              if (ch == 1) load_x(c0);
              ptx::tmem_ld_wait();
              if (row_ok) {
#pragma unroll
                for (int vv = 0; vv < 4; vv++) {
                  const int col = c0 + vv * 16;
                  if (col < cend && col < t.n_valid) {
                    float a[16], b[16], o1[16], o3[16], hv[16];
                    unpack8(xa[2 * vv], a);
                    unpack8(xa[2 * vv + 1], a + 8);
                    unpack8(xb[2 * vv], b);
                    unpack8(xb[2 * vv + 1], b + 8);
                    const int left = t.n_valid - col;
#pragma unroll
                    for (int q = 0; q < 16; q++) {
                      const float acc_dh = (q < left) ? __uint_as_float(r[vv * 16 + q]) : 0.f;
                      const float s = sigmoid_f(a[q]);
                      const float silu = a[q] * s;
                      hv[q] = silu * b[q];
                      if (q < left) dp_part += bf16_round(hv[q]) * acc_dh;
                      const float dh = bf16_round(acc_dh);  // the reference stores dh as bf16 before swiglu_bwd_x
                      o3[q] = dh * silu;
                      o1[q] = dh * b[q] * (s + a[q] * (s * (1.0f - s)));
                    }
                    st16(static_cast<__nv_bfloat16 *>(p.dx1) + base + col, left, pack8(o1), pack8(o1 + 8));
                    st16(static_cast<__nv_bfloat16 *>(p.dx3) + base + col, left, pack8(o3), pack8(o3 + 8));
                    if (p.hs) st16(static_cast<__nv_bfloat16 *>(p.hs) + base + col, left, pack8(hv), pack8(hv + 8));
                  }
                }
              }
            }
          }
          if (row_ok) {
            // <h, (w dOut) W2> = w <Y, dOut>: divide the gate weight back out (w == 0 contributes nothing downstream)
            const float w = p.row_w[orow];
            if (w != 0.f) atomicAdd(p.dP + orow, dp_part / w);
          }
        }

        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR && !leader) ptx::mbar_arrive_remote(tempty_bar(acc), 0);
          else ptx::mbar_arrive(tempty_bar(acc));
          if (warp == 2 && leader) {
          }
        }
        acc_par ^= 1u << acc;
      }
      seq++;
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
  if (PAIR) ptx::cluster_sync_all();  // neither CTA leaves while the other may still reach into it
  if (warp == 1) {
    ptx::tc_fence_after();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

constexpr size_t GEMM_SMEM_LIMIT = 232448;  // 227 KiB: the most one CTA can be given on sm_100

template <bool PAIR, int SUP>
static size_t gemm_smem_bytes(int groups, bool stage_out) {
  using CF = Cfg<PAIR, SUP>;
  return 1024 + (size_t)CF::STAGES * CF::STAGE_BYTES + sizeof(GemmSmemTail) + 4 * (size_t)table_ints(groups) +
         (stage_out ? (size_t)EPI_WARPS * STAGE_OUT_BYTES_PER_WARP : 0);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// bf16 tensor [d2][d1][d0] (d0 contiguous), 64 x 64 x 1 boxes, 128-byte swizzle, zero fill.
static int make_tmap(CUtensorMap *m, const void *base, int rank, uint64_t d0, uint64_t d1, uint64_t d2,
                     uint64_t stride1_bytes, uint64_t stride2_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  B200_REQUIRE(fn != nullptr, "gemm: cuTensorMapEncodeTiled is not available from this driver");
  B200_REQUIRE(b200_aligned16(base), "gemm: operand base must be 16-byte aligned");
  B200_REQUIRE(stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0, "gemm: operand row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// Per-device host state. One process may drive several GPUs (cudaSetDevice between calls), so everything that is a
// property of a device - its SM count, the address of its copy of the status word, whether a kernel variant has been
// given its shared-memory attribute there - is kept per device ordinal.
constexpr int MAX_DEVICES = 64;

static int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

static int sm_count_cached() {
  static int sms[MAX_DEVICES];
  const int dev = current_device();
  if (dev < 0) return 148;
  if (!sms[dev]) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    sms[dev] = v > 0 ? v : 148;
  }
  return sms[dev];
}

static int *status_ptr() {
  static int *ptr[MAX_DEVICES];
  const int dev = current_device();
  if (dev < 0) return nullptr;
  if (!ptr[dev] && cudaGetSymbolAddress((void **)&ptr[dev], g_gemm_status) != cudaSuccess) ptr[dev] = nullptr;
  return ptr[dev];
}

// 0 = one CTA per tile (cta_group::1), 1 = CTA pairs (cta_group::2) wherever a launch allows it.
// Initialised from the environment variable B200_GEMM_PAIR on first use; b200_gemm_set_pair_mode overrides it.
static int g_pair_mode = -1;

static int pair_mode() {
  if (g_pair_mode < 0) {
    const char *e = getenv("B200_GEMM_PAIR");
    g_pair_mode = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pair_mode;
}

// Which kinds of launch let one fetch of the A rows feed two column tiles (256 x 512 per CTA pair): bit 0 the
// row-grouped expert GEMMs (forward, dgrad), bit 1 the reduction-grouped weight gradients, bit 2 the dense matmul,
// bit 3 = also when the launch then has too few units to fill the GPU (for tests on small shapes).
// Environment variable B200_GEMM_WIDE on first use; b200_gemm_set_wide_mode overrides it.
constexpr int WIDE_GROUPED_M = 1, WIDE_GROUPED_K = 2, WIDE_DENSE = 4, WIDE_ALWAYS = 8;
#ifndef B200_GEMM_WIDE_DEFAULT
#define B200_GEMM_WIDE_DEFAULT 0  // measured: no launch kind of the layer gains from it (forward 864 -> 794, weight
                                  // gradients 904 -> 884 TFLOP/s at 4096 rows per expert, sustained, real data)
#endif
static int g_wide_mode = -1;

static int wide_mode() {
  if (g_wide_mode < 0) {
    const char *e = getenv("B200_GEMM_WIDE");
    g_wide_mode = (e && e[0] >= '0' && e[0] <= '9') ? (atoi(e) & 15) : B200_GEMM_WIDE_DEFAULT;
  }
  return g_wide_mode;
}

template <int EPI, bool PAIR, int SUP>
static int launch_gemm_variant(GemmParams &p, int64_t max_tiles, cudaStream_t s) {
  auto kern = gemm_sm100_kernel<EPI, PAIR, SUP>;
  // staging of scattered rows is used whenever it fits beside the pipeline stages and the group tables
  p.stage_out = (EPI == EPI_STORE && p.row_tags != nullptr && gemm_smem_bytes<PAIR, SUP>(p.num_groups, true) <= GEMM_SMEM_LIMIT) ? 1 : 0;
  const size_t smem = gemm_smem_bytes<PAIR, SUP>(p.num_groups, p.stage_out != 0);
  B200_REQUIRE(smem <= GEMM_SMEM_LIMIT, "gemm: %d groups need %zu bytes of shared memory (limit %zu)", p.num_groups, smem,
               GEMM_SMEM_LIMIT);
  const int dev = current_device();
  B200_REQUIRE(dev >= 0, "gemm: no current device (or its ordinal is %d or more)", MAX_DEVICES);
  static bool configured[MAX_DEVICES];
  static int max_clusters[MAX_DEVICES];
  if (!configured[dev]) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_LIMIT));
    if (PAIR) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * (unsigned)(sm_count_cached() / 2));
      q.blockDim = dim3(GEMM_THREADS);
      q.dynamicSmemBytes = GEMM_SMEM_LIMIT;
      cudaLaunchAttribute a[1];
      a[0].id = cudaLaunchAttributeClusterDimension;
      a[0].val.clusterDim.x = 2;
      a[0].val.clusterDim.y = 1;
      a[0].val.clusterDim.z = 1;
      q.attrs = a;
      q.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&max_clusters[dev], kern, &q) != cudaSuccess || max_clusters[dev] <= 0) {
        cudaGetLastError();
        max_clusters[dev] = sm_count_cached() / 2;
      }
    }
    configured[dev] = true;
  }
  if (max_tiles < 1) return 0;
  if (!PAIR) {
    int64_t grid = sm_count_cached();
    if (max_tiles < grid) grid = max_tiles;
    kern<<<(unsigned)grid, GEMM_THREADS, smem, s>>>(p);
    B200_CHECK_LAUNCH("gemm_sm100");
    return 0;
  }
  int64_t pairs = max_clusters[dev];
  if (max_tiles < pairs) pairs = max_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return 0;
}

// max_tiles: an upper bound on the number of 128-row x one-column-tile units (pair and wide units are never more
// numerous). row_tiles_hint: about how many 256-row tiles the launch has (decides whether wide units still fill the GPU).
template <int EPI>
static int launch_gemm(GemmParams &p, int64_t max_tiles, cudaStream_t s, bool pair_ok = true, int64_t row_tiles_hint = 0) {
  p.status = status_ptr();
  B200_REQUIRE(p.status != nullptr, "gemm: status word unavailable");
  {
    // 256-bit epilogue accesses need every bf16 row start to be 32-byte aligned
    auto a32 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 31u) == 0; };
    bool wide;
    if (EPI == EPI_STORE)
    {
      wide = !p.out_fp32 && a32(p.D) && a32(p.C) && p.ldd % 16 == 0 && p.d_group_stride % 16 == 0;
      for (int i = 0; i < p.scatter_world; i++) wide = wide && (p.scatter_base[i] & 31ull) == 0;
    }
    else if (EPI == EPI_SWIGLU_FWD)
      wide = a32(p.x1_out) && a32(p.x3_out) && a32(p.h_out) && p.N % 16 == 0;
    else
      wide = a32(p.x1_in) && a32(p.x3_in) && a32(p.dx1) && a32(p.dx3) && a32(p.hs) && p.N % 16 == 0;
    p.wide = wide ? 1 : 0;
  }
  if (pair_ok && pair_mode()) {
    // two column tiles per unit: when the kind of launch is enabled, there are at least two column tiles, the units
    // still outnumber the CTA pairs a few times over, and the deeper stages fit beside the group tables
    const int kind = p.group_mode == GROUPED_M ? WIDE_GROUPED_M : (p.group_mode == GROUPED_K ? WIDE_GROUPED_K : WIDE_DENSE);
    const int col_tiles = (p.N + (p.dual_b ? 127 : 255)) / (p.dual_b ? 128 : 256);
    const int64_t units2 = row_tiles_hint * ((col_tiles + 1) / 2);
    // the two accumulators of a wide unit finish together, so their epilogues are not hidden behind the next unit's
    // MMAs: it pays only where the reduction is long (measured: weight gradients from about 2048 rows per expert)
    const bool long_reduction = p.group_mode == GROUPED_K ? p.k_hint >= 2048 : (int64_t)p.K * p.k_segments >= 1024;
    if ((wide_mode() & kind) && col_tiles >= 2 && (long_reduction || (wide_mode() & WIDE_ALWAYS)) &&
        ((wide_mode() & WIDE_ALWAYS) || units2 >= 2 * (int64_t)(sm_count_cached() / 2)) &&
        gemm_smem_bytes<true, 2>(p.num_groups, false) <= GEMM_SMEM_LIMIT)
      return launch_gemm_variant<EPI, true, 2>(p, max_tiles, s);
    return launch_gemm_variant<EPI, true, 1>(p, max_tiles, s);
  }
  return launch_gemm_variant<EPI, false, 1>(p, max_tiles, s);
}

static void zero_params(GemmParams &p) { memset(&p, 0, sizeof(p)); }

// D = alpha * sum_i partial[i] + beta * C over n elements (a multiple of 4); partial[i] = partials + i * n, fp32
__global__ void splitk_reduce_kernel(int64_t n, int splits, const float *__restrict__ partials, float alpha, float beta,
                                     const void *C, int c_fp32, void *D, int d_fp32) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = *reinterpret_cast<const float4 *>(partials + i);
  for (int sidx = 1; sidx < splits; sidx++) {
    const float4 v = *reinterpret_cast<const float4 *>(partials + (int64_t)sidx * n + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  float f[4] = {alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w};
  if (C != nullptr) {
    if (c_fp32) {
      const float4 c = *reinterpret_cast<const float4 *>(static_cast<const float *>(C) + i);
      f[0] += beta * c.x; f[1] += beta * c.y; f[2] += beta * c.z; f[3] += beta * c.w;
    } else {
      const uint2 c = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(C) + i);
      f[0] += beta * bf16lo(c.x); f[1] += beta * bf16hi(c.x); f[2] += beta * bf16lo(c.y); f[3] += beta * bf16hi(c.y);
    }
  }
  if (d_fp32) {
    *reinterpret_cast<float4 *>(static_cast<float *>(D) + i) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(D) + i) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
}

}  // namespace b200

using namespace b200;


// Host run of the kernels' tile scheduler (same Sched code as the device uses): lists the tiles a launch would
// process, in order. counts / cumsum_incl are HOST arrays here. Nothing touches a GPU.
extern "C" int b200_gemm_enumerate_tiles(int group_mode, int pair, int M, int N, int K, int dual_b, int num_groups,
                                         const int *counts, const int *cumsum_incl, int k_splits, int k_split_len,
                                         int max_tiles, int *out) {
  B200_REQUIRE(group_mode >= DENSE && group_mode <= GROUPED_K && num_groups >= 1 && num_groups <= MAX_GROUPS && out,
               "gemm_enumerate_tiles: bad arguments");
  B200_REQUIRE(group_mode == DENSE || (counts && cumsum_incl), "gemm_enumerate_tiles: group tables missing");
  const int tile_rows = pair ? 2 * BM : BM;
  std::vector<int> cnt(num_groups, 0), base(num_groups, 0), tpre(num_groups + 1, 0);
  if (group_mode != DENSE) {
    for (int e = 0; e < num_groups; e++) {
      cnt[e] = counts[e];
      base[e] = cumsum_incl[e] - counts[e];
      tpre[e + 1] = tpre[e] + (cnt[e] + tile_rows - 1) / tile_rows;
    }
  }
  Sched sc;
  sc.init(group_mode, M, N, K, dual_b, pair != 0, tile_rows, pair == 2 ? 2 : 1, k_splits, k_split_len, cnt.data(),
          base.data(), tpre.data(), num_groups);
  Tile t;
  int n = 0;
  for (int id = 0; sc.get(id, t); id++) {
    for (int sub = 0; sub < t.nsub; sub++) {
      sc.set_sub(t, sub);
      if (n < max_tiles) {
        const int rec[9] = {t.group, t.a_row0, t.out_row0, t.m_valid, t.n0, t.n_valid, t.nw, t.k_row0, t.k_len};
        memcpy(out + (size_t)n * 9, rec, sizeof(rec));
      }
      n++;
    }
  }
  return n;
}


extern "C" int b200_gemm_set_pair_mode(int on) {
  g_pair_mode = on ? 1 : 0;
  return 0;
}

extern "C" int b200_gemm_set_wide_mode(int mask) {
  g_wide_mode = mask & 15;
  return 0;
}

// Reads (and clears) the status word the GEMM kernels raise when a bounded wait runs out.
// Synchronises the device. 0 = no kernel has given up since the last call.
extern "C" int b200_gemm_status(int *status_out) {
  int v = 0;
  B200_CUDA(cudaDeviceSynchronize());
  B200_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    B200_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  }
  if (status_out) *status_out = v;
  return 0;
}

// lda / ldb / ldd: row pitches in elements of A, B and of C = D as stored (0 = packed); a_m_extent: how many of A's M
// rows (or columns, when A is stored [K][M]) exist in memory, the rest of M reads as zeros (0 = all M).
static int matmul_impl(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                       float alpha, float beta, const void *A, const void *B, const void *C, void *D,
                       uint64_t workspaceBytes, void *workspace, int64_t lda, int64_t ldb, int64_t ldd, int a_m_extent,
                       void *stream) {
  const bool packed = lda == 0 && ldb == 0 && ldd == 0 && a_m_extent == 0;
  if (lda == 0) lda = to_trans_a ? K : M;
  if (ldb == 0) ldb = to_trans_b ? N : K;
  if (ldd == 0) ldd = M;
  if (a_m_extent == 0) a_m_extent = M;
  B200_REQUIRE(a_dt == B200_DT_BF16 && b_dt == B200_DT_BF16, "matmul: A and B must be bf16 (got %d, %d)", a_dt, b_dt);
  B200_REQUIRE(d_dt == B200_DT_BF16 || d_dt == B200_DT_FP32, "matmul: D must be bf16 or fp32 (got %d)", d_dt);
  const bool use_c = (C != nullptr) && (c_dt != B200_DT_NONE) && (beta != 0.0f);
  B200_REQUIRE(!use_c || c_dt == B200_DT_BF16 || c_dt == B200_DT_FP32, "matmul: C must be bf16 or fp32 (got %d)", c_dt);
  B200_REQUIRE(M > 0 && N > 0 && K > 0, "matmul: M, K, N must be positive (got %d, %d, %d)", M, K, N);
  // every dimension that is the contiguous one of some operand must keep rows 16-byte aligned
  B200_REQUIRE(M % 8 == 0, "matmul: M must be a multiple of 8 (got %d)", M);
  B200_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldd % 8 == 0 && lda >= (to_trans_a ? K : a_m_extent) &&
                   ldb >= (to_trans_b ? N : K) && ldd >= M && a_m_extent >= 1 && a_m_extent <= M,
               "matmul: the contiguous dimension of every operand (or its row pitch) must be a multiple of 8 elements and "
               "cover the row (M %d, K %d, N %d, pitches %lld, %lld, %lld)", M, K, N, (long long)lda, (long long)ldb,
               (long long)ldd);
  B200_REQUIRE(A && B && D, "matmul: null operand");
  B200_REQUIRE(b200_aligned16(D) && b200_aligned16(C), "matmul: C and D must be 16-byte aligned");

  // Row-major view: D_rm[N][M] = Brm . Arm^T. Kernel rows come from B, kernel columns from A.
  GemmParams p;
  zero_params(p);
  p.group_mode = DENSE;
  p.num_groups = 1;
  p.M = N;
  p.N = M;
  p.K = K;
  p.a_mn_major = to_trans_b ? 1 : 0;  // B stored [N][K] when not transposed, [K][N] when transposed
  p.b_mn_major = to_trans_a ? 0 : 1;  // A stored [M][K] when transposed, [K][M] when not
  p.k_segments = 1;
  p.alpha = alpha;
  p.beta = use_c ? beta : 0.0f;
  p.out_fp32 = d_dt == B200_DT_FP32;
  p.c_fp32 = c_dt == B200_DT_FP32;
  p.D = D;
  p.C = use_c ? C : nullptr;
  p.ldd = ldd;
  if (p.a_mn_major) {
    if (make_tmap(&p.tmA, B, 2, (uint64_t)N, (uint64_t)K, 1, (uint64_t)ldb * 2, 0)) return -1;
  } else {
    if (make_tmap(&p.tmA, B, 2, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldb * 2, 0)) return -1;
  }
  if (p.b_mn_major) {
    if (make_tmap(&p.tmB, A, 3, (uint64_t)a_m_extent, (uint64_t)K, 1, (uint64_t)lda * 2, (uint64_t)lda * K * 2)) return -1;
  } else {
    if (make_tmap(&p.tmB, A, 3, (uint64_t)K, (uint64_t)a_m_extent, 1, (uint64_t)lda * 2, (uint64_t)lda * a_m_extent * 2))
      return -1;
  }
  p.tmA2 = p.tmA;
  p.tmB2 = p.tmB;
  const int64_t tiles = (int64_t)((N + BM - 1) / BM) * ((M + 255) / 256);
  // a 256-row pair tile only pays off when there are at least 256 output rows
  const bool pair_ok = N >= 256;
  // Few output tiles and a long reduction (the router's GEMMs): cut the reduction so that every SM gets a tile.
  // Needs fp32 scratch for the partial results; without it (or when it is too small) the plain form runs.
  const int64_t launched_tiles = (pair_ok && pair_mode()) ? (int64_t)((N + 255) / 256) * ((M + 255) / 256) : tiles;
  const int sms = sm_count_cached();
  const int64_t units = (pair_ok && pair_mode()) ? sms / 2 : sms;
  int splits = 1;
  if (packed && workspace != nullptr && b200_aligned16(workspace) && launched_tiles * 2 <= units && K >= 2048 && M % 4 == 0) {
    splits = (int)std::min<int64_t>(std::min<int64_t>(units / launched_tiles, K / 1024), 16);
    const uint64_t per_split = (uint64_t)N * M * sizeof(float);
    if ((uint64_t)splits * per_split > workspaceBytes) splits = (int)(workspaceBytes / per_split);
  }
  if (splits < 2) return launch_gemm<EPI_STORE>(p, tiles, (cudaStream_t)stream, pair_ok, (N + 255) / 256);
  const int split_len = (((K + splits - 1) / splits) + BK - 1) / BK * BK;
  splits = (K + split_len - 1) / split_len;
  p.k_splits = splits;
  p.k_split_len = split_len;
  p.alpha = 1.0f;
  p.beta = 0.0f;
  p.C = nullptr;
  p.out_fp32 = 1;
  p.D = workspace;
  p.d_group_stride = (int64_t)N * M;
  if (launch_gemm<EPI_STORE>(p, tiles * splits, (cudaStream_t)stream, pair_ok, (int64_t)((N + 255) / 256) * splits)) return -1;
  const int64_t n = (int64_t)N * M;
  splitk_reduce_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      n, splits, static_cast<const float *>(workspace), alpha, use_c ? beta : 0.0f, use_c ? C : nullptr,
      c_dt == B200_DT_FP32, D, d_dt == B200_DT_FP32);
  B200_CHECK_LAUNCH("matmul split-k reduce");
  return 0;
}

extern "C" int b200_matmul(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                           float alpha, float beta, const void *A, const void *B, const void *C, void *D,
                           uint64_t workspaceBytes, void *workspace, void *stream) {
  B200_REQUIRE(!(to_trans_a || !to_trans_b) || K % 8 == 0, "matmul: K must be a multiple of 8 for this layout (got %d)", K);
  B200_REQUIRE(!to_trans_b || N % 8 == 0, "matmul: N must be a multiple of 8 when B is transposed (got %d)", N);
  return matmul_impl(a_dt, b_dt, c_dt, d_dt, to_trans_a, to_trans_b, M, K, N, alpha, beta, A, B, C, D, workspaceBytes,
                     workspace, 0, 0, 0, 0, stream);
}

extern "C" int b200_matmul_strided(int a_dt, int b_dt, int c_dt, int d_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                                   float alpha, float beta, const void *A, int64_t lda, int a_m_extent, const void *B,
                                   int64_t ldb, const void *C, void *D, int64_t ldd, void *stream) {
  B200_REQUIRE(lda > 0 && ldb > 0 && ldd > 0 && a_m_extent > 0, "matmul_strided: pitches and extent must be positive");
  return matmul_impl(a_dt, b_dt, c_dt, d_dt, to_trans_a, to_trans_b, M, K, N, alpha, beta, A, B, C, D, 0, nullptr, lda, ldb,
                     ldd, a_m_extent, stream);
}

static int check_grouped(const char *op, int total_rows, int model_dim, int ffn_dim, int num_experts,
                         const int *counts, const int *cumsum) {
  B200_REQUIRE(total_rows >= 0, "%s: negative row count", op);
  B200_REQUIRE(model_dim > 0 && model_dim % 8 == 0 && ffn_dim > 0 && ffn_dim % 8 == 0,
               "%s: model_dim and ffn_dim must be positive multiples of 8 (got %d, %d)", op, model_dim, ffn_dim);
  B200_REQUIRE(num_experts >= 1 && num_experts <= MAX_GROUPS, "%s: need 1 <= num_experts <= %d (got %d)", op, MAX_GROUPS,
               num_experts);
  B200_REQUIRE(counts && cumsum, "%s: expert_counts / expert_counts_cumsum missing", op);
  return 0;
}

// Where the rows of the last GEMM of a pass go when they are not stored in place: see GemmParams::row_tags.
struct RowScatter {
  const unsigned long long *row_tags;
  const unsigned long long *buffers;  // host array, one device address per rank
  int world;
  int64_t rows_per_buffer;
};

static int apply_scatter(const char *op, GemmParams &p, const RowScatter *sc) {
  if (!sc) return 0;
  B200_REQUIRE(sc->row_tags && sc->buffers && sc->world >= 1 && sc->world <= SCATTER_MAX_RANKS && sc->rows_per_buffer >= 0,
               "%s: bad scatter description (world %d, at most %d ranks)", op, sc->world, SCATTER_MAX_RANKS);
  for (int i = 0; i < sc->world; i++)
    B200_REQUIRE(sc->buffers[i] != 0 && (sc->buffers[i] & 15ull) == 0, "%s: destination buffer %d missing or unaligned", op, i);
  p.row_tags = sc->row_tags;
  p.scatter_world = sc->world;
  p.scatter_rows = sc->rows_per_buffer;
  for (int i = 0; i < sc->world; i++) p.scatter_base[i] = sc->buffers[i];
  p.D = reinterpret_cast<void *>(sc->buffers[0]);  // never written through: only its alignment is looked at
  return 0;
}

static int experts_fwd_impl(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *zone,
                            const void *W1, const void *W3, const void *W2, int64_t w1_stride_elems,
                            int64_t w3_stride_elems, int64_t w2_stride_elems, const int *expert_counts,
                            const int *expert_counts_cumsum, void *x1, void *x3, void *h, void *Y,
                            const RowScatter *sc, void *stream) {
  if (check_grouped("moe_experts_fwd", total_rows, model_dim, ffn_dim, num_experts, expert_counts, expert_counts_cumsum))
    return -1;
  B200_REQUIRE(zone && W1 && W3 && x1 && x3 && h && (W2 || (!Y && !sc)), "moe_experts_fwd: null buffer");
  B200_REQUIRE(w1_stride_elems % 8 == 0 && w3_stride_elems % 8 == 0 && w2_stride_elems % 8 == 0,
               "moe_experts_fwd: expert strides must be multiples of 8 elements");
  B200_REQUIRE(b200_aligned16(x1) && b200_aligned16(x3) && b200_aligned16(h) && b200_aligned16(Y),
               "moe_experts_fwd: outputs must be 16-byte aligned");
  if (total_rows == 0) return 0;
  const int64_t m_tiles_max = (int64_t)(total_rows + BM - 1) / BM + num_experts;
  cudaStream_t s = (cudaStream_t)stream;
  {
    // x1 | x3 = Z [W1 ; W3]^T with the SwiGLU epilogue
    GemmParams p;
    zero_params(p);
    p.group_mode = GROUPED_M;
    p.num_groups = num_experts;
    p.N = ffn_dim;
    p.K = model_dim;
    p.dual_b = 1;
    p.k_segments = 1;
    p.counts = expert_counts;
    p.cumsum_incl = expert_counts_cumsum;
    p.x1_out = x1;
    p.x3_out = x3;
    p.h_out = h;
    if (make_tmap(&p.tmA, zone, 2, (uint64_t)model_dim, (uint64_t)total_rows, 1, (uint64_t)model_dim * 2, 0)) return -1;
    if (make_tmap(&p.tmB, W1, 3, (uint64_t)model_dim, (uint64_t)ffn_dim, (uint64_t)num_experts, (uint64_t)model_dim * 2,
                  (uint64_t)w1_stride_elems * 2))
      return -1;
    if (make_tmap(&p.tmB2, W3, 3, (uint64_t)model_dim, (uint64_t)ffn_dim, (uint64_t)num_experts,
                  (uint64_t)model_dim * 2, (uint64_t)w3_stride_elems * 2))
      return -1;
    p.tmA2 = p.tmA;
    if (launch_gemm<EPI_SWIGLU_FWD>(p, m_tiles_max * ((ffn_dim + 127) / 128), s, true, total_rows / 256)) return -1;
  }
  if (Y == nullptr && sc == nullptr) return 0;  // gate-up only (recompute of x1, x3, h)
  {
    // Y = h W2^T
    GemmParams p;
    zero_params(p);
    p.group_mode = GROUPED_M;
    p.num_groups = num_experts;
    p.N = model_dim;
    p.K = ffn_dim;
    p.k_segments = 1;
    p.counts = expert_counts;
    p.cumsum_incl = expert_counts_cumsum;
    p.alpha = 1.0f;
    p.D = Y;
    p.ldd = model_dim;
    if (apply_scatter("moe_experts_fwd_scatter", p, sc)) return -1;
    if (make_tmap(&p.tmA, h, 2, (uint64_t)ffn_dim, (uint64_t)total_rows, 1, (uint64_t)ffn_dim * 2, 0)) return -1;
    if (make_tmap(&p.tmB, W2, 3, (uint64_t)ffn_dim, (uint64_t)model_dim, (uint64_t)num_experts, (uint64_t)ffn_dim * 2,
                  (uint64_t)w2_stride_elems * 2))
      return -1;
    p.tmA2 = p.tmA;
    p.tmB2 = p.tmB;
    if (launch_gemm<EPI_STORE>(p, m_tiles_max * ((model_dim + 255) / 256), s, true, total_rows / 256)) return -1;
  }
  return 0;
}

extern "C" int b200_moe_experts_fwd(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *zone,
                                    const void *W1, const void *W3, const void *W2, int64_t w1_stride_elems,
                                    int64_t w3_stride_elems, int64_t w2_stride_elems, const int *expert_counts,
                                    const int *expert_counts_cumsum, void *x1, void *x3, void *h, void *Y,
                                    void *stream) {
  return experts_fwd_impl(total_rows, model_dim, ffn_dim, num_experts, zone, W1, W3, W2, w1_stride_elems,
                          w3_stride_elems, w2_stride_elems, expert_counts, expert_counts_cumsum, x1, x3, h, Y, nullptr,
                          stream);
}

extern "C" int b200_moe_experts_fwd_scatter(int total_rows, int model_dim, int ffn_dim, int num_experts,
                                            const void *zone, const void *W1, const void *W3, const void *W2,
                                            int64_t w1_stride_elems, int64_t w3_stride_elems, int64_t w2_stride_elems,
                                            const int *expert_counts, const int *expert_counts_cumsum, void *x1,
                                            void *x3, void *h, const unsigned long long *row_tags,
                                            const unsigned long long *dest_buffers, int world,
                                            int64_t rows_per_buffer, void *stream) {
  RowScatter sc = {row_tags, dest_buffers, world, rows_per_buffer};
  return experts_fwd_impl(total_rows, model_dim, ffn_dim, num_experts, zone, W1, W3, W2, w1_stride_elems,
                          w3_stride_elems, w2_stride_elems, expert_counts, expert_counts_cumsum, x1, x3, h, nullptr,
                          &sc, stream);
}

static int experts_bwd_x_impl(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                              const float *row_weights, const void *x1, const void *x3, const void *W1,
                              const void *W3, const void *W2, int64_t w1_stride_elems, int64_t w3_stride_elems,
                              int64_t w2_stride_elems, const int *expert_counts, const int *expert_counts_cumsum,
                              void *dx1, void *dx3, void *hs, float *dP, void *dZ, const RowScatter *sc,
                              void *stream) {
  if (check_grouped("moe_experts_bwd_x", total_rows, model_dim, ffn_dim, num_experts, expert_counts,
                    expert_counts_cumsum))
    return -1;
  B200_REQUIRE(dY_zone && row_weights && x1 && x3 && W1 && W3 && W2 && dx1 && dx3 && dP && (dZ || sc),
               "moe_experts_bwd_x: null buffer");
  B200_REQUIRE(w1_stride_elems % 8 == 0 && w3_stride_elems % 8 == 0 && w2_stride_elems % 8 == 0,
               "moe_experts_bwd_x: expert strides must be multiples of 8 elements");
  B200_REQUIRE(b200_aligned16(x1) && b200_aligned16(x3) && b200_aligned16(dx1) && b200_aligned16(dx3) &&
                   b200_aligned16(hs) && b200_aligned16(dZ),
               "moe_experts_bwd_x: buffers must be 16-byte aligned");
  if (total_rows == 0) return 0;
  const int64_t m_tiles_max = (int64_t)(total_rows + BM - 1) / BM + num_experts;
  cudaStream_t s = (cudaStream_t)stream;
  {
    // dh = dY W2 (W2_e is [model_dim][ffn_dim]: the reduction index is the slow one -> MN-major B)
    GemmParams p;
    zero_params(p);
    p.group_mode = GROUPED_M;
    p.num_groups = num_experts;
    p.N = ffn_dim;
    p.K = model_dim;
    p.b_mn_major = 1;
    p.k_segments = 1;
    p.counts = expert_counts;
    p.cumsum_incl = expert_counts_cumsum;
    p.x1_in = x1;
    p.x3_in = x3;
    p.row_w = row_weights;
    p.dx1 = dx1;
    p.dx3 = dx3;
    p.hs = hs;
    p.dP = dP;
    if (make_tmap(&p.tmA, dY_zone, 2, (uint64_t)model_dim, (uint64_t)total_rows, 1, (uint64_t)model_dim * 2, 0))
      return -1;
    if (make_tmap(&p.tmB, W2, 3, (uint64_t)ffn_dim, (uint64_t)model_dim, (uint64_t)num_experts, (uint64_t)ffn_dim * 2,
                  (uint64_t)w2_stride_elems * 2))
      return -1;
    p.tmA2 = p.tmA;
    p.tmB2 = p.tmB;
    if (launch_gemm<EPI_SWIGLU_BWD>(p, m_tiles_max * ((ffn_dim + 255) / 256), s, true, total_rows / 256)) return -1;
  }
  {
    // dZ = dx1 W1 + dx3 W3: one accumulator, two reduction segments
    GemmParams p;
    zero_params(p);
    p.group_mode = GROUPED_M;
    p.num_groups = num_experts;
    p.N = model_dim;
    p.K = ffn_dim;
    p.b_mn_major = 1;
    p.k_segments = 2;
    p.counts = expert_counts;
    p.cumsum_incl = expert_counts_cumsum;
    p.alpha = 1.0f;
    p.D = dZ;
    p.ldd = model_dim;
    if (apply_scatter("moe_experts_bwd_x_scatter", p, sc)) return -1;
    if (make_tmap(&p.tmA, dx1, 2, (uint64_t)ffn_dim, (uint64_t)total_rows, 1, (uint64_t)ffn_dim * 2, 0)) return -1;
    if (make_tmap(&p.tmA2, dx3, 2, (uint64_t)ffn_dim, (uint64_t)total_rows, 1, (uint64_t)ffn_dim * 2, 0)) return -1;
    if (make_tmap(&p.tmB, W1, 3, (uint64_t)model_dim, (uint64_t)ffn_dim, (uint64_t)num_experts, (uint64_t)model_dim * 2,
                  (uint64_t)w1_stride_elems * 2))
      return -1;
    if (make_tmap(&p.tmB2, W3, 3, (uint64_t)model_dim, (uint64_t)ffn_dim, (uint64_t)num_experts,
                  (uint64_t)model_dim * 2, (uint64_t)w3_stride_elems * 2))
      return -1;
    if (launch_gemm<EPI_STORE>(p, m_tiles_max * ((model_dim + 255) / 256), s, true, total_rows / 256)) return -1;
  }
  return 0;
}

extern "C" int b200_moe_experts_bwd_x(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                                      const float *row_weights, const void *x1, const void *x3, const void *W1,
                                      const void *W3, const void *W2, int64_t w1_stride_elems, int64_t w3_stride_elems,
                                      int64_t w2_stride_elems, const int *expert_counts,
                                      const int *expert_counts_cumsum, void *dx1, void *dx3, void *hs, float *dP,
                                      void *dZ, void *stream) {
  return experts_bwd_x_impl(total_rows, model_dim, ffn_dim, num_experts, dY_zone, row_weights, x1, x3, W1, W3, W2,
                            w1_stride_elems, w3_stride_elems, w2_stride_elems, expert_counts, expert_counts_cumsum, dx1,
                            dx3, hs, dP, dZ, nullptr, stream);
}

extern "C" int b200_moe_experts_bwd_x_scatter(int total_rows, int model_dim, int ffn_dim, int num_experts,
                                              const void *dY_zone, const float *row_weights, const void *x1,
                                              const void *x3, const void *W1, const void *W3, const void *W2,
                                              int64_t w1_stride_elems, int64_t w3_stride_elems,
                                              int64_t w2_stride_elems, const int *expert_counts,
                                              const int *expert_counts_cumsum, void *dx1, void *dx3, void *hs,
                                              float *dP, const unsigned long long *row_tags,
                                              const unsigned long long *dest_buffers, int world,
                                              int64_t rows_per_buffer, void *stream) {
  RowScatter sc = {row_tags, dest_buffers, world, rows_per_buffer};
  return experts_bwd_x_impl(total_rows, model_dim, ffn_dim, num_experts, dY_zone, row_weights, x1, x3, W1, W3, W2,
                            w1_stride_elems, w3_stride_elems, w2_stride_elems, expert_counts, expert_counts_cumsum, dx1,
                            dx3, hs, dP, nullptr, &sc, stream);
}

// One grouped wgrad: dW[e][Mrows][Ncols] += A[rows_e, Mrows]^T . B[rows_e, Ncols]
static int launch_wgrad(int total_rows, int Mrows, int Ncols, int num_experts, const void *A, const void *B, void *dW,
                        int64_t dw_stride, const int *counts, const int *cumsum, bool accumulate, cudaStream_t s) {
  B200_REQUIRE(dw_stride % 8 == 0 && b200_aligned16(dW), "moe_experts_bwd_w: gradient buffers must be 16-byte aligned");
  GemmParams p;
  zero_params(p);
  p.group_mode = GROUPED_K;
  p.num_groups = num_experts;
  p.M = Mrows;
  p.N = Ncols;
  p.a_mn_major = 1;
  p.b_mn_major = 1;
  p.k_segments = 1;
  p.counts = counts;
  p.cumsum_incl = cumsum;
  p.alpha = 1.0f;
  p.beta = accumulate ? 1.0f : 0.0f;
  p.D = dW;
  p.C = accumulate ? dW : nullptr;  // without it the epilogue does not read the old gradient at all
  p.ldd = Ncols;
  p.d_group_stride = dw_stride;
  p.k_hint = total_rows / num_experts;
  if (make_tmap(&p.tmA, A, 2, (uint64_t)Mrows, (uint64_t)total_rows, 1, (uint64_t)Mrows * 2, 0)) return -1;
  if (make_tmap(&p.tmB, B, 3, (uint64_t)Ncols, (uint64_t)total_rows, 1, (uint64_t)Ncols * 2,
                (uint64_t)Ncols * 2 * (uint64_t)total_rows))
    return -1;
  p.tmA2 = p.tmA;
  p.tmB2 = p.tmB;
  const int64_t tiles = (int64_t)num_experts * ((Mrows + BM - 1) / BM) * ((Ncols + 255) / 256);
  return launch_gemm<EPI_STORE>(p, tiles, s, true, (int64_t)num_experts * ((Mrows + 255) / 256));
}

static int experts_bwd_w(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone, const void *hs,
                         const void *zone_x, const void *dx1, const void *dx3, void *dW1, void *dW3, void *dW2,
                         int64_t dw1_stride_elems, int64_t dw3_stride_elems, int64_t dw2_stride_elems,
                         const int *expert_counts, const int *expert_counts_cumsum, bool accumulate, void *stream) {
  if (check_grouped("moe_experts_bwd_w", total_rows, model_dim, ffn_dim, num_experts, expert_counts,
                    expert_counts_cumsum))
    return -1;
  if (total_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dW2) {
    B200_REQUIRE(dY_zone && hs, "moe_experts_bwd_w: dW2 needs dY_zone and hs");
    if (launch_wgrad(total_rows, model_dim, ffn_dim, num_experts, dY_zone, hs, dW2, dw2_stride_elems, expert_counts,
                     expert_counts_cumsum, accumulate, s))
      return -1;
  }
  if (dW1) {
    B200_REQUIRE(dx1 && zone_x, "moe_experts_bwd_w: dW1 needs dx1 and zone_x");
    if (launch_wgrad(total_rows, ffn_dim, model_dim, num_experts, dx1, zone_x, dW1, dw1_stride_elems, expert_counts,
                     expert_counts_cumsum, accumulate, s))
      return -1;
  }
  if (dW3) {
    B200_REQUIRE(dx3 && zone_x, "moe_experts_bwd_w: dW3 needs dx3 and zone_x");
    if (launch_wgrad(total_rows, ffn_dim, model_dim, num_experts, dx3, zone_x, dW3, dw3_stride_elems, expert_counts,
                     expert_counts_cumsum, accumulate, s))
      return -1;
  }
  return 0;
}

extern "C" int b200_moe_experts_bwd_w(int total_rows, int model_dim, int ffn_dim, int num_experts, const void *dY_zone,
                                      const void *hs, const void *zone_x, const void *dx1, const void *dx3, void *dW1,
                                      void *dW3, void *dW2, int64_t dw1_stride_elems, int64_t dw3_stride_elems,
                                      int64_t dw2_stride_elems, const int *expert_counts,
                                      const int *expert_counts_cumsum, void *stream) {
  return experts_bwd_w(total_rows, model_dim, ffn_dim, num_experts, dY_zone, hs, zone_x, dx1, dx3, dW1, dW3, dW2,
                       dw1_stride_elems, dw3_stride_elems, dw2_stride_elems, expert_counts, expert_counts_cumsum, true, stream);
}

extern "C" int b200_moe_experts_bwd_w_overwrite(int total_rows, int model_dim, int ffn_dim, int num_experts,
                                                const void *dY_zone, const void *hs, const void *zone_x, const void *dx1,
                                                const void *dx3, void *dW1, void *dW3, void *dW2, int64_t dw1_stride_elems,
                                                int64_t dw3_stride_elems, int64_t dw2_stride_elems,
                                                const int *expert_counts, const int *expert_counts_cumsum, void *stream) {
  return experts_bwd_w(total_rows, model_dim, ffn_dim, num_experts, dY_zone, hs, zone_x, dx1, dx3, dW1, dW3, dW2,
                       dw1_stride_elems, dw3_stride_elems, dw2_stride_elems, expert_counts, expert_counts_cumsum, false, stream);
}
