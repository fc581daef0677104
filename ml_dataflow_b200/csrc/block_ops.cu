// Bandwidth-bound ops of the transformer block around the MoE feed-forward and of the model head, bf16 with fp32
// arithmetic: RMSNorm (forward, recompute, backward-x, backward-w), RoPE (forward, backward), softmax,
// cross-entropy, average loss, AdamW, embedding table (forward, backward-w). Same argument order and meaning as the
// reference's submitters (libdataflowops/include/dataflow_ops.h:136-213, 298-316). Every kernel streams its rows
// once with 16-byte accesses that bypass L1, keeps a row in registers between its reduction and its output pass, and
// runs on a grid of a few blocks per SM that strides over the rows.
#include "common.cuh"
#include "../../include/b200_moe.h"

namespace b200 {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VPT = 4;  // 16-byte vectors a thread keeps per row: rows of up to 8192 columns stay in registers

// sum over the block; every thread gets the result. scratch: 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  __syncthreads();  // scratch may still be read from the previous use
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? scratch[lane] : 0.0f;
  return warp_sum(t);
}

// out = bf16(x * r * w), r = rsqrt(mean(x^2) + eps) (norm/rms_norm.cu:226-340 of the reference), or r taken from
// rms_in (norm/rms_norm_recompute.cu:63-133). VPT == 0: rows longer than the register budget are read twice.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_kernel(int n_rows, int n_vec, float inv_n, float eps, const uint4 *__restrict__ w, const uint4 *__restrict__ X,
                uint4 *__restrict__ out, float *__restrict__ rms_out, const float *__restrict__ rms_in) {
  __shared__ float scratch[32];
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const uint4 *x = X + row * n_vec;
    uint4 *o = out + row * n_vec;
    uint4 v[VPT > 0 ? VPT : 1];
    float r;
    if (rms_in == nullptr) {
      float ss = 0.0f;
      if (VPT > 0) {
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int c = i * NORM_THREADS + threadIdx.x;
          if (c < n_vec) v[i] = ld_stream(x + c);
        }
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int c = i * NORM_THREADS + threadIdx.x;
          if (c < n_vec) {
            float f[8];
            unpack8(v[i], f);
#pragma unroll
            for (int q = 0; q < 8; q++) ss += f[q] * f[q];
          }
        }
      } else {
        for (int c = threadIdx.x; c < n_vec; c += NORM_THREADS) {
          float f[8];
          unpack8(x[c], f);
#pragma unroll
          for (int q = 0; q < 8; q++) ss += f[q] * f[q];
        }
      }
      ss = block_sum(ss, scratch);
      r = rsqrtf(ss * inv_n + eps);
      if (rms_out != nullptr && threadIdx.x == 0) rms_out[row] = r;
    } else {
      r = rms_in[row];
      if (VPT > 0) {
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int c = i * NORM_THREADS + threadIdx.x;
          if (c < n_vec) v[i] = ld_stream(x + c);
        }
      }
    }
    if (VPT > 0) {
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int c = i * NORM_THREADS + threadIdx.x;
        if (c < n_vec) {
          float f[8], g[8];
          unpack8(v[i], f);
          unpack8(__ldg(w + c), g);
#pragma unroll
          for (int q = 0; q < 8; q++) f[q] = f[q] * r * g[q];
          st_stream(o + c, pack8(f));
        }
      }
    } else {
      for (int c = threadIdx.x; c < n_vec; c += NORM_THREADS) {
        float f[8], g[8];
        unpack8(x[c], f);
        unpack8(__ldg(w + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) f[q] = f[q] * r * g[q];
        st_stream(o + c, pack8(f));
      }
    }
  }
}

// norm/rms_norm_bwd_x.cu:241-394: C = sum_c (x r w) up; dX = bf16(f32(dX) + r (up w - (C / n) x r)); X_out (optional)
// = bf16(x r w). The row of X and of the upstream gradient stay in registers between the two passes.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_bwd_x_kernel(int n_rows, int n_vec, float inv_n, const float *__restrict__ rms, const uint4 *__restrict__ w,
                      const uint4 *__restrict__ X, const uint4 *__restrict__ up, uint4 *__restrict__ dX,
                      uint4 *__restrict__ X_out) {
  __shared__ float scratch[32];
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const int64_t base = row * n_vec;
    const float r = rms[row];
    uint4 xv[VPT], uv[VPT], dv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int c = i * NORM_THREADS + threadIdx.x;
      if (c < n_vec) {
        xv[i] = ld_stream(X + base + c);
        uv[i] = ld_stream(up + base + c);
        dv[i] = dX[base + c];
      }
    }
    float csum = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int c = i * NORM_THREADS + threadIdx.x;
      if (c < n_vec) {
        float x[8], u[8], g[8], o[8];
        unpack8(xv[i], x);
        unpack8(uv[i], u);
        unpack8(__ldg(w + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) {
          o[q] = x[q] * r * g[q];
          csum += o[q] * u[q];
        }
        if (X_out != nullptr) st_stream(X_out + base + c, pack8(o));
      }
    }
    const float c_div_n = block_sum(csum, scratch) * inv_n;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int c = i * NORM_THREADS + threadIdx.x;
      if (c < n_vec) {
        float x[8], u[8], g[8], d[8];
        unpack8(xv[i], x);
        unpack8(uv[i], u);
        unpack8(__ldg(w + c), g);
        unpack8(dv[i], d);
#pragma unroll
        for (int q = 0; q < 8; q++) d[q] += r * (u[q] * g[q] - c_div_n * (x[q] * r));
        dX[base + c] = pack8(d);
      }
    }
  }
}

// Rows of up to 4096 columns (forward) / 2048 columns (backward-x): one WARP per row, the whole row in the lanes'
// registers, reduction by shuffles only. No block-wide barrier sits between a row's loads and its stores, and a block
// of eight warps keeps eight rows in flight, which is what a few-KB row needs to cover the memory latency.
constexpr int NORM_WARPS = 8;

template <int VPL>  // 16-byte vectors per lane: the row has at most 32 * VPL of them
__global__ void __launch_bounds__(NORM_WARPS * 32)
rms_norm_warp_kernel(int n_rows, int n_vec, float inv_n, float eps, const uint4 *__restrict__ w, const uint4 *__restrict__ X,
                     uint4 *__restrict__ out, float *__restrict__ rms_out, const float *__restrict__ rms_in) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * NORM_WARPS;
  for (int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5); row < n_rows; row += warps) {
    const uint4 *x = X + row * n_vec;
    uint4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c < n_vec) v[i] = ld_stream(x + c);
    }
    float r;
    if (rms_in == nullptr) {
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < VPL; i++) {
        if (i * 32 + lane < n_vec) {
          float f[8];
          unpack8(v[i], f);
#pragma unroll
          for (int q = 0; q < 8; q++) ss += f[q] * f[q];
        }
      }
      r = rsqrtf(warp_sum(ss) * inv_n + eps);
      if (rms_out != nullptr && lane == 0) rms_out[row] = r;
    } else {
      r = rms_in[row];
    }
    uint4 *o = out + row * n_vec;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c < n_vec) {
        float f[8], g[8];
        unpack8(v[i], f);
        unpack8(__ldg(w + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) f[q] = f[q] * r * g[q];
        st_stream(o + c, pack8(f));
      }
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rms_norm_bwd_x_warp_kernel(int n_rows, int n_vec, float inv_n, const float *__restrict__ rms, const uint4 *__restrict__ w,
                           const uint4 *__restrict__ X, const uint4 *__restrict__ up, uint4 *__restrict__ dX,
                           uint4 *__restrict__ X_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * NORM_WARPS;
  for (int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5); row < n_rows; row += warps) {
    const int64_t base = row * n_vec;
    const float r = rms[row];
    uint4 xv[VPL], uv[VPL], dv[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c < n_vec) {
        xv[i] = ld_stream(X + base + c);
        uv[i] = ld_stream(up + base + c);
        dv[i] = dX[base + c];
      }
    }
    float csum = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c < n_vec) {
        float x[8], u[8], g[8], o[8];
        unpack8(xv[i], x);
        unpack8(uv[i], u);
        unpack8(__ldg(w + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) {
          o[q] = x[q] * r * g[q];
          csum += o[q] * u[q];
        }
        if (X_out != nullptr) st_stream(X_out + base + c, pack8(o));
      }
    }
    const float c_div_n = warp_sum(csum) * inv_n;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c < n_vec) {
        float x[8], u[8], g[8], d[8];
        unpack8(xv[i], x);
        unpack8(uv[i], u);
        unpack8(__ldg(w + c), g);
        unpack8(dv[i], d);
#pragma unroll
        for (int q = 0; q < 8; q++) d[q] += r * (u[q] * g[q] - c_div_n * (x[q] * r));
        dX[base + c] = pack8(d);
      }
    }
  }
}

// Weight gradient of RMSNorm, first pass (norm/rms_norm_bwd_w.cu:225-325): block b sums up * x * r over its slice of
// the rows for every column into partial[b][.] (fp32). Thread = one 8-column vector; eight rows in flight.
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_bwd_w_partial_kernel(int n_rows, int n_vec, const float *__restrict__ rms, const uint4 *__restrict__ X,
                              const uint4 *__restrict__ up, float *__restrict__ partial) {
  const int blocks = gridDim.y;
  const int per = (n_rows + blocks - 1) / blocks;
  const int r0 = blockIdx.y * per, r1 = min(n_rows, r0 + per);
  const int c = blockIdx.x * NORM_THREADS + threadIdx.x;
  if (c >= n_vec) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int row = r0;
  for (; row + 8 <= r1; row += 8) {
    uint4 xv[8], uv[8];
    float rv[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      xv[j] = ld_stream(X + (int64_t)(row + j) * n_vec + c);
      uv[j] = ld_stream(up + (int64_t)(row + j) * n_vec + c);
      rv[j] = rms[row + j];
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      float x[8], u[8];
      unpack8(xv[j], x);
      unpack8(uv[j], u);
#pragma unroll
      for (int q = 0; q < 8; q++) acc[q] += u[q] * x[q] * rv[j];
    }
  }
  for (; row < r1; row++) {
    float x[8], u[8];
    unpack8(ld_stream(X + (int64_t)row * n_vec + c), x);
    unpack8(ld_stream(up + (int64_t)row * n_vec + c), u);
    const float rv = rms[row];
#pragma unroll
    for (int q = 0; q < 8; q++) acc[q] += u[q] * x[q] * rv;
  }
  float4 *dst = reinterpret_cast<float4 *>(partial + ((int64_t)blockIdx.y * n_vec + c) * 8);
  dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// second pass (norm/rms_norm_bwd_w_combine.cu:200-294): dW = bf16(f32(dW) + sum of the slices' partial sums). A
// block takes 32 columns; its 8 warps each add every eighth slice (independent loads, 128 contiguous bytes per warp),
// then the eight sums are added in warp order: the same order on every run.
__global__ void __launch_bounds__(256)
rms_norm_bwd_w_combine_kernel(int n_cols, int blocks, const float *__restrict__ partial, __nv_bfloat16 *__restrict__ dW) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.0f;
  if (c < n_cols) {
    int b = grp;
    for (; b + 24 < blocks; b += 32) {
      const float v0 = partial[(int64_t)b * n_cols + c], v1 = partial[(int64_t)(b + 8) * n_cols + c];
      const float v2 = partial[(int64_t)(b + 16) * n_cols + c], v3 = partial[(int64_t)(b + 24) * n_cols + c];
      s += v0;
      s += v1;
      s += v2;
      s += v3;
    }
    for (; b < blocks; b += 8) s += partial[(int64_t)b * n_cols + c];
  }
  part[grp][lane] = s;
  __syncthreads();
  if (grp == 0 && c < n_cols) {
    float t = 0.0f;
#pragma unroll
    for (int g = 0; g < 8; g++) t += part[g][lane];
    dW[c] = __float2bfloat16_rn(__bfloat162float(dW[c]) + t);
  }
}

// ---- RoPE ----------------------------------------------------------------------------------------------------
// attention_misc/rope.cu:152-256 and rope_bwd_x.cu:146-248: in place on interleaved pairs (2i, 2i+1) of every head,
// angle = pos * theta^(-2i / head_dim); sign = +1 rotates, -1 rotates back. The angles of a token are formed once
// per block (full-precision powf / sincosf: positions reach tens of thousands of radians) and shared by its heads.
constexpr int ROPE_THREADS = 128;
constexpr int ROPE_MAX_HEAD_DIM = 256;

__global__ void __launch_bounds__(ROPE_THREADS)
rope_kernel(int num_tokens, int q_vec, int k_vec, int head_dim, float theta, float sign, const int *__restrict__ seq_positions,
            uint4 *__restrict__ X_q, uint4 *__restrict__ X_k) {
  __shared__ float s_cos[ROPE_MAX_HEAD_DIM / 2], s_sin[ROPE_MAX_HEAD_DIM / 2];
  const int pairs = head_dim >> 1;
  const int head_vec = head_dim >> 3;
  for (int64_t tok = blockIdx.x; tok < num_tokens; tok += gridDim.x) {
    const float pos = (float)seq_positions[tok];
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += ROPE_THREADS) {
      const float inv_freq = powf(theta, -(float)(2 * i) / (float)head_dim);
      float sn, cs;
      sincosf(pos * inv_freq, &sn, &cs);
      s_cos[i] = cs;
      s_sin[i] = sign * sn;
    }
    __syncthreads();
    for (int part = 0; part < 2; part++) {
      uint4 *row = part == 0 ? X_q + tok * q_vec : (X_k ? X_k + tok * k_vec : nullptr);
      const int n_vec = part == 0 ? q_vec : k_vec;
      if (row == nullptr) continue;
      for (int c = threadIdx.x; c < n_vec; c += ROPE_THREADS) {
        const int p0 = (c % head_vec) * 4;  // first pair of this vector inside its head
        float f[8];
        unpack8(row[c], f);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float cs = s_cos[p0 + j], sn = s_sin[p0 + j];
          const float e = f[2 * j], o = f[2 * j + 1];
          f[2 * j] = cs * e - sn * o;
          f[2 * j + 1] = cs * o + sn * e;
        }
        row[c] = pack8(f);
      }
    }
  }
}

// The same with one WARP per token, for head sizes whose vectors tile a warp (head_dim 64, 128 or 256): vector
// c = lane + 32 i of a row always falls on the same four pairs of its head, so every lane forms just those four
// angles and keeps them in registers; no shared memory, no barrier, all of a token's loads in flight at once.
constexpr int ROPE_WARPS = 4;
constexpr int ROPE_MAX_VPL = 12;  // 16-byte vectors per lane over the q and k rows together

__global__ void __launch_bounds__(ROPE_WARPS * 32)
rope_warp_kernel(int num_tokens, int q_vec, int k_vec, int head_dim, float theta, float sign,
                 const int *__restrict__ seq_positions, uint4 *__restrict__ X_q, uint4 *__restrict__ X_k) {
  const int lane = threadIdx.x & 31;
  const int head_vec = head_dim >> 3;
  const int p0 = (lane % head_vec) * 4;
  float inv_freq[4];
#pragma unroll
  for (int j = 0; j < 4; j++) inv_freq[j] = powf(theta, -(float)(2 * (p0 + j)) / (float)head_dim);
  const int qn = (q_vec + 31) >> 5, kn = (X_k != nullptr) ? (k_vec + 31) >> 5 : 0;
  const int64_t warps = (int64_t)gridDim.x * ROPE_WARPS;
  for (int64_t tok = (int64_t)blockIdx.x * ROPE_WARPS + (threadIdx.x >> 5); tok < num_tokens; tok += warps) {
    uint4 v[ROPE_MAX_VPL];
    uint4 *qrow = X_q + tok * q_vec, *krow = X_k ? X_k + tok * k_vec : nullptr;
#pragma unroll
    for (int i = 0; i < ROPE_MAX_VPL; i++) {
      const int c = (i < qn ? i : i - qn) * 32 + lane;
      if (i < qn) { if (c < q_vec) v[i] = qrow[c]; }
      else if (i < qn + kn) { if (c < k_vec) v[i] = krow[c]; }
    }
    const float pos = (float)seq_positions[tok];
    float cs[4], sn[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
      sn[j] *= sign;
    }
#pragma unroll
    for (int i = 0; i < ROPE_MAX_VPL; i++) {
      const bool is_q = i < qn;
      const int c = (is_q ? i : i - qn) * 32 + lane;
      if (i >= qn + kn || c >= (is_q ? q_vec : k_vec)) continue;
      float f[8];
      unpack8(v[i], f);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float e = f[2 * j], o = f[2 * j + 1];
        f[2 * j] = cs[j] * e - sn[j] * o;
        f[2 * j + 1] = cs[j] * o + sn[j] * e;
      }
      (is_q ? qrow : krow)[c] = pack8(f);
    }
  }
}

// ---- softmax over long rows (the vocabulary) -------------------------------------------------------------------
// loss_misc/softmax.cu:249-394: out = bf16(exp(x - max) / sum). One block per row; pass 1 folds maximum and sum of
// eight elements at a time (one rescale per vector), pass 2 re-reads the row, which is still in L2 (a row of 128 K
// bf16 is 250 KB, a few hundred rows are in flight) and writes the result.
constexpr int SOFTMAX_THREADS = 1024;
constexpr float LOG2E = 1.4426950408889634f;
// exp(a - b) as 2^((a - b) log2 e): the difference is formed first, so the result is as accurate as expf's to within
// the rounding of one multiplication (relative 6e-8 * |a - b|; the differences of a softmax row stay within tens)
__device__ __forceinline__ float exp_diff(float a, float b) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"((a - b) * LOG2E));  // 2 ulp; results below 2^-126 become 0
  return r;
}

__global__ void __launch_bounds__(SOFTMAX_THREADS)
softmax_kernel(int n_rows, int n_cols, const __nv_bfloat16 *__restrict__ X, __nv_bfloat16 *__restrict__ out) {
  __shared__ float s_max[32], s_sum[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = SOFTMAX_THREADS / 32;
  const int n_vec = n_cols >> 3;
  const float NEG = -3.402823466e38f;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const __nv_bfloat16 *x = X + row * n_cols;
    __nv_bfloat16 *o = out + row * n_cols;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(o)) & 15u) == 0;
    const int nv = vec_ok ? n_vec : 0;
    float m = NEG, s = 0.0f;
#pragma unroll 4
    for (int c = threadIdx.x; c < nv; c += SOFTMAX_THREADS) {
      float f[8];
      unpack8(reinterpret_cast<const uint4 *>(x)[c], f);
      float vm = f[0];
#pragma unroll
      for (int q = 1; q < 8; q++) vm = fmaxf(vm, f[q]);
      const float nm = fmaxf(m, vm);
      float part = 0.0f;
#pragma unroll
      for (int q = 0; q < 8; q++) part += exp_diff(f[q], nm);
      s = s * exp_diff(m, nm) + part;
      m = nm;
    }
    for (int c = nv * 8 + threadIdx.x; c < n_cols; c += SOFTMAX_THREADS) {
      const float v = __bfloat162float(x[c]);
      const float nm = fmaxf(m, v);
      s = s * exp_diff(m, nm) + exp_diff(v, nm);
      m = nm;
    }
    // (max, sum) pairs: warp, then block
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float pm = __shfl_xor_sync(0xffffffffu, m, off), ps = __shfl_xor_sync(0xffffffffu, s, off);
      const float nm = fmaxf(m, pm);
      s = s * exp_diff(m, nm) + ps * exp_diff(pm, nm);
      m = nm;
    }
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = m;
      s_sum[warp] = s;
    }
    __syncthreads();
    m = lane < nwarps ? s_max[lane] : NEG;
    s = lane < nwarps ? s_sum[lane] : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float pm = __shfl_xor_sync(0xffffffffu, m, off), ps = __shfl_xor_sync(0xffffffffu, s, off);
      const float nm = fmaxf(m, pm);
      s = s * exp_diff(m, nm) + ps * exp_diff(pm, nm);
      m = nm;
    }
    const float inv_s = 1.0f / s;
#pragma unroll 4
    for (int c = threadIdx.x; c < nv; c += SOFTMAX_THREADS) {
      float f[8];
      unpack8(reinterpret_cast<const uint4 *>(x)[c], f);
#pragma unroll
      for (int q = 0; q < 8; q++) f[q] = exp_diff(f[q], m) * inv_s;
      st_stream(reinterpret_cast<uint4 *>(o) + c, pack8(f));
    }
    for (int c = nv * 8 + threadIdx.x; c < n_cols; c += SOFTMAX_THREADS)
      o[c] = __float2bfloat16_rn(exp_diff(__bfloat162float(x[c]), m) * inv_s);
  }
}

// loss_misc/cross_entropy.cu:48-68: on the softmax output p: loss_vec[row] = -log(p[label]); p[label] -= 1 (bf16)
__global__ void cross_entropy_kernel(int n_rows, int n_cols, __nv_bfloat16 *__restrict__ p, const uint32_t *__restrict__ labels,
                                     float *__restrict__ loss_vec) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows) return;
  __nv_bfloat16 *e = p + (int64_t)row * n_cols + labels[row];
  const float v = __bfloat162float(*e);
  loss_vec[row] = -1.0f * logf(v);
  *e = __float2bfloat16_rn(v - 1.0f);
}

// loss_misc/cross_entropy.cu:70-119: one block; loss_vec[num_tokens] = mean of the entries before it
__global__ void __launch_bounds__(1024) average_loss_kernel(int num_tokens, float *__restrict__ loss_vec) {
  __shared__ float scratch[32];
  float s = 0.0f;
  for (int i = threadIdx.x; i < num_tokens; i += blockDim.x) s += loss_vec[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) loss_vec[num_tokens] = s / (float)num_tokens;
}

// ---- AdamW -----------------------------------------------------------------------------------------------------
// optimizer/adamw_step.cu:6-65, eight elements per thread; c1 = 1 / (1 - beta1^step), c2 = 1 / (1 - beta2^step).
// The bias corrections are multiplications by reciprocals formed once on the host, the square root and the quotient use
// the hardware approximations (2 ulp of fp32, far below the bf16 rounding of the result): three IEEE divisions and an
// IEEE square root per element made the kernel instruction-bound (0.60 of the HBM rate on a 7 B-parameter model). The
// reference builds its kernel with --use_fast_math, i.e. with the same class of approximations.
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void adamw_one(float &p, float g, float &m, float &v, float lr, float b1, float b2, float wd,
                                          float eps, float c1, float c2) {
  m = b1 * m + (1.0f - b1) * g;
  v = b2 * v + (1.0f - b2) * g * g;
  const float m_hat = m * c1, v_hat = v * c2;
  p = p - lr * (__fdividef(m_hat, sqrt_approx(v_hat) + eps) + wd * p);
}

__global__ void __launch_bounds__(256)
adamw_kernel(uint64_t num_els, float lr, float b1, float b2, float wd, float eps, float c1, float c2,
             __nv_bfloat16 *__restrict__ param, const __nv_bfloat16 *__restrict__ grad, __nv_bfloat16 *__restrict__ mean,
             __nv_bfloat16 *__restrict__ var) {
  const uint64_t n_vec = num_els >> 3;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float p[8], g[8], m[8], v[8];
    unpack8(reinterpret_cast<const uint4 *>(param)[i], p);
    unpack8(ld_stream(reinterpret_cast<const uint4 *>(grad) + i), g);
    unpack8(reinterpret_cast<const uint4 *>(mean)[i], m);
    unpack8(reinterpret_cast<const uint4 *>(var)[i], v);
#pragma unroll
    for (int q = 0; q < 8; q++) adamw_one(p[q], g[q], m[q], v[q], lr, b1, b2, wd, eps, c1, c2);
    reinterpret_cast<uint4 *>(param)[i] = pack8(p);
    reinterpret_cast<uint4 *>(mean)[i] = pack8(m);
    reinterpret_cast<uint4 *>(var)[i] = pack8(v);
  }
  // the last num_els % 8 elements
  if (blockIdx.x == 0 && threadIdx.x < (num_els & 7)) {
    const uint64_t i = (n_vec << 3) + threadIdx.x;
    float p = __bfloat162float(param[i]), m = __bfloat162float(mean[i]), v = __bfloat162float(var[i]);
    adamw_one(p, __bfloat162float(grad[i]), m, v, lr, b1, b2, wd, eps, c1, c2);
    param[i] = __float2bfloat16_rn(p);
    mean[i] = __float2bfloat16_rn(m);
    var[i] = __float2bfloat16_rn(v);
  }
}

// ---- embedding table ---------------------------------------------------------------------------------------------
// preprocess/embedding_table.cu:81-116: block per unique token; its table row is read once and stored to every
// position that holds the token.
__global__ void __launch_bounds__(256)
embedding_kernel(int num_unique, int dim_vec, const uint32_t *__restrict__ sorted_ids, const uint32_t *__restrict__ sorted_map,
                 const uint32_t *__restrict__ starts, const uint4 *__restrict__ table, uint4 *__restrict__ output) {
  for (int u = blockIdx.x; u < num_unique; u += gridDim.x) {
    const uint32_t b = starts[u], e = starts[u + 1];
    const uint4 *src = table + (int64_t)sorted_ids[b] * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += blockDim.x) {
      const uint4 v = ld_stream(src + c);
      for (uint32_t i = b; i < e; i++) st_stream(output + (int64_t)sorted_map[i] * dim_vec + c, v);
    }
  }
}

// warp per unique token for rows of up to 256 vectors (embed_dim <= 2048): the row sits in the lanes' registers
constexpr int EMB_WARPS = 8;
template <int VPL>
__global__ void __launch_bounds__(EMB_WARPS * 32)
embedding_warp_kernel(int num_unique, int dim_vec, const uint32_t *__restrict__ sorted_ids, const uint32_t *__restrict__ sorted_map,
                      const uint32_t *__restrict__ starts, const uint4 *__restrict__ table, uint4 *__restrict__ output) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * EMB_WARPS;
  for (int64_t u = (int64_t)blockIdx.x * EMB_WARPS + (threadIdx.x >> 5); u < num_unique; u += warps) {
    const uint32_t b = starts[u], e = starts[u + 1];
    const uint4 *src = table + (int64_t)sorted_ids[b] * dim_vec;
    uint4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++)
      if (i * 32 + lane < dim_vec) v[i] = ld_stream(src + i * 32 + lane);
    for (uint32_t r = b; r < e; r++) {
      uint4 *dst = output + (int64_t)sorted_map[r] * dim_vec;
#pragma unroll
      for (int i = 0; i < VPL; i++)
        if (i * 32 + lane < dim_vec) st_stream(dst + i * 32 + lane, v[i]);
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(EMB_WARPS * 32)
embedding_bwd_w_warp_kernel(int num_unique, int dim_vec, const uint32_t *__restrict__ sorted_ids,
                            const uint32_t *__restrict__ sorted_map, const uint32_t *__restrict__ starts,
                            const uint4 *__restrict__ grad_stream, uint4 *__restrict__ grad_table) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * EMB_WARPS;
  for (int64_t u = (int64_t)blockIdx.x * EMB_WARPS + (threadIdx.x >> 5); u < num_unique; u += warps) {
    const uint32_t b = starts[u], e = starts[u + 1];
    uint4 *dst = grad_table + (int64_t)sorted_ids[b] * dim_vec;
    if (e - b == 1) {
      // the usual case with a large vocabulary: bf16(0 + g) is g itself, so the row is table + g with one rounding;
      // both rows are requested at once
      const uint4 *src = grad_stream + (int64_t)sorted_map[b] * dim_vec;
      uint4 t[VPL], g4[VPL];
#pragma unroll
      for (int i = 0; i < VPL; i++) {
        if (i * 32 + lane < dim_vec) {
          t[i] = dst[i * 32 + lane];
          g4[i] = ld_stream(src + i * 32 + lane);
        }
      }
#pragma unroll
      for (int i = 0; i < VPL; i++) {
        if (i * 32 + lane < dim_vec) {
          float f[8], g[8];
          unpack8(t[i], f);
          unpack8(g4[i], g);
#pragma unroll
          for (int q = 0; q < 8; q++) f[q] += g[q];
          dst[i * 32 + lane] = pack8(f);
        }
      }
      continue;
    }
    for (int i = 0; i < VPL; i++) {
      const int c = i * 32 + lane;
      if (c >= dim_vec) break;
      const uint4 t = dst[c];
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (uint32_t r = b; r < e; r++) {
        float g[8];
        unpack8(ld_stream(grad_stream + (int64_t)sorted_map[r] * dim_vec + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) acc[q] = bf16_round(acc[q] + g[q]);
      }
      float f[8];
      unpack8(t, f);
#pragma unroll
      for (int q = 0; q < 8; q++) f[q] += acc[q];
      dst[c] = pack8(f);
    }
  }
}

// preprocess/embedding_table_bwd_w.cu:99-145: the gradient rows of a token are added up in bf16, in sorted order,
// from zero (one rounding per addition, as the reference's bf16 shared-memory accumulator does), then added to the
// table row in bf16.
__global__ void __launch_bounds__(256)
embedding_bwd_w_kernel(int num_unique, int dim_vec, const uint32_t *__restrict__ sorted_ids,
                       const uint32_t *__restrict__ sorted_map, const uint32_t *__restrict__ starts,
                       const uint4 *__restrict__ grad_stream, uint4 *__restrict__ grad_table) {
  for (int u = blockIdx.x; u < num_unique; u += gridDim.x) {
    const uint32_t b = starts[u], e = starts[u + 1];
    uint4 *dst = grad_table + (int64_t)sorted_ids[b] * dim_vec;
    for (int c = threadIdx.x; c < dim_vec; c += blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (uint32_t i = b; i < e; i++) {
        float g[8];
        unpack8(ld_stream(grad_stream + (int64_t)sorted_map[i] * dim_vec + c), g);
#pragma unroll
        for (int q = 0; q < 8; q++) acc[q] = bf16_round(acc[q] + g[q]);
      }
      float t[8];
      unpack8(dst[c], t);
#pragma unroll
      for (int q = 0; q < 8; q++) t[q] += acc[q];
      dst[c] = pack8(t);
    }
  }
}

}  // namespace b200

using namespace b200;

static int block_ops_grid(int64_t units, int per_sm) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap = (int64_t)sms * per_sm;
  return (int)(units < cap ? (units > 0 ? units : 1) : cap);
}

#define B200_BF16_ONLY(op, dt) B200_REQUIRE((dt) == B200_DT_BF16, "%s: only bf16 is implemented (datatype code %d)", op, (int)(dt))

static int rms_norm_launch(const char *op, int n_rows, int n_cols, float eps, const void *w, const void *X, void *out,
                           float *rms_out, const float *rms_in, void *stream) {
  B200_REQUIRE(n_rows >= 0 && n_cols > 0 && n_cols % 8 == 0, "%s: n_cols must be a positive multiple of 8 (got %d)", op, n_cols);
  B200_REQUIRE(w && X && out && b200_aligned16(w) && b200_aligned16(X) && b200_aligned16(out),
               "%s: weight, input and output must be non-null and 16-byte aligned", op);
  if (n_rows == 0) return 0;
  const int n_vec = n_cols / 8;
  const int vpt = (n_vec + NORM_THREADS - 1) / NORM_THREADS;
  const int grid = block_ops_grid(n_rows, 8);
  const float inv_n = 1.0f / (float)n_cols;
  cudaStream_t s = (cudaStream_t)stream;
  const uint4 *wv = (const uint4 *)w, *xv = (const uint4 *)X;
  uint4 *ov = (uint4 *)out;
  if (n_vec <= 32 * 16) {
    // warp per row
    const int vpl = (n_vec + 31) / 32;
    const int wgrid = block_ops_grid((n_rows + NORM_WARPS - 1) / NORM_WARPS, 8);
#define B200_RMSW(V) rms_norm_warp_kernel<V><<<wgrid, NORM_WARPS * 32, 0, s>>>(n_rows, n_vec, inv_n, eps, wv, xv, ov, rms_out, rms_in)
    if (vpl <= 2) B200_RMSW(2);
    else if (vpl <= 4) B200_RMSW(4);
    else if (vpl <= 8) B200_RMSW(8);
    else B200_RMSW(16);
#undef B200_RMSW
  } else if (vpt <= 1) rms_norm_kernel<1><<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, inv_n, eps, wv, xv, ov, rms_out, rms_in);
  else if (vpt <= 2) rms_norm_kernel<2><<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, inv_n, eps, wv, xv, ov, rms_out, rms_in);
  else if (vpt <= NORM_MAX_VPT) rms_norm_kernel<4><<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, inv_n, eps, wv, xv, ov, rms_out, rms_in);
  else rms_norm_kernel<0><<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, inv_n, eps, wv, xv, ov, rms_out, rms_in);
  B200_CHECK_LAUNCH(op);
  return 0;
}

extern "C" int b200_rms_norm(int fwd_dt, int n_rows, int n_cols, float eps, const void *rms_weight, const void *X, void *out,
                             float *rms_vals, void *stream) {
  B200_BF16_ONLY("rms_norm", fwd_dt);
  return rms_norm_launch("rms_norm", n_rows, n_cols, eps, rms_weight, X, out, rms_vals, nullptr, stream);
}

extern "C" int b200_rms_norm_recompute(int fwd_dt, int n_rows, int n_cols, const void *rms_weight, const float *rms_vals,
                                       const void *X, void *out, void *stream) {
  B200_BF16_ONLY("rms_norm_recompute", fwd_dt);
  B200_REQUIRE(rms_vals != nullptr, "rms_norm_recompute: rms_vals missing");
  return rms_norm_launch("rms_norm_recompute", n_rows, n_cols, 0.0f, rms_weight, X, out, nullptr, rms_vals, stream);
}

extern "C" int b200_rms_norm_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float *fwd_rms_vals,
                                   const void *rms_weight, const void *X_inp, const void *upstream_dX, void *dX, void *X_out,
                                   void *stream) {
  (void)eps;
  B200_BF16_ONLY("rms_norm_bwd_x", fwd_dt);
  B200_BF16_ONLY("rms_norm_bwd_x", bwd_dt);
  B200_REQUIRE(n_rows >= 0 && n_cols > 0 && n_cols % 8 == 0 && n_cols <= 8 * NORM_THREADS * NORM_MAX_VPT,
               "rms_norm_bwd_x: n_cols must be a multiple of 8, at most %d (got %d)", 8 * NORM_THREADS * NORM_MAX_VPT, n_cols);
  B200_REQUIRE(fwd_rms_vals && rms_weight && X_inp && upstream_dX && dX, "rms_norm_bwd_x: null argument");
  B200_REQUIRE(b200_aligned16(rms_weight) && b200_aligned16(X_inp) && b200_aligned16(upstream_dX) && b200_aligned16(dX) &&
                   b200_aligned16(X_out),
               "rms_norm_bwd_x: tensors must be 16-byte aligned");
  if (n_rows == 0) return 0;
  const int n_vec = n_cols / 8;
  const int vpt = (n_vec + NORM_THREADS - 1) / NORM_THREADS;
  const int grid = block_ops_grid(n_rows, 6);
  const float inv_n = 1.0f / (float)n_cols;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_BWDX(V)                                                                                                   \
  rms_norm_bwd_x_kernel<V><<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, inv_n, fwd_rms_vals, (const uint4 *)rms_weight, \
                                                         (const uint4 *)X_inp, (const uint4 *)upstream_dX, (uint4 *)dX, \
                                                         (uint4 *)X_out)
#define B200_BWDXW(V)                                                                                                         \
  rms_norm_bwd_x_warp_kernel<V><<<block_ops_grid((n_rows + NORM_WARPS - 1) / NORM_WARPS, 6), NORM_WARPS * 32, 0, s>>>(           \
      n_rows, n_vec, inv_n, fwd_rms_vals, (const uint4 *)rms_weight, (const uint4 *)X_inp, (const uint4 *)upstream_dX, (uint4 *)dX, \
      (uint4 *)X_out)
  if (n_vec <= 32 * 2) B200_BWDXW(2);
  else if (n_vec <= 32 * 4) B200_BWDXW(4);
  else if (n_vec <= 32 * 8) B200_BWDXW(8);
  else if (vpt <= 1) B200_BWDX(1);
  else if (vpt <= 2) B200_BWDX(2);
  else B200_BWDX(4);
#undef B200_BWDXW
#undef B200_BWDX
  B200_CHECK_LAUNCH("rms_norm_bwd_x");
  return 0;
}

// row slices of the first pass: four per SM, no more than the rows, no more than the workspace holds
static int bwd_w_slices(int n_rows, int n_cols, uint64_t workspace_bytes) {
  int slices = block_ops_grid(n_rows, 4);
  const uint64_t fit = workspace_bytes / ((uint64_t)n_cols * sizeof(float));
  if ((uint64_t)slices > fit) slices = (int)fit;
  return slices;
}

extern "C" uint64_t b200_rms_norm_bwd_w_workspace_bytes(int n_rows, int n_cols) {
  if (n_rows <= 0 || n_cols <= 0) return 0;
  return (uint64_t)block_ops_grid(n_rows, 4) * (uint64_t)n_cols * sizeof(float);
}

extern "C" int b200_rms_norm_bwd_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float *fwd_rms_vals,
                                   const void *X_inp, const void *upstream_dX, void *dW, uint64_t workspace_bytes,
                                   void *workspace, void *stream) {
  (void)eps;
  B200_BF16_ONLY("rms_norm_bwd_w", fwd_dt);
  B200_BF16_ONLY("rms_norm_bwd_w", bwd_dt);
  B200_REQUIRE(n_rows >= 0 && n_cols > 0 && n_cols % 8 == 0, "rms_norm_bwd_w: n_cols must be a positive multiple of 8");
  B200_REQUIRE(fwd_rms_vals && X_inp && upstream_dX && dW && b200_aligned16(X_inp) && b200_aligned16(upstream_dX),
               "rms_norm_bwd_w: null or unaligned argument");
  if (n_rows == 0) return 0;
  const int slices = bwd_w_slices(n_rows, n_cols, workspace_bytes);
  B200_REQUIRE(workspace != nullptr && b200_aligned16(workspace) && slices >= 1,
               "rms_norm_bwd_w: the workspace must hold at least one fp32 row of n_cols (%llu bytes given)",
               (unsigned long long)workspace_bytes);
  const int n_vec = n_cols / 8;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((n_vec + NORM_THREADS - 1) / NORM_THREADS, slices);
  rms_norm_bwd_w_partial_kernel<<<grid, NORM_THREADS, 0, s>>>(n_rows, n_vec, fwd_rms_vals, (const uint4 *)X_inp,
                                                             (const uint4 *)upstream_dX, (float *)workspace);
  B200_CHECK_LAUNCH("rms_norm_bwd_w");
  rms_norm_bwd_w_combine_kernel<<<(n_cols + 31) / 32, 256, 0, s>>>(n_cols, slices, (const float *)workspace,
                                                                    (__nv_bfloat16 *)dW);
  B200_CHECK_LAUNCH("rms_norm_bwd_w (combine)");
  return 0;
}

static int rope_launch(const char *op, int dt, int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta,
                       const int *seq_positions, void *X_q, void *X_k, float sign, void *stream) {
  B200_BF16_ONLY(op, dt);
  B200_REQUIRE(num_tokens >= 0 && head_dim >= 8 && head_dim % 8 == 0 && head_dim <= ROPE_MAX_HEAD_DIM && model_dim > 0 &&
                   model_dim % head_dim == 0 && num_kv_heads >= 0,
               "%s: head_dim must be a multiple of 8 up to %d and divide model_dim (model_dim %d, head_dim %d)", op,
               ROPE_MAX_HEAD_DIM, model_dim, head_dim);
  B200_REQUIRE(seq_positions && X_q && b200_aligned16(X_q) && b200_aligned16(X_k), "%s: null or unaligned argument", op);
  if (num_tokens == 0) return 0;
  const int q_vec = model_dim / 8, k_vec = num_kv_heads * head_dim / 8;
  const int lanes_vectors = (q_vec + 31) / 32 + (X_k ? (k_vec + 31) / 32 : 0);
  if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && lanes_vectors <= ROPE_MAX_VPL)
    rope_warp_kernel<<<block_ops_grid((num_tokens + ROPE_WARPS - 1) / ROPE_WARPS, 16), ROPE_WARPS * 32, 0, (cudaStream_t)stream>>>(
        num_tokens, q_vec, k_vec, head_dim, (float)theta, sign, seq_positions, (uint4 *)X_q, (uint4 *)X_k);
  else
    rope_kernel<<<block_ops_grid(num_tokens, 16), ROPE_THREADS, 0, (cudaStream_t)stream>>>(
        num_tokens, q_vec, k_vec, head_dim, (float)theta, sign, seq_positions, (uint4 *)X_q, (uint4 *)X_k);
  B200_CHECK_LAUNCH(op);
  return 0;
}

extern "C" int b200_rope(int fwd_dt, int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta,
                         const int *seq_positions, void *X_q, void *X_k, void *stream) {
  return rope_launch("rope", fwd_dt, num_tokens, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k, 1.0f, stream);
}

extern "C" int b200_rope_bwd_x(int bwd_dt, int num_tokens, int model_dim, int head_dim, int num_kv_heads, int theta,
                               const int *seq_positions, void *dX_q, void *dX_k, void *stream) {
  return rope_launch("rope_bwd_x", bwd_dt, num_tokens, model_dim, head_dim, num_kv_heads, theta, seq_positions, dX_q, dX_k, -1.0f,
                     stream);
}

extern "C" int b200_softmax(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void *X, void *out, void *stream) {
  B200_BF16_ONLY("softmax", fwd_dt);
  B200_BF16_ONLY("softmax", bwd_dt);
  B200_REQUIRE(n_rows >= 0 && n_cols > 0 && X && out, "softmax: bad arguments");
  if (n_rows == 0) return 0;
  softmax_kernel<<<block_ops_grid(n_rows, 1), SOFTMAX_THREADS, 0, (cudaStream_t)stream>>>(
      n_rows, n_cols, (const __nv_bfloat16 *)X, (__nv_bfloat16 *)out);
  B200_CHECK_LAUNCH("softmax");
  return 0;
}

extern "C" int b200_cross_entropy_loss(int bwd_dt, int n_rows, int n_cols, void *pred_logits, const uint32_t *labels,
                                       float *loss_vec, void *stream) {
  B200_BF16_ONLY("cross_entropy_loss", bwd_dt);
  B200_REQUIRE(n_rows >= 0 && n_cols > 0 && pred_logits && labels && loss_vec, "cross_entropy_loss: bad arguments");
  if (n_rows == 0) return 0;
  cross_entropy_kernel<<<(n_rows + 255) / 256, 256, 0, (cudaStream_t)stream>>>(n_rows, n_cols, (__nv_bfloat16 *)pred_logits,
                                                                               labels, loss_vec);
  B200_CHECK_LAUNCH("cross_entropy_loss");
  return 0;
}

extern "C" int b200_set_average_loss(int n_tokens, float *loss_vec, void *stream) {
  B200_REQUIRE(n_tokens > 0 && loss_vec, "set_average_loss: bad arguments");
  average_loss_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(n_tokens, loss_vec);
  B200_CHECK_LAUNCH("set_average_loss");
  return 0;
}

extern "C" int b200_adamw_step(int param_dt, int grad_dt, int mean_dt, int var_dt, uint64_t num_els, int step_num, float lr,
                               float beta1, float beta2, float weight_decay, float epsilon, void *param, const void *grad,
                               void *mean, void *var, void *stream) {
  B200_BF16_ONLY("adamw_step", param_dt);
  B200_BF16_ONLY("adamw_step", grad_dt);
  B200_BF16_ONLY("adamw_step", mean_dt);
  B200_BF16_ONLY("adamw_step", var_dt);
  B200_REQUIRE(step_num >= 1, "adamw_step: step_num counts from 1 (got %d)", step_num);
  B200_REQUIRE(param && grad && mean && var && b200_aligned16(param) && b200_aligned16(grad) && b200_aligned16(mean) &&
                   b200_aligned16(var),
               "adamw_step: null or unaligned argument");
  if (num_els == 0) return 0;
  const float c1 = (float)(1.0 / (1.0 - pow((double)beta1, (double)step_num))),
              c2 = (float)(1.0 / (1.0 - pow((double)beta2, (double)step_num)));
  const uint64_t n_vec = num_els / 8;
  adamw_kernel<<<block_ops_grid((int64_t)((n_vec + 255) / 256), 8), 256, 0, (cudaStream_t)stream>>>(
      num_els, lr, beta1, beta2, weight_decay, epsilon, c1, c2, (__nv_bfloat16 *)param, (const __nv_bfloat16 *)grad,
      (__nv_bfloat16 *)mean, (__nv_bfloat16 *)var);
  B200_CHECK_LAUNCH("adamw_step");
  return 0;
}

static int embedding_check(const char *op, int dt, int num_unique_tokens, int embed_dim, const void *a, const void *b,
                           const void *c, const void *d, const void *e) {
  B200_BF16_ONLY(op, dt);
  B200_REQUIRE(num_unique_tokens >= 0 && embed_dim > 0 && embed_dim % 8 == 0, "%s: embed_dim must be a positive multiple of 8", op);
  B200_REQUIRE(a && b && c && d && e && b200_aligned16(d) && b200_aligned16(e), "%s: null or unaligned argument", op);
  return 0;
}

extern "C" int b200_embedding_table(int fwd_dt, int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                                    const uint32_t *sorted_token_mapping, const uint32_t *unique_token_sorted_inds_start,
                                    const void *embedding_table, void *output, void *stream) {
  if (embedding_check("embedding_table", fwd_dt, num_unique_tokens, embed_dim, sorted_token_ids, sorted_token_mapping,
                      unique_token_sorted_inds_start, embedding_table, output))
    return -1;
  if (num_unique_tokens == 0) return 0;
  const int dim_vec = embed_dim / 8;
  const uint4 *tab = (const uint4 *)embedding_table;
  uint4 *outv = (uint4 *)output;
  cudaStream_t s = (cudaStream_t)stream;
  const int wgrid = block_ops_grid((num_unique_tokens + EMB_WARPS - 1) / EMB_WARPS, 8);
#define B200_EMB(V)                                                                                              \
  embedding_warp_kernel<V><<<wgrid, EMB_WARPS * 32, 0, s>>>(num_unique_tokens, dim_vec, sorted_token_ids, sorted_token_mapping, \
                                                           unique_token_sorted_inds_start, tab, outv)
  if (dim_vec <= 64) B200_EMB(2);
  else if (dim_vec <= 128) B200_EMB(4);
  else if (dim_vec <= 256) B200_EMB(8);
  else
    embedding_kernel<<<block_ops_grid(num_unique_tokens, 8), 256, 0, s>>>(num_unique_tokens, dim_vec, sorted_token_ids,
                                                                          sorted_token_mapping,
                                                                          unique_token_sorted_inds_start, tab, outv);
#undef B200_EMB
  B200_CHECK_LAUNCH("embedding_table");
  return 0;
}

extern "C" int b200_embedding_table_bwd_w(int bwd_dt, int num_unique_tokens, int embed_dim, const uint32_t *sorted_token_ids,
                                          const uint32_t *sorted_token_mapping,
                                          const uint32_t *unique_token_sorted_inds_start, const void *grad_stream,
                                          void *grad_embedding_table, void *stream) {
  if (embedding_check("embedding_table_bwd_w", bwd_dt, num_unique_tokens, embed_dim, sorted_token_ids, sorted_token_mapping,
                      unique_token_sorted_inds_start, grad_stream, grad_embedding_table))
    return -1;
  if (num_unique_tokens == 0) return 0;
  const int dim_vec = embed_dim / 8;
  const uint4 *gs = (const uint4 *)grad_stream;
  uint4 *gt = (uint4 *)grad_embedding_table;
  cudaStream_t s = (cudaStream_t)stream;
  const int wgrid = block_ops_grid((num_unique_tokens + EMB_WARPS - 1) / EMB_WARPS, 8);
#define B200_EMBW(V)                                                                                                   \
  embedding_bwd_w_warp_kernel<V><<<wgrid, EMB_WARPS * 32, 0, s>>>(num_unique_tokens, dim_vec, sorted_token_ids,            \
                                                                 sorted_token_mapping, unique_token_sorted_inds_start, gs, gt)
  if (dim_vec <= 64) B200_EMBW(2);
  else if (dim_vec <= 128) B200_EMBW(4);
  else if (dim_vec <= 256) B200_EMBW(8);
  else
    embedding_bwd_w_kernel<<<block_ops_grid(num_unique_tokens, 8), 256, 0, s>>>(
        num_unique_tokens, dim_vec, sorted_token_ids, sorted_token_mapping, unique_token_sorted_inds_start, gs, gt);
#undef B200_EMBW
  B200_CHECK_LAUNCH("embedding_table_bwd_w");
  return 0;
}
