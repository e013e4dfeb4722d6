// Conformer convolution module core on packed rows: GLU -> depthwise conv along time -> BatchNorm (statistics over the
// valid frames) -> SiLU, forward and backward.
//
// x [N, 2C] bf16 (output of the first pointwise GEMM), packed rows of B sequences (row_batch / row_pos / lens give the
// sequence, position and length of each row). Depthwise filter [C, K] taps, "same" padding with (K-1)/2 taps to the
// left, zero outside each sequence.
//
//   forward   glu_dwconv_fwd : h = a * sigmoid(g); y[r,c] = bias[c] + sum_k f[c,k] * h[r+k-left, c]; per-CTA partial sums
//                              of y and y^2 per channel (scratch)
//             bn_stats       : partials -> mean, rstd (and running statistics)
//             bn_silu_fwd    : z = silu((y - mean) * rstd * gamma + beta)
//   backward  bn_silu_bwd_a  : ds = dz * silu'(s); per-CTA partial sums of ds and ds * yhat
//             bn_bwd_reduce  : partials -> dgamma, dbeta (and the two means used below)
//             bn_silu_bwd_b  : dy = gamma * rstd * (ds - mean(ds) - yhat * mean(ds * yhat))
//             glu_dwconv_bwd : dh[r,c] = sum_k f[c,k] * dy[r-k+left, c]; dx = (dh * sigmoid(g), dh * a * sigmoid'(g));
//                              per-CTA partial sums for dfilter [C,K] and dbias
// All reductions go through per-CTA partials and a second pass: no atomics, deterministic.
#include "common.cuh"

namespace {

constexpr int TT = 32;       // output rows per CTA
constexpr int CC = 64;       // channels per CTA
constexpr int KMAX = 64;     // maximum number of taps
constexpr int kThreads = 256;  // 64 channels x 4 row groups of 8 rows

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
glu_dwconv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ filt, const float* __restrict__ bias,
                      const int* __restrict__ row_batch, const int* __restrict__ row_pos, const int* __restrict__ lens,
                      __nv_bfloat16* __restrict__ y, float* __restrict__ part, int n_rows, int C, int K) {
  __shared__ float sh[(TT + KMAX - 1) * CC];
  __shared__ float red[2][4][CC];
  const int left = (K - 1) / 2;
  const int r0 = blockIdx.x * TT;
  const int c0 = blockIdx.y * CC;
  const int n_in = TT + K - 1;
  // stage h = a * sigmoid(g) for rows r0-left .. r0-left+n_in-1
  for (int idx = threadIdx.x; idx < n_in * CC; idx += kThreads) {
    const int s = idx / CC, c = idx % CC;
    const int r = r0 - left + s;
    float h = 0.f;
    if (r >= 0 && r < n_rows) {
      const float a = __bfloat162float(x[(size_t)r * 2 * C + c0 + c]);
      const float g = __bfloat162float(x[(size_t)r * 2 * C + C + c0 + c]);
      h = a * sigmoidf_(g);
    }
    sh[s * CC + c] = h;
  }
  __syncthreads();
  const int c = threadIdx.x % CC;
  const int rg = threadIdx.x / CC;
  float f[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) f[k] = k < K ? filt[(size_t)(c0 + c) * K + k] : 0.f;
  const float bv = bias ? bias[c0 + c] : 0.f;
  float s1 = 0.f, s2 = 0.f;
  for (int i = 0; i < TT / 4; ++i) {
    const int lr = rg * (TT / 4) + i;
    const int r = r0 + lr;
    if (r >= n_rows) break;
    const int t = row_pos[r];
    const int L = lens[row_batch[r]];
    const int k_lo = max(0, left - t);
    const int k_hi = min(K, L - t + left);
    float acc = bv;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      if (k >= k_lo && k < k_hi) acc += f[k] * sh[(lr + k) * CC + c];
    }
    const __nv_bfloat16 o = __float2bfloat16(acc);
    y[(size_t)r * C + c0 + c] = o;
    const float of = __bfloat162float(o);
    s1 += of;
    s2 += of * of;
  }
  red[0][rg][c] = s1;
  red[1][rg][c] = s2;
  __syncthreads();
  if (threadIdx.x < CC) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      a += red[0][g][threadIdx.x];
      b += red[1][g][threadIdx.x];
    }
    part[((size_t)blockIdx.x * 2 + 0) * C + c0 + threadIdx.x] = a;
    part[((size_t)blockIdx.x * 2 + 1) * C + c0 + threadIdx.x] = b;
  }
}

__global__ void __launch_bounds__(256)
bn_silu_fwd_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                   const float* __restrict__ gamma, const float* __restrict__ beta, __nv_bfloat16* __restrict__ z, long long total, int C) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const long long i8 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= total) return;
  const int c = (int)(i8 % C);
  F8 v = load8(y, i8, 1);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float s = (v.v[k] - mean[c + k]) * rstd[c + k] * (gamma ? gamma[c + k] : 1.f) + (beta ? beta[c + k] : 0.f);
    v.v[k] = s * sigmoidf_(s);
  }
  store8(z, i8, v, 1);
}

// ---------------------------------------------------------------------------------------------------------------------
// ds = dz * silu'(s) written to ds_out (bf16); per-CTA partials of sum(ds) and sum(ds*yhat) per channel.
// grid.x tiles of 64 rows; block 256 = 64 channel-octets?  -> layout: thread handles 8 channels of one row at a time.
__global__ void __launch_bounds__(256)
bn_silu_bwd_a_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dz, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const float* __restrict__ gamma, const float* __restrict__ beta,
                     __nv_bfloat16* __restrict__ ds_out, float* __restrict__ part, int n_rows, int C, int rows_per_cta) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  // threads: C/8 column groups x (256 / (C/8)) row lanes; requires C/8 <= 256 and 256 % (C/8) == 0
  extern __shared__ float shm[];  // [row_lanes][2][C]
  const int groups = C / 8;
  const int row_lanes = blockDim.x / groups;
  const int cg = threadIdx.x % groups;
  const int rl = threadIdx.x / groups;
  const int c = cg * 8;
  float a1[8], a2[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a1[k] = a2[k] = 0.f;
  const int r_begin = blockIdx.x * rows_per_cta;
  const int r_end = min(n_rows, r_begin + rows_per_cta);
  if (rl < row_lanes) {
    // per-channel constants once; then four rows per step with all of their loads issued before the first use (a thread owns few
    // rows: their load latency is the cost of this kernel)
    float mu[8], rs[8], ga[8], be[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      mu[k] = mean[c + k];
      rs[k] = rstd[c + k];
      ga[k] = gamma ? gamma[c + k] : 1.f;
      be[k] = beta ? beta[c + k] : 0.f;
    }
    for (int r0 = r_begin + rl; r0 < r_end; r0 += 4 * row_lanes) {
      F8 yv[4], dv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = r0 + j * row_lanes;
        if (r < r_end) {
          yv[j] = load8(y, (long long)r * C + c, 1);
          dv[j] = load8(dz, (long long)r * C + c, 1);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = r0 + j * row_lanes;
        if (r < r_end) {
          F8 o;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float yh = (yv[j].v[k] - mu[k]) * rs[k];
            const float s = yh * ga[k] + be[k];
            const float sg = sigmoidf_(s);
            const float d = dv[j].v[k] * (sg * (1.f + s * (1.f - sg)));
            o.v[k] = d;
            a1[k] += d;
            a2[k] += d * yh;
          }
          store8(ds_out, (long long)r * C + c, o, 1);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      shm[(rl * 2 + 0) * C + c + k] = a1[k];
      shm[(rl * 2 + 1) * C + c + k] = a2[k];
    }
  }
  __syncthreads();
  for (int cc = threadIdx.x; cc < C; cc += blockDim.x) {
    float s1 = 0.f, s2 = 0.f;
    for (int l = 0; l < row_lanes; ++l) {
      s1 += shm[(l * 2 + 0) * C + cc];
      s2 += shm[(l * 2 + 1) * C + cc];
    }
    part[((size_t)blockIdx.x * 2 + 0) * C + cc] = s1;
    part[((size_t)blockIdx.x * 2 + 1) * C + cc] = s2;
  }
}

// dy = gamma * rstd * (ds - sum_ds/count - yhat * sum_ds_yh/count), in place over ds
__global__ void __launch_bounds__(256)
bn_silu_bwd_b_kernel(const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ ds, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const float* __restrict__ gamma, const float* __restrict__ sum_ds,
                     const float* __restrict__ sum_ds_yh, float inv_count, long long total, int C) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const long long i8 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= total) return;
  const int c = (int)(i8 % C);
  F8 yv = load8(y, i8, 1);
  F8 dv = load8(ds, i8, 1);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float yh = (yv.v[k] - mean[c + k]) * rstd[c + k];
    dv.v[k] = (gamma ? gamma[c + k] : 1.f) * rstd[c + k] * (dv.v[k] - sum_ds[c + k] * inv_count - yh * sum_ds_yh[c + k] * inv_count);
  }
  store8(ds, i8, dv, 1);
}

// depthwise conv backward + GLU backward. Each CTA owns CC channels and walks over row tiles (tile = blockIdx.x, += gridDim.x),
// keeping its dfilter / dbias sums in registers; one partial per CTA at the end: part layout [gridDim.x][C][K+1].
template <int KM>
__global__ void __launch_bounds__(kThreads)
glu_dwconv_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ filt,
                      const int* __restrict__ row_batch, const int* __restrict__ row_pos, const int* __restrict__ lens,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ part, int n_rows, int C, int K) {
  __shared__ float sh_dy[(TT + KM - 1) * CC];   // dy rows r0-(K-1-left) .. : used for dh
  __shared__ float sh_h[(TT + KM - 1) * CC];    // h rows r0-left .. : used for dfilter
  __shared__ int sh_t[TT], sh_len[TT];
  const int left = (K - 1) / 2;
  const int right = K - 1 - left;
  const int c0 = blockIdx.y * CC;
  const int n_in = TT + K - 1;
  const int n_tiles = (n_rows + TT - 1) / TT;
  const int c = threadIdx.x % CC;
  const int rg = threadIdx.x / CC;
  float f[KM];
#pragma unroll
  for (int k = 0; k < KM; ++k) f[k] = k < K ? filt[(size_t)(c0 + c) * K + k] : 0.f;
  float df[KM];
#pragma unroll
  for (int k = 0; k < KM; ++k) df[k] = 0.f;
  float dbias = 0.f;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int r0 = tile * TT;
    __syncthreads();  // the previous tile's readers are done with the shared arrays
    // stage dy and h = a * sigmoid(g), 8 channels per thread-iteration
    for (int idx = threadIdx.x; idx < n_in * (CC / 8); idx += kThreads) {
      const int s = idx / (CC / 8), cg = (idx % (CC / 8)) * 8;
      // dh[r] = sum_k f[k] * dy[r - k + left]  ->  needs dy rows r0 - right .. r0 + TT - 1 + left
      const int rd = r0 - right + s;
      F8 d;
      if (rd >= 0 && rd < n_rows) d = load8(dy, (int64_t)rd * C + c0 + cg, 1);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) d.v[i] = 0.f;
      }
      const int rh = r0 - left + s;
      F8 h;
      if (rh >= 0 && rh < n_rows) {
        F8 a = load8(x, (int64_t)rh * 2 * C + c0 + cg, 1);
        F8 g = load8(x, (int64_t)rh * 2 * C + C + c0 + cg, 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) h.v[i] = a.v[i] * sigmoidf_(g.v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) h.v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sh_dy[s * CC + cg + i] = d.v[i];
        sh_h[s * CC + cg + i] = h.v[i];
      }
    }
    if (threadIdx.x < TT) {
      const int r = r0 + threadIdx.x;
      sh_t[threadIdx.x] = r < n_rows ? row_pos[r] : 0;
      sh_len[threadIdx.x] = r < n_rows ? lens[row_batch[r]] : 0;
    }
    __syncthreads();
    for (int i = 0; i < TT / 4; ++i) {
      const int lr = rg * (TT / 4) + i;
      const int r = r0 + lr;
      if (r >= n_rows) break;
      const int t = sh_t[lr];
      const int L = sh_len[lr];
      // dh: contributions from output rows r' = r - k + left (position t - k + left) that lie inside the sequence
      float dh = 0.f;
#pragma unroll
      for (int k = 0; k < KM; ++k) {
        const int tp = t - k + left;
        if (k < K && tp >= 0 && tp < L) dh += f[k] * sh_dy[(lr + right - k + left) * CC + c];
      }
      // a and g of this row: h = a * sig(g) is staged at row lr + left; recover a, g from global (coalesced over c)
      const float a = __bfloat162float(x[(size_t)r * 2 * C + c0 + c]);
      const float g = __bfloat162float(x[(size_t)r * 2 * C + C + c0 + c]);
      const float sg = sigmoidf_(g);
      dx[(size_t)r * 2 * C + c0 + c] = __float2bfloat16(dh * sg);
      dx[(size_t)r * 2 * C + C + c0 + c] = __float2bfloat16(dh * a * sg * (1.f - sg));
      // dfilter[k] += dy[r] * h[r + k - left] for taps inside the sequence
      const float dyr = sh_dy[(lr + right) * CC + c];
      dbias += dyr;
      const int k_lo = max(0, left - t);
      const int k_hi = min(K, L - t + left);
#pragma unroll
      for (int k = 0; k < KM; ++k) {
        if (k >= k_lo && k < k_hi) df[k] += dyr * sh_h[(lr + k) * CC + c];
      }
    }
  }
  // reduce the 4 row groups through shared memory (reuse sh_h as [K+1][CC] accumulators), then one partial per CTA
  __syncthreads();
  float* red = sh_h;
  for (int g = 0; g < 4; ++g) {
    if (rg == g) {
#pragma unroll
      for (int k = 0; k < KM; ++k)
        if (k < K) red[k * CC + c] = (g == 0 ? 0.f : red[k * CC + c]) + df[k];
      red[K * CC + c] = (g == 0 ? 0.f : red[K * CC + c]) + dbias;
    }
    __syncthreads();
  }
  for (int idx = threadIdx.x; idx < (K + 1) * CC; idx += kThreads) {
    const int k = idx / CC, cc = idx % CC;
    part[((size_t)blockIdx.x * C + c0 + cc) * (K + 1) + k] = red[k * CC + cc];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Sliding-window versions for K <= 32 taps. A thread owns one channel and RPT consecutive output rows: it walks once over
// the RPT + 31 staged rows of its window, and every staged value feeds up to RPT accumulators through compile-time filter
// indices, so the filter and the accumulators stay in registers and each staged value is read from shared memory once
// (the kernels above read one value per tap and output). Rows of other sequences are masked by comparing sequence ids
// (packed rows are sorted by sequence); a window that lies inside one sequence takes the unmasked path.
constexpr int TT2 = 64;  // output rows per tile
constexpr int KM2 = 32;  // taps (filters with fewer taps are zero-padded)
constexpr int NST2 = TT2 + KM2 - 1;  // staged rows per tile
constexpr int NID2 = TT2 + KM2 + 2;  // staged sequence ids per tile

template <int RPT, bool MASKED>
__device__ __forceinline__ void window_conv(const float* __restrict__ col, const int* __restrict__ ids, const float (&w)[KM2],
                                            const int (&bo)[RPT], float (&acc)[RPT]) {
#pragma unroll
  for (int j = 0; j < RPT + KM2 - 1; ++j) {
    const float v = col[j * CC];
    const int b = MASKED ? ids[j] : 0;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      if (j - i >= 0 && j - i < KM2) {
        if (MASKED) acc[i] = (b == bo[i]) ? fmaf(w[j - i], v, acc[i]) : acc[i];
        else acc[i] = fmaf(w[j - i], v, acc[i]);
      }
    }
  }
}

template <int RPT, bool MASKED>
__device__ __forceinline__ void window_corr(const float* __restrict__ col, const int* __restrict__ ids, const float (&d)[RPT],
                                            const int (&bo)[RPT], float (&df)[KM2]) {
#pragma unroll
  for (int j = 0; j < RPT + KM2 - 1; ++j) {
    const float v = col[j * CC];
    const int b = MASKED ? ids[j] : 0;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      if (j - i >= 0 && j - i < KM2) {
        if (MASKED) df[j - i] = (b == bo[i]) ? fmaf(d[i], v, df[j - i]) : df[j - i];
        else df[j - i] = fmaf(d[i], v, df[j - i]);
      }
    }
  }
}

// sequence id of rows first .. first + n - 1 (a distinct negative number for rows outside the buffer: equal to nothing)
__device__ __forceinline__ void stage_ids(int* __restrict__ ids, const int* __restrict__ row_batch, int first, int n, int n_rows) {
  for (int s = threadIdx.x; s < n; s += blockDim.x) {
    const int r = first + s;
    ids[s] = (r >= 0 && r < n_rows) ? row_batch[r] : -1 - s;
  }
}

constexpr int kFwd2Threads = 256;  // 64 channels x 4 row groups of 16 rows
constexpr int kFwd2Rpt = 16;

__global__ void __launch_bounds__(kFwd2Threads, 2)
glu_dwconv_fwd2_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ filt, const float* __restrict__ bias,
                       const int* __restrict__ row_batch, __nv_bfloat16* __restrict__ y, float* __restrict__ part, int n_rows, int C, int K) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  __shared__ float sh[NST2 * CC];
  __shared__ int ids[NID2];
  __shared__ float red[2][4][CC];
  const int left = (K - 1) / 2;
  const int r0 = blockIdx.x * TT2;
  const int c0 = blockIdx.y * CC;
  for (int idx = threadIdx.x; idx < NST2 * (CC / 8); idx += kFwd2Threads) {
    const int s = idx / (CC / 8), cg = (idx % (CC / 8)) * 8;
    const int r = r0 - left + s;
    F8 h;
    if (r >= 0 && r < n_rows) {
      const F8 a = load8(x, (int64_t)r * 2 * C + c0 + cg, 1);
      const F8 g = load8(x, (int64_t)r * 2 * C + C + c0 + cg, 1);
#pragma unroll
      for (int i = 0; i < 8; ++i) h.v[i] = a.v[i] * sigmoidf_(g.v[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) h.v[i] = 0.f;
    }
    float4* dst = reinterpret_cast<float4*>(sh + s * CC + cg);
    dst[0] = make_float4(h.v[0], h.v[1], h.v[2], h.v[3]);
    dst[1] = make_float4(h.v[4], h.v[5], h.v[6], h.v[7]);
  }
  stage_ids(ids, row_batch, r0 - left, NST2, n_rows);
  __syncthreads();
  const int c = threadIdx.x % CC;
  const int rg = threadIdx.x / CC;
  const int base = rg * kFwd2Rpt;
  float f[KM2];
#pragma unroll
  for (int k = 0; k < KM2; ++k) f[k] = k < K ? filt[(size_t)(c0 + c) * K + k] : 0.f;
  const float bv = bias ? bias[c0 + c] : 0.f;
  float acc[kFwd2Rpt];
  int bo[kFwd2Rpt];
#pragma unroll
  for (int i = 0; i < kFwd2Rpt; ++i) {
    acc[i] = bv;
    bo[i] = ids[base + i + left];
  }
  const int id_first = ids[base], id_last = ids[base + kFwd2Rpt + KM2 - 2];
  if (id_first >= 0 && id_first == id_last) window_conv<kFwd2Rpt, false>(sh + base * CC + c, ids + base, f, bo, acc);
  else window_conv<kFwd2Rpt, true>(sh + base * CC + c, ids + base, f, bo, acc);
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < kFwd2Rpt; ++i) {
    const int r = r0 + base + i;
    if (r < n_rows) {
      const __nv_bfloat16 o = __float2bfloat16(acc[i]);
      y[(size_t)r * C + c0 + c] = o;
      const float of = __bfloat162float(o);
      s1 += of;
      s2 += of * of;
    }
  }
  red[0][rg][c] = s1;
  red[1][rg][c] = s2;
  __syncthreads();
  if (threadIdx.x < CC) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      a += red[0][g][threadIdx.x];
      b += red[1][g][threadIdx.x];
    }
    // the partial layout has one slot per 32 rows: this CTA fills two of them
    const int slot = blockIdx.x * (TT2 / TT);
    const int n_slots = (n_rows + TT - 1) / TT;
    part[((size_t)slot * 2 + 0) * C + c0 + threadIdx.x] = a;
    part[((size_t)slot * 2 + 1) * C + c0 + threadIdx.x] = b;
    if (slot + 1 < n_slots) {
      part[((size_t)(slot + 1) * 2 + 0) * C + c0 + threadIdx.x] = 0.f;
      part[((size_t)(slot + 1) * 2 + 1) * C + c0 + threadIdx.x] = 0.f;
    }
  }
}

constexpr int kBwd2Threads = 512;  // 64 channels x 8 row groups of 8 rows
constexpr int kBwd2Rpt = 8;
constexpr size_t kBwd2Smem = (size_t)2 * NST2 * CC * sizeof(float) + NID2 * sizeof(int);

// persistent over row tiles (tile = blockIdx.x, += gridDim.x); dfilter / dbias sums stay in registers; partial per CTA
// [gridDim.x][C][K+1]
__global__ void __launch_bounds__(kBwd2Threads, 1)
glu_dwconv_bwd2_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ filt,
                       const int* __restrict__ row_batch, __nv_bfloat16* __restrict__ dx, float* __restrict__ part, int n_rows, int C, int K) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  extern __shared__ __align__(16) unsigned char smem2[];
  float* sh_dy = reinterpret_cast<float*>(smem2);  // rows r0 - right ..
  float* sh_h = sh_dy + NST2 * CC;                 // rows r0 - left ..
  int* ids = reinterpret_cast<int*>(sh_h + NST2 * CC);  // rows r0 - right ..
  const int left = (K - 1) / 2;
  const int right = K - 1 - left;
  const int c0 = blockIdx.y * CC;
  const int n_tiles = (n_rows + TT2 - 1) / TT2;
  const int c = threadIdx.x % CC;
  const int rg = threadIdx.x / CC;
  const int base = rg * kBwd2Rpt;
  float fr[KM2];  // flipped filter: fr[m] = f[K-1-m]
#pragma unroll
  for (int m = 0; m < KM2; ++m) fr[m] = m < K ? filt[(size_t)(c0 + c) * K + (K - 1 - m)] : 0.f;
  float df[KM2];
#pragma unroll
  for (int k = 0; k < KM2; ++k) df[k] = 0.f;
  float dbias = 0.f;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int r0 = tile * TT2;
    __syncthreads();
    for (int idx = threadIdx.x; idx < NST2 * (CC / 8); idx += kBwd2Threads) {
      const int s = idx / (CC / 8), cg = (idx % (CC / 8)) * 8;
      const int rd = r0 - right + s;
      F8 d;
      if (rd >= 0 && rd < n_rows) d = load8(dy, (int64_t)rd * C + c0 + cg, 1);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) d.v[i] = 0.f;
      }
      const int rh = r0 - left + s;
      F8 h;
      if (rh >= 0 && rh < n_rows) {
        const F8 a = load8(x, (int64_t)rh * 2 * C + c0 + cg, 1);
        const F8 g = load8(x, (int64_t)rh * 2 * C + C + c0 + cg, 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) h.v[i] = a.v[i] * sigmoidf_(g.v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) h.v[i] = 0.f;
      }
      float4* pd = reinterpret_cast<float4*>(sh_dy + s * CC + cg);
      pd[0] = make_float4(d.v[0], d.v[1], d.v[2], d.v[3]);
      pd[1] = make_float4(d.v[4], d.v[5], d.v[6], d.v[7]);
      float4* ph = reinterpret_cast<float4*>(sh_h + s * CC + cg);
      ph[0] = make_float4(h.v[0], h.v[1], h.v[2], h.v[3]);
      ph[1] = make_float4(h.v[4], h.v[5], h.v[6], h.v[7]);
    }
    stage_ids(ids, row_batch, r0 - right, NID2, n_rows);
    __syncthreads();
    int bo[kBwd2Rpt];
#pragma unroll
    for (int i = 0; i < kBwd2Rpt; ++i) bo[i] = ids[base + i + right];
    // one test covers both windows: rows r0+base-right .. r0+base+RPT-1+left+1 (the id array has two spare entries)
    const int id_first = ids[base], id_last = ids[base + kBwd2Rpt + KM2 - 1];
    const bool inside = id_first >= 0 && id_first == id_last;
    {
      // dh[r] = sum_k f[k] * dy[r - k + left]: staged index of that row is (r - r0) + (K-1) - k
      float acc[kBwd2Rpt];
#pragma unroll
      for (int i = 0; i < kBwd2Rpt; ++i) acc[i] = 0.f;
      if (inside) window_conv<kBwd2Rpt, false>(sh_dy + base * CC + c, ids + base, fr, bo, acc);
      else window_conv<kBwd2Rpt, true>(sh_dy + base * CC + c, ids + base, fr, bo, acc);
#pragma unroll
      for (int i = 0; i < kBwd2Rpt; ++i) {
        const int r = r0 + base + i;
        if (r < n_rows) {
          const float a = __bfloat162float(x[(size_t)r * 2 * C + c0 + c]);
          const float g = __bfloat162float(x[(size_t)r * 2 * C + C + c0 + c]);
          const float sg = sigmoidf_(g);
          dx[(size_t)r * 2 * C + c0 + c] = __float2bfloat16(acc[i] * sg);
          dx[(size_t)r * 2 * C + C + c0 + c] = __float2bfloat16(acc[i] * a * sg * (1.f - sg));
        }
      }
    }
    {
      // dfilter[k] += dy[r] * h[r + k - left]: staged index of that h row is (r - r0) + k; its id sits at + right - left
      float d[kBwd2Rpt];
#pragma unroll
      for (int i = 0; i < kBwd2Rpt; ++i) {
        d[i] = sh_dy[(base + i + right) * CC + c];
        dbias += d[i];
      }
      if (inside) window_corr<kBwd2Rpt, false>(sh_h + base * CC + c, ids + base + right - left, d, bo, df);
      else window_corr<kBwd2Rpt, true>(sh_h + base * CC + c, ids + base + right - left, d, bo, df);
    }
  }
  // sum the 8 row groups in shared memory, one partial per CTA
  __syncthreads();
  float* red = sh_h;  // [KM2 + 1][CC]
  for (int idx = threadIdx.x; idx < (KM2 + 1) * CC; idx += kBwd2Threads) red[idx] = 0.f;
  __syncthreads();
#pragma unroll
  for (int k = 0; k < KM2; ++k) atomicAdd(&red[k * CC + c], df[k]);
  atomicAdd(&red[KM2 * CC + c], dbias);
  __syncthreads();
  for (int idx = threadIdx.x; idx < (K + 1) * CC; idx += kBwd2Threads) {
    const int cc = idx / (K + 1), k = idx % (K + 1);
    part[((size_t)blockIdx.x * C + c0 + cc) * (K + 1) + k] = red[(k < K ? k : KM2) * CC + cc];
  }
}

// Reductions of per-CTA partials with 8 tile lanes per output and a shared-memory sum (coalesced over the outputs; the
// one-thread-per-output loops above take tens of microseconds for a few hundred tiles).
__device__ __forceinline__ float lane_sum8(float s, float (*sh)[32], int tl, int lane) {
  sh[tl][lane] = s;
  __syncthreads();
  if (tl == 0) {
#pragma unroll
    for (int g = 1; g < 8; ++g) s += sh[g][lane];
  }
  __syncthreads();
  return s;
}

// part [n_tiles][C][K+1] -> dfilt [C][K], dbias [C]
__global__ void __launch_bounds__(256)
dwconv_bwd_reduce2_kernel(const float* __restrict__ part, int n_tiles, int C, int K, float* __restrict__ dfilt, float* __restrict__ dbias,
                          int accumulate) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  __shared__ float sh[8][32];
  const int lane = threadIdx.x % 32, tl = threadIdx.x / 32;
  const int idx = blockIdx.x * 32 + lane;
  const int n_out = C * (K + 1);
  float s = 0.f;
  if (idx < n_out)
    for (int t = tl; t < n_tiles; t += 8) s += part[(size_t)t * n_out + idx];
  s = lane_sum8(s, sh, tl, lane);
  if (tl == 0 && idx < n_out) {
    const int c = idx / (K + 1), k = idx % (K + 1);
    if (k < K) dfilt[(size_t)c * K + k] = accumulate ? dfilt[(size_t)c * K + k] + s : s;
    else if (dbias) dbias[c] = accumulate ? dbias[c] + s : s;
  }
}

// part [n_tiles][2][C] -> the two sums per channel (thread tl == 0 of each lane holds them)
__device__ __forceinline__ void pair_sums(const float* __restrict__ part, int n_tiles, int C, int c, float (*sh)[32], int tl, int lane,
                                          float& s1, float& s2) {
  s1 = 0.f;
  s2 = 0.f;
  if (c < C)
    for (int t = tl; t < n_tiles; t += 8) {
      s1 += part[((size_t)t * 2 + 0) * C + c];
      s2 += part[((size_t)t * 2 + 1) * C + c];
    }
  s1 = lane_sum8(s1, sh, tl, lane);
  s2 = lane_sum8(s2, sh, tl, lane);
}

__global__ void __launch_bounds__(256)
bn_stats2_kernel(const float* __restrict__ part, int n_tiles, int C, float count, float eps, float momentum, float* __restrict__ mean,
                 float* __restrict__ rstd, float* __restrict__ running_mean, float* __restrict__ running_var) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  __shared__ float sh[8][32];
  const int lane = threadIdx.x % 32, tl = threadIdx.x / 32;
  const int c = blockIdx.x * 32 + lane;
  float s1, s2;
  pair_sums(part, n_tiles, C, c, sh, tl, lane, s1, s2);
  if (tl == 0 && c < C) {
    const double m = (double)s1 / count;
    double var = (double)s2 / count - m * m;
    if (var < 0.0) var = 0.0;
    mean[c] = (float)m;
    rstd[c] = rsqrtf((float)var + eps);
    if (running_mean) {
      running_mean[c] += momentum * ((float)m - running_mean[c]);
      running_var[c] += momentum * ((float)var - running_var[c]);
    }
  }
}

__global__ void __launch_bounds__(256)
bn_bwd_reduce2_kernel(const float* __restrict__ part, int n_tiles, int C, float* __restrict__ sum_ds, float* __restrict__ sum_ds_yh,
                      float* __restrict__ dgamma_acc, float* __restrict__ dbeta_acc) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  __shared__ float sh[8][32];
  const int lane = threadIdx.x % 32, tl = threadIdx.x / 32;
  const int c = blockIdx.x * 32 + lane;
  float s1, s2;
  pair_sums(part, n_tiles, C, c, sh, tl, lane, s1, s2);
  if (tl == 0 && c < C) {
    sum_ds[c] = s1;
    sum_ds_yh[c] = s2;
    if (dgamma_acc) dgamma_acc[c] += s2;
    if (dbeta_acc) dbeta_acc[c] += s1;
  }
}

__global__ void dwconv_bwd_reduce_kernel(const float* __restrict__ part, int n_tiles, int C, int K, float* __restrict__ dfilt,
                                         float* __restrict__ dbias, int accumulate = 0) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= C * (K + 1)) return;
  const int c = idx / (K + 1), k = idx % (K + 1);
  double s = 0.0;
  for (int t = 0; t < n_tiles; ++t) s += part[((size_t)t * C + c) * (K + 1) + k];
  if (accumulate) {
    if (k < K) dfilt[(size_t)c * K + k] += (float)s;
    else if (dbias) dbias[c] += (float)s;
  } else {
    if (k < K) dfilt[(size_t)c * K + k] = (float)s;
    else if (dbias) dbias[c] = (float)s;
  }
}

}  // namespace

// scratch `part` sizes (floats): forward ceil(N/32)*2*C; backward-a n_tiles_a*2*C; backward conv ceil(N/32)*C*(K+1)
RB_EXPORT int rb200_glu_dwconv_fwd(const void* x, const float* filt, const float* bias, const int* row_batch, const int* row_pos,
                                   const int* lens, void* y, float* part, int n_rows, int C, int K, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  if (C % CC || K > KMAX || K < 1) {
    rb_set_error("glu_dwconv: C=%d must be a multiple of %d and K=%d <= %d", C, CC, K, KMAX);
    return RB_ERR_ARG;
  }
  if (K <= KM2) {
    dim3 grid((n_rows + TT2 - 1) / TT2, C / CC);
    rb_launch_pdl(glu_dwconv_fwd2_kernel, dim3(grid), dim3(kFwd2Threads), 0, stream, (const __nv_bfloat16*)x, filt, bias, row_batch, (__nv_bfloat16*)y, part, n_rows, C, K);
    return rb_check_launch("glu_dwconv_fwd2");
  }
  dim3 grid((n_rows + TT - 1) / TT, C / CC);
  glu_dwconv_fwd_kernel<<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, filt, bias, row_batch, row_pos, lens, (__nv_bfloat16*)y, part, n_rows, C, K);
  return rb_check_launch("glu_dwconv_fwd");
}

RB_EXPORT int rb200_bn_stats(const float* part, int n_tiles, int C, float count, float eps, float momentum, float* mean, float* rstd,
                             float* running_mean, float* running_var, cudaStream_t stream) {
  rb_launch_pdl(bn_stats2_kernel, dim3((C + 31) / 32), dim3(256), 0, stream, part, n_tiles, C, count, eps, momentum, mean, rstd, running_mean, running_var);
  return rb_check_launch("bn_stats");
}

RB_EXPORT int rb200_bn_silu_fwd(const void* y, const float* mean, const float* rstd, const float* gamma, const float* beta, void* z,
                                long long n_rows, int C, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  if (C % 8) return RB_ERR_ARG;
  long long total = n_rows * C;
  rb_launch_pdl(bn_silu_fwd_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)y, mean, rstd, gamma, beta, (__nv_bfloat16*)z, total, C);
  return rb_check_launch("bn_silu_fwd");
}

// ds (bf16 [N,C]) receives ds, later overwritten in place by dy. part: n_tiles*2*C floats.
// dgamma_acc / dbeta_acc (optional): the parameter gradients are also added there
RB_EXPORT int rb200_bn_silu_bwd_ex(const void* y, const void* dz, const float* mean, const float* rstd, const float* gamma, const float* beta,
                                   void* ds, float* part, int n_tiles, float* sum_ds, float* sum_ds_yh, long long n_rows, int C,
                                   int training, float* dgamma_acc, float* dbeta_acc, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  const int groups = C / 8;
  if (C % 8 || groups > 256 || 256 % groups) {
    rb_set_error("bn_silu_bwd: C=%d unsupported", C);
    return RB_ERR_ARG;
  }
  const int row_lanes = 256 / groups;
  const int rows_per_cta = (int)((n_rows + n_tiles - 1) / n_tiles);
  size_t smem = (size_t)row_lanes * 2 * C * sizeof(float);
  rb_launch_pdl(bn_silu_bwd_a_kernel, dim3(n_tiles), dim3(256), smem, stream, (const __nv_bfloat16*)y, (const __nv_bfloat16*)dz, mean, rstd, gamma, beta,
                                                       (__nv_bfloat16*)ds, part, (int)n_rows, C, rows_per_cta);
  int st = rb_check_launch("bn_silu_bwd_a");
  if (st) return st;
  rb_launch_pdl(bn_bwd_reduce2_kernel, dim3((C + 31) / 32), dim3(256), 0, stream, part, n_tiles, C, sum_ds, sum_ds_yh, dgamma_acc, dbeta_acc);
  st = rb_check_launch("bn_bwd_reduce");
  if (st) return st;
  if (training) {
    long long total = n_rows * C;
    rb_launch_pdl(bn_silu_bwd_b_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)y, (__nv_bfloat16*)ds, mean, rstd, gamma,
                                                                                 sum_ds, sum_ds_yh, 1.f / (float)n_rows, total, C);
    st = rb_check_launch("bn_silu_bwd_b");
  }
  return st;
}

RB_EXPORT int rb200_bn_silu_bwd(const void* y, const void* dz, const float* mean, const float* rstd, const float* gamma, const float* beta,
                                void* ds, float* part, int n_tiles, float* sum_ds, float* sum_ds_yh, long long n_rows, int C,
                                int training, cudaStream_t stream) {
  return rb200_bn_silu_bwd_ex(y, dz, mean, rstd, gamma, beta, ds, part, n_tiles, sum_ds, sum_ds_yh, n_rows, C, training, nullptr, nullptr, stream);
}

// accumulate: dfilt / dbias += instead of =
RB_EXPORT int rb200_glu_dwconv_bwd_ex(const void* x, const void* dy, const float* filt, const int* row_batch, const int* row_pos,
                                      const int* lens, void* dx, float* part, float* dfilt, float* dbias, int n_rows, int C, int K,
                                      int accumulate, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  if (C % CC || K > KMAX || K < 1) return RB_ERR_ARG;
  const int n_tiles = (n_rows + TT - 1) / TT;
  // about four CTAs per SM in total; every CTA leaves one partial
  int row_ctas = (4 * 148 + C / CC - 1) / (C / CC);
  if (row_ctas > n_tiles) row_ctas = n_tiles;
  dim3 grid(row_ctas, C / CC);
  if (K <= KM2) {
    static bool attr2 = false;
    if (!attr2) {
      cudaFuncSetAttribute(glu_dwconv_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBwd2Smem);
      attr2 = true;
    }
    // one 512-thread CTA per SM; every CTA leaves one partial (the scratch holds ceil(N/32) of them, more than enough)
    const int n_tiles2 = (n_rows + TT2 - 1) / TT2;
    row_ctas = 148 / (C / CC);
    if (row_ctas < 1) row_ctas = 1;
    if (row_ctas > n_tiles2) row_ctas = n_tiles2;
    grid = dim3(row_ctas, C / CC);
    rb_launch_pdl(glu_dwconv_bwd2_kernel, dim3(grid), dim3(kBwd2Threads), kBwd2Smem, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, filt, row_batch,
                                                                     (__nv_bfloat16*)dx, part, n_rows, C, K);
    int st2 = rb_check_launch("glu_dwconv_bwd2");
    if (st2) return st2;
    rb_launch_pdl(dwconv_bwd_reduce2_kernel, dim3((C * (K + 1) + 31) / 32), dim3(256), 0, stream, part, row_ctas, C, K, dfilt, dbias, accumulate);
    return rb_check_launch("dwconv_bwd_reduce2");
  } else {
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(glu_dwconv_bwd_kernel<KMAX>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
      attr = true;
    }
    glu_dwconv_bwd_kernel<KMAX><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, filt, row_batch, row_pos, lens,
                                                               (__nv_bfloat16*)dx, part, n_rows, C, K);
  }
  int st = rb_check_launch("glu_dwconv_bwd");
  if (st) return st;
  dwconv_bwd_reduce_kernel<<<(C * (K + 1) + 255) / 256, 256, 0, stream>>>(part, row_ctas, C, K, dfilt, dbias, accumulate);
  return rb_check_launch("dwconv_bwd_reduce");
}

RB_EXPORT int rb200_glu_dwconv_bwd(const void* x, const void* dy, const float* filt, const int* row_batch, const int* row_pos,
                                   const int* lens, void* dx, float* part, float* dfilt, float* dbias, int n_rows, int C, int K,
                                   cudaStream_t stream) {
  return rb200_glu_dwconv_bwd_ex(x, dy, filt, row_batch, row_pos, lens, dx, part, dfilt, dbias, n_rows, C, K, 0, stream);
}
