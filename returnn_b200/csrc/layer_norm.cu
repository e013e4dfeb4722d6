// LayerNorm / RMSNorm over the last axis.
//
// Forward: one warp per row, the row is held in registers (n <= 2048) or re-read from L2 (larger n);
// statistics in fp32; saves mean and rstd. Backward: one warp per row for dx; every CTA accumulates its
// rows' contributions to dgamma/dbeta in registers and writes one partial per CTA into scratch memory,
// which a second kernel reduces: that pair (ln_bwd_kernel + ln_bwd_reduce_kernel, also behind the allocation-free entry
// point) uses no atomics and is deterministic. The accumulating variant used by the native encoder executor
// (ln_bwd_acc_kernel) adds its per-CTA sums into dgamma/dbeta with fp32 atomics instead: no scratch and no second launch,
// but the summation order, and so the last bits of dgamma/dbeta, can differ from run to run.
#include "common.cuh"

namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kMaxChunks = 8;  // 8 chunks * 32 lanes * 8 elems = 2048 elements in registers

template <int CHUNKS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
ln_fwd_kernel(const void* __restrict__ x, const void* __restrict__ gamma, const void* __restrict__ beta,
              void* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
              int64_t rows, int n, float eps, int x_bf16, int w_bf16, int rms) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = row * (int64_t)n;
  F8 v[CHUNKS];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    int col = (c * 32 + lane) * 8;
    if (col < n) {
      v[c] = load8(x, base + col, x_bf16);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[c].v[i];
    }
  }
  float mean = rms ? 0.f : warp_sum(s) / (float)n;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    int col = (c * 32 + lane) * 8;
    if (col < n) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float d = v[c].v[i] - mean;
        q += d * d;
      }
    }
  }
  float rstd = rsqrtf(warp_sum(q) / (float)n + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    int col = (c * 32 + lane) * 8;
    if (col < n) {
      F8 g = load8(gamma, col, w_bf16);
      F8 o;
      if (beta) {
        F8 b = load8(beta, col, w_bf16);
#pragma unroll
        for (int i = 0; i < 8; ++i) o.v[i] = (v[c].v[i] - mean) * rstd * g.v[i] + b.v[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o.v[i] = (v[c].v[i] - mean) * rstd * g.v[i];
      }
      store8(y, base + col, o, x_bf16);
    }
  }
}

// general n: re-reads the row (second and third pass hit L1/L2)
__global__ void __launch_bounds__(kWarpsPerCta * 32)
ln_fwd_kernel_big(const void* __restrict__ x, const void* __restrict__ gamma, const void* __restrict__ beta,
                  void* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                  int64_t rows, int n, float eps, int x_bf16, int w_bf16, int rms) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = row * (int64_t)n;
  float s = 0.f;
  for (int col = lane * 8; col < n; col += 256) {
    F8 a = load8(x, base + col, x_bf16);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += a.v[i];
  }
  float mean = rms ? 0.f : warp_sum(s) / (float)n;
  float q = 0.f;
  for (int col = lane * 8; col < n; col += 256) {
    F8 a = load8(x, base + col, x_bf16);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float d = a.v[i] - mean;
      q += d * d;
    }
  }
  float rstd = rsqrtf(warp_sum(q) / (float)n + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  for (int col = lane * 8; col < n; col += 256) {
    F8 a = load8(x, base + col, x_bf16);
    F8 g = load8(gamma, col, w_bf16);
    F8 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = (a.v[i] - mean) * rstd * g.v[i];
    if (beta) {
      F8 b = load8(beta, col, w_bf16);
#pragma unroll
      for (int i = 0; i < 8; ++i) o.v[i] += b.v[i];
    }
    store8(y, base + col, o, x_bf16);
  }
}

// Backward. grid = n_part CTAs; CTA c handles rows c*4+w, stepping by n_part*4.
// part layout: [2][n_part][n] (dgamma partials, then dbeta partials).
template <int CHUNKS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
ln_bwd_kernel(const void* __restrict__ x, const void* __restrict__ dy, const void* __restrict__ gamma,
              const float* __restrict__ mean_in, const float* __restrict__ rstd_in, void* __restrict__ dx,
              float* __restrict__ part, int64_t rows, int n, int n_part, int x_bf16, int w_bf16, int rms,
              const void* __restrict__ dres = nullptr) {
  extern __shared__ float smem[];  // [kWarpsPerCta][2][n]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  F8 g[CHUNKS];
  F8 acc_g[CHUNKS], acc_b[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    int col = (c * 32 + lane) * 8;
    if (col < n) g[c] = load8(gamma, col, w_bf16);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc_g[c].v[i] = 0.f;
      acc_b[c].v[i] = 0.f;
    }
  }
  for (int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + warp; row < rows; row += (int64_t)n_part * kWarpsPerCta) {
    const int64_t base = row * (int64_t)n;
    const float mean = mean_in[row], rstd = rstd_in[row];
    F8 xh[CHUNKS], d[CHUNKS];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      int col = (c * 32 + lane) * 8;
      if (col < n) {
        xh[c] = load8(x, base + col, x_bf16);
        d[c] = load8(dy, base + col, x_bf16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c].v[i] = (xh[c].v[i] - mean) * rstd;
          float gd = g[c].v[i] * d[c].v[i];
          s1 += gd;
          s2 += gd * xh[c].v[i];
          acc_g[c].v[i] += d[c].v[i] * xh[c].v[i];
          acc_b[c].v[i] += d[c].v[i];
        }
      }
    }
    s1 = rms ? 0.f : warp_sum(s1) / (float)n;
    s2 = warp_sum(s2) / (float)n;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      int col = (c * 32 + lane) * 8;
      if (col < n) {
        F8 o;
#pragma unroll
        for (int i = 0; i < 8; ++i) o.v[i] = rstd * (g[c].v[i] * d[c].v[i] - s1 - xh[c].v[i] * s2);
        if (dres) {
          // gradient that reaches x along the residual branch
          F8 rr = load8(dres, base + col, x_bf16);
#pragma unroll
          for (int i = 0; i < 8; ++i) o.v[i] += rr.v[i];
        }
        store8(dx, base + col, o, x_bf16);
      }
    }
  }
  // reduce the 4 warps of the CTA through shared memory
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    int col = (c * 32 + lane) * 8;
    if (col < n) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        smem[(warp * 2 + 0) * n + col + i] = acc_g[c].v[i];
        smem[(warp * 2 + 1) * n + col + i] = acc_b[c].v[i];
      }
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < n; col += blockDim.x) {
    float sg = 0.f, sb = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerCta; ++w) {
      sg += smem[(w * 2 + 0) * n + col];
      sb += smem[(w * 2 + 1) * n + col];
    }
    part[((int64_t)0 * n_part + blockIdx.x) * n + col] = sg;
    part[((int64_t)1 * n_part + blockIdx.x) * n + col] = sb;
  }
}

// Backward for bf16 activations with accumulation into fp32 dgamma / dbeta (the form the training step uses). One CTA of
// 16 warps per SM. A warp owns only two or three rows of a launch, so the cost of a row is the latency of its loads: every warp
// keeps a ring of kBwdAccDepth rows (x, dy, residual gradient) in flight through cp.async into shared memory, each lane fetching
// exactly the 16-byte pieces it reads back itself (no barrier between fetch and use), with the rows' mean / rstd parked in the
// lanes of the warp. The 16 warps' column sums meet in the same shared memory afterwards and leave as one atomic per column and
// CTA: no partials buffer and no second kernel.
constexpr int kBwdAccWarps = 16;
constexpr int kBwdAccDepth = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int CHUNKS>
__global__ void __launch_bounds__(kBwdAccWarps * 32, 1)
ln_bwd_acc_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const void* __restrict__ gamma,
                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                  float* __restrict__ dgamma, float* __restrict__ dbeta, int64_t rows, int n, int w_bf16, int rms,
                  const __nv_bfloat16* __restrict__ dres) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  extern __shared__ __align__(16) unsigned char smem_raw[];  // [warps][depth][3][n] bf16, later [warps][2][n] fp32
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * kBwdAccDepth * 3 * n;
  F8 g[CHUNKS], acc_g[CHUNKS], acc_b[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < n) g[c] = load8(gamma, col, w_bf16);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_g[c].v[i] = acc_b[c].v[i] = 0.f;
  }
  const int64_t stride = (int64_t)gridDim.x * kBwdAccWarps;
  const int64_t row0 = (int64_t)blockIdx.x * kBwdAccWarps + warp;
  float my_mean = 0.f, my_rstd = 0.f;  // of the row in ring slot `lane` (lanes < depth)
  auto fetch = [&](int64_t r, int slot) {
    if (r < rows) {
      const int64_t base = r * (int64_t)n;
      __nv_bfloat16* dst = ring + (size_t)slot * 3 * n;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < n) {
          cp_async16(dst + col, x + base + col);
          cp_async16(dst + n + col, dy + base + col);
          if (dres) cp_async16(dst + 2 * n + col, dres + base + col);
        }
      }
      if (lane == slot) {
        my_mean = mean_in[r];
        my_rstd = rstd_in[r];
      }
    }
    cp_async_commit();  // also when nothing was issued: the group count per iteration stays fixed
  };
  auto unpack = [](const uint4& u, F8& f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __bfloat1622float2(h[i]);
      f.v[2 * i] = p.x;
      f.v[2 * i + 1] = p.y;
    }
  };
#pragma unroll
  for (int k = 0; k < kBwdAccDepth; ++k) fetch(row0 + k * stride, k);
  int slot = 0;
  for (int64_t row = row0; row < rows; row += stride) {
    cp_async_wait<kBwdAccDepth - 1>();  // the oldest group (this row) has landed; own copies only, so no barrier
    const float mean = __shfl_sync(0xffffffffu, my_mean, slot), rstd = __shfl_sync(0xffffffffu, my_rstd, slot);
    const int64_t base = row * (int64_t)n;
    const __nv_bfloat16* src = ring + (size_t)slot * 3 * n;
    F8 xh[CHUNKS], d[CHUNKS], res[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < n) {
        unpack(*reinterpret_cast<const uint4*>(src + col), xh[c]);
        unpack(*reinterpret_cast<const uint4*>(src + n + col), d[c]);
        if (dres) unpack(*reinterpret_cast<const uint4*>(src + 2 * n + col), res[c]);
      }
    }
    fetch(row + (int64_t)kBwdAccDepth * stride, slot);  // the slot is in registers now
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < n) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c].v[i] = (xh[c].v[i] - mean) * rstd;
          const float gd = g[c].v[i] * d[c].v[i];
          s1 += gd;
          s2 += gd * xh[c].v[i];
          acc_g[c].v[i] += d[c].v[i] * xh[c].v[i];
          acc_b[c].v[i] += d[c].v[i];
        }
      }
    }
    s1 = rms ? 0.f : warp_sum(s1) / (float)n;
    s2 = warp_sum(s2) / (float)n;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < n) {
        F8 o;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o.v[i] = rstd * (g[c].v[i] * d[c].v[i] - s1 - xh[c].v[i] * s2);
          if (dres) o.v[i] += res[c].v[i];
        }
        store8(dx, base + col, o, 1);
      }
    }
    slot = slot + 1 == kBwdAccDepth ? 0 : slot + 1;
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the memory becomes [warps][2][n] fp32
  float* sums = reinterpret_cast<float*>(smem_raw);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < n) {
      float* pg = sums + (size_t)(warp * 2) * n + col;
      *reinterpret_cast<float4*>(pg) = make_float4(acc_g[c].v[0], acc_g[c].v[1], acc_g[c].v[2], acc_g[c].v[3]);
      *reinterpret_cast<float4*>(pg + 4) = make_float4(acc_g[c].v[4], acc_g[c].v[5], acc_g[c].v[6], acc_g[c].v[7]);
      *reinterpret_cast<float4*>(pg + n) = make_float4(acc_b[c].v[0], acc_b[c].v[1], acc_b[c].v[2], acc_b[c].v[3]);
      *reinterpret_cast<float4*>(pg + n + 4) = make_float4(acc_b[c].v[4], acc_b[c].v[5], acc_b[c].v[6], acc_b[c].v[7]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {  // i < n: dgamma column i, else dbeta column i - n
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kBwdAccWarps; ++w) t += sums[(size_t)w * 2 * n + i];
    if (i < n) {
      if (dgamma) atomicAdd(dgamma + i, t);
    } else if (dbeta) {
      atomicAdd(dbeta + i - n, t);
    }
  }
}

// partial sums -> dgamma / dbeta. Block = 32 columns x 8 slices of the partials; grid = ceil(n / 32).
__global__ void __launch_bounds__(256)
ln_bwd_reduce_kernel(const float* __restrict__ part, float* __restrict__ dgamma, float* __restrict__ dbeta, int n, int n_part,
                     int accumulate = 0) {
  __shared__ float red[2][8][32];
  const int cl = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cl;
  float sg = 0.f, sb = 0.f;
  if (col < n) {
    for (int p = sl; p < n_part; p += 8) {
      sg += part[((int64_t)0 * n_part + p) * n + col];
      sb += part[((int64_t)1 * n_part + p) * n + col];
    }
  }
  red[0][sl][cl] = sg;
  red[1][sl][cl] = sb;
  __syncthreads();
  if (sl == 0 && col < n) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      sg += red[0][k][cl];
      sb += red[1][k][cl];
    }
    if (accumulate) {
      if (dgamma) dgamma[col] += sg;
      if (dbeta) dbeta[col] += sb;
    } else {
      if (dgamma) dgamma[col] = sg;
      if (dbeta) dbeta[col] = sb;
    }
  }
}

}  // namespace

RB_EXPORT int rb200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                   long long rows, int n, float eps, int x_bf16, int w_bf16, int rms, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  if (n % 8 != 0 || n <= 0) {
    rb_set_error("layer_norm: n=%d must be a positive multiple of 8", n);
    return RB_ERR_ARG;
  }
  dim3 grid((unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta)), block(kWarpsPerCta * 32);
  int chunks = (n + 255) / 256;
#define LN_FWD(C) rb_launch_pdl(ln_fwd_kernel<C>, dim3(grid), dim3(block), 0, stream, x, gamma, beta, y, mean, rstd, rows, n, eps, x_bf16, w_bf16, rms)
  if (chunks <= 1) LN_FWD(1);
  else if (chunks <= 2) LN_FWD(2);
  else if (chunks <= 4) LN_FWD(4);
  else if (chunks <= 8) LN_FWD(8);
  else ln_fwd_kernel_big<<<grid, block, 0, stream>>>(x, gamma, beta, y, mean, rstd, rows, n, eps, x_bf16, w_bf16, rms);
#undef LN_FWD
  return rb_check_launch("layer_norm_fwd");
}

// dres (optional, same layout as dx): added to dx; accumulate: dgamma / dbeta += instead of =
RB_EXPORT int rb200_layer_norm_bwd_ex(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                                      void* dx, float* part, float* dgamma, float* dbeta, long long rows, int n, int n_part,
                                      int x_bf16, int w_bf16, int rms, const void* dres, int accumulate, cudaStream_t stream) {
  if (n % 8 != 0 || n <= 0 || n > kMaxChunks * 256) {
    rb_set_error("layer_norm_bwd: n=%d must be a multiple of 8 and <= %d", n, kMaxChunks * 256);
    return RB_ERR_ARG;
  }
  if (n_part <= 0) return RB_ERR_ARG;
  if (accumulate && x_bf16 && n <= 512 && rows > 0 && (dgamma || dbeta)) {
    int ctas = (int)((rows + kBwdAccWarps - 1) / kBwdAccWarps);
    if (ctas > 148) ctas = 148;
    const size_t sm = (size_t)kBwdAccWarps * kBwdAccDepth * 3 * n * sizeof(__nv_bfloat16);  // >= the [warps][2][n] fp32 it becomes at the end
    const int ch = (n + 255) / 256;
    static bool attr_set[2] = {false, false};
#define LN_ACC(C)                                                                                                                       \
  if (!attr_set[C - 1]) {                                                                                                               \
    if (cudaFuncSetAttribute(ln_bwd_acc_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)kBwdAccWarps * kBwdAccDepth * 3 * 512 * 2)) != cudaSuccess) { \
      rb_set_error("layer_norm_bwd_acc: cannot reserve shared memory");                                                                 \
      return RB_ERR_LAUNCH;                                                                                                              \
    }                                                                                                                                   \
    attr_set[C - 1] = true;                                                                                                             \
  }                                                                                                                                     \
  rb_launch_pdl(ln_bwd_acc_kernel<C>, dim3(ctas), dim3(kBwdAccWarps * 32), sm, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, gamma, mean, rstd, \
                                                                 (__nv_bfloat16*)dx, dgamma, dbeta, rows, n, w_bf16, rms,              \
                                                                 (const __nv_bfloat16*)dres)
    if (ch <= 1) {
      LN_ACC(1);
    } else {
      LN_ACC(2);
    }
#undef LN_ACC
    return rb_check_launch("layer_norm_bwd_acc");
  }
  dim3 grid(n_part), block(kWarpsPerCta * 32);
  size_t smem = (size_t)kWarpsPerCta * 2 * n * sizeof(float);
  int chunks = (n + 255) / 256;
#define LN_BWD(C)                                                                                          \
  do {                                                                                                     \
    if (smem > 48 * 1024) cudaFuncSetAttribute(ln_bwd_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    ln_bwd_kernel<C><<<grid, block, smem, stream>>>(x, dy, gamma, mean, rstd, dx, part, rows, n, n_part, x_bf16, w_bf16, rms, dres); \
  } while (0)
  if (chunks <= 1) LN_BWD(1);
  else if (chunks <= 2) LN_BWD(2);
  else if (chunks <= 4) LN_BWD(4);
  else LN_BWD(8);
#undef LN_BWD
  int st = rb_check_launch("layer_norm_bwd");
  if (st) return st;
  ln_bwd_reduce_kernel<<<(n + 31) / 32, 256, 0, stream>>>(part, dgamma, dbeta, n, n_part, accumulate);
  return rb_check_launch("layer_norm_bwd_reduce");
}

RB_EXPORT int rb200_layer_norm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                                   void* dx, float* part, float* dgamma, float* dbeta, long long rows, int n, int n_part,
                                   int x_bf16, int w_bf16, int rms, cudaStream_t stream) {
  return rb200_layer_norm_bwd_ex(x, dy, gamma, mean, rstd, dx, part, dgamma, dbeta, rows, n, n_part, x_bf16, w_bf16, rms, nullptr, 0, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared in no_alloc.h).
//
// rb200_layer_norm_bwd above takes its scratch (the per-CTA partial sums of dgamma / dbeta) from the caller, who has to
// allocate n_part * n * 2 floats of device memory for every call. Some callers cannot do that: a host program that links
// this library without an allocator of its own (no torch), a serving process whose memory pool already owns all of the
// device memory so that a cudaMalloc at call time fails, or a latency-critical loop in which the implicit device-wide
// synchronisation of cudaMalloc / cudaFree is not acceptable. For them the scratch lives in the fixed array below.
//
// The array is part of the library image: every GPU on which the library is used holds kNoAllocScratchFloats * 4 bytes
// (2.3 MiB) from the first use until the process exits. All calls on a device share it and it keeps the contents of the
// previous call. Nothing in it has to start at zero: each launch overwrites every partial that its second pass reads.
// Two calls that overlap on the same GPU (different streams, or different host threads) race on the array; callers
// must serialise them, e.g. by using one stream.
namespace {

constexpr int kNoAllocParts = 148;                                   // one partial per SM
constexpr int kNoAllocMaxN = kMaxChunks * 256;                       // 2048 columns
constexpr size_t kNoAllocScratchFloats = (size_t)2 * kNoAllocParts * kNoAllocMaxN;

static __device__ __align__(256) float g_ln_bwd_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// The name g_ln_bwd_scratch is only a host-side handle here; the device address has to be looked up once per device,
// with that device current.
int no_alloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    rb_set_error("layer_norm_bwd_noalloc: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return RB_ERR_LAUNCH;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_ln_bwd_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      rb_set_error("layer_norm_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return RB_ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return RB_OK;
}

}  // namespace

RB_EXPORT int rb200_layer_norm_bwd_noalloc(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                                           void* dx, float* dgamma, float* dbeta, long long rows, int n, int x_bf16, int w_bf16, int rms,
                                           cudaStream_t stream) {
  if (n <= 0 || n % 8 != 0 || n > kNoAllocMaxN) {
    rb_set_error("layer_norm_bwd_noalloc: n=%d is not supported: the built-in scratch holds rows of at most %d columns (multiple of 8)",
                 n, kNoAllocMaxN);
    return RB_ERR_ARG;
  }
  if (rows <= 0) {
    rb_set_error("layer_norm_bwd_noalloc: rows=%lld", rows);
    return RB_ERR_ARG;
  }
  float* scratch = nullptr;
  int st = no_alloc_scratch(&scratch);
  if (st) return st;
  return rb200_layer_norm_bwd(x, dy, gamma, mean, rstd, dx, scratch, dgamma, dbeta, rows, n, kNoAllocParts, x_bf16, w_bf16, rms, stream);
}

RB_EXPORT int rb200_layer_norm_bwd_noalloc_max_n() { return kNoAllocMaxN; }
RB_EXPORT int rb200_layer_norm_bwd_noalloc_parts() { return kNoAllocParts; }
