// Optimizer kernels over a flat arena: fused Adam/AdamW with in-kernel clip coefficient, sum of squares, Lion.
#include "common.cuh"
#include "adamw.cuh"

namespace {

__global__ void __launch_bounds__(256) adamw_kernel(const AdamwArgs a) {
  adamw_update_range(a, (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
}

constexpr int kSsqCtas = 1024;

__global__ void __launch_bounds__(256) sumsq_partial_kernel(const void* __restrict__ x, int64_t n, int is_bf16, float* __restrict__ part) {
  float s = 0.f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 8;
  const int64_t n8 = n & ~(int64_t)7;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n8; i += stride) {
    F8 a = load8(x, i, is_bf16);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += a.v[k] * a.v[k];
  }
  if (blockIdx.x == 0 && threadIdx.x < (n - n8)) {
    float t = load_grad(x, n8 + threadIdx.x, is_bf16);
    s += t * t;
  }
  __shared__ float sh[8];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? sh[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) part[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(1024) sumsq_final_kernel(const float* __restrict__ part, int n_part, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = threadIdx.x < n_part ? part[threadIdx.x] : 0.f;
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = sh[threadIdx.x];
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = t;
  }
}

__global__ void __launch_bounds__(256)
lion_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, int64_t n, float lr, float wd, float b1, float b2) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float pv = p[i], gv = g[i], mv = m[i];
    pv *= (1.f - lr * wd);
    float u = b1 * mv + (1.f - b1) * gv;
    pv -= lr * (u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f));
    m[i] = b2 * mv + (1.f - b2) * gv;
    p[i] = pv;
  }
}

}  // namespace

RB_EXPORT int rb200_adamw_arena(float* p, const void* g, float* m, float* v, const uint8_t* wd_flags, long long n, int g_bf16,
                                float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, int decoupled, float clip,
                                const float* norm, __nv_bfloat16* p_bf16, cudaStream_t stream) {
  if (n <= 0) return RB_OK;
  long long threads = (n + 3) / 4;
  int grid = (int)((threads + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  AdamwArgs a{p, g, m, v, wd_flags, (int64_t)n, g_bf16, lr, b1, b2, eps, wd, bc1, bc2, decoupled, clip, norm, p_bf16};
  adamw_kernel<<<grid, 256, 0, stream>>>(a);
  return rb_check_launch("adamw_arena");
}

// scratch: at least 1024 floats of device memory for the per-CTA partial sums
RB_EXPORT int rb200_sum_squares(const void* x, long long n, int is_bf16, float* scratch, float* out, cudaStream_t stream) {
  int grid = (int)((n / 8 + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > kSsqCtas) grid = kSsqCtas;
  sumsq_partial_kernel<<<grid, 256, 0, stream>>>(x, n, is_bf16, scratch);
  int st = rb_check_launch("sum_squares_partial");
  if (st) return st;
  sumsq_final_kernel<<<1, 1024, 0, stream>>>(scratch, grid, out);
  return rb_check_launch("sum_squares_final");
}

RB_EXPORT int rb200_lion(float* p, const float* g, float* m, long long n, float lr, float wd, float b1, float b2, cudaStream_t stream) {
  if (n <= 0) return RB_OK;
  int grid = (int)((n + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  lion_kernel<<<grid, 256, 0, stream>>>(p, g, m, n, lr, wd, b1, b2);
  return rb_check_launch("lion");
}
