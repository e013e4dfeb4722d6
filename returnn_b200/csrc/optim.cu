// Optimizer kernels over a flat arena: fused Adam/AdamW with in-kernel clip coefficient, sum of squares, Lion.
#include "common.cuh"

namespace {

__device__ __forceinline__ float load_grad(const void* g, int64_t i, int g_bf16) {
  return g_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]) : reinterpret_cast<const float*>(g)[i];
}

// one thread handles 4 consecutive elements (16-byte accesses on p, m, v and fp32 g)
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const void* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             const uint8_t* __restrict__ wd_flags, int64_t n, int g_bf16, float lr, float b1, float b2, float eps, float wd,
             float bc1, float bc2, int decoupled, float clip, const float* __restrict__ norm, __nv_bfloat16* __restrict__ p_bf16) {
  float scale = 1.f;
  if (norm != nullptr && clip > 0.f) scale = fminf(1.f, clip / (norm[0] + 1e-6f));
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i4 < n; i4 += (int64_t)gridDim.x * blockDim.x * 4) {
    float pv[4], gv[4], mv[4], vv[4];
    const bool full = i4 + 4 <= n;
    if (full) {
      float4 a = *reinterpret_cast<const float4*>(p + i4);
      pv[0] = a.x; pv[1] = a.y; pv[2] = a.z; pv[3] = a.w;
      a = *reinterpret_cast<const float4*>(m + i4);
      mv[0] = a.x; mv[1] = a.y; mv[2] = a.z; mv[3] = a.w;
      a = *reinterpret_cast<const float4*>(v + i4);
      vv[0] = a.x; vv[1] = a.y; vv[2] = a.z; vv[3] = a.w;
      if (g_bf16) {
        uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(g) + i4);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
        float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
        gv[0] = f0.x; gv[1] = f0.y; gv[2] = f1.x; gv[3] = f1.y;
      } else {
        a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + i4);
        gv[0] = a.x; gv[1] = a.y; gv[2] = a.z; gv[3] = a.w;
      }
    } else {
      for (int k = 0; k < 4; ++k) {
        bool ok = i4 + k < n;
        pv[k] = ok ? p[i4 + k] : 0.f;
        mv[k] = ok ? m[i4 + k] : 0.f;
        vv[k] = ok ? v[i4 + k] : 0.f;
        gv[k] = ok ? load_grad(g, i4 + k, g_bf16) : 0.f;
      }
    }
    const float decay = wd_flags[i4 >> 7] ? wd : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gg = gv[k] * scale;
      if (!decoupled) gg += decay * pv[k];
      mv[k] = b1 * mv[k] + (1.f - b1) * gg;
      vv[k] = b2 * vv[k] + (1.f - b2) * gg * gg;
      float denom = sqrtf(vv[k]) * inv_sqrt_bc2 + eps;
      float w = pv[k];
      if (decoupled) w *= (1.f - lr * decay);
      pv[k] = w - lr * (mv[k] * inv_bc1) / denom;
    }
    if (full) {
      *reinterpret_cast<float4*>(p + i4) = make_float4(pv[0], pv[1], pv[2], pv[3]);
      *reinterpret_cast<float4*>(m + i4) = make_float4(mv[0], mv[1], mv[2], mv[3]);
      *reinterpret_cast<float4*>(v + i4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (p_bf16) {
        uint2 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
        h[0] = __floats2bfloat162_rn(pv[0], pv[1]);
        h[1] = __floats2bfloat162_rn(pv[2], pv[3]);
        *reinterpret_cast<uint2*>(p_bf16 + i4) = u;
      }
    } else {
      for (int k = 0; k < 4 && i4 + k < n; ++k) {
        p[i4 + k] = pv[k];
        m[i4 + k] = mv[k];
        v[i4 + k] = vv[k];
        if (p_bf16) p_bf16[i4 + k] = __float2bfloat16(pv[k]);
      }
    }
  }
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
  adamw_kernel<<<grid, 256, 0, stream>>>(p, g, m, v, wd_flags, n, g_bf16, lr, b1, b2, eps, wd, bc1, bc2, decoupled, clip, norm, p_bf16);
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
