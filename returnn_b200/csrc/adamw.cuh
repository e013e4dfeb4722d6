// AdamW element update shared by the optimizer kernel and the fused parameter-averaging kernel.
#pragma once
#include "common.cuh"

__device__ __forceinline__ float load_grad(const void* g, int64_t i, int g_bf16) {
  return g_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]) : reinterpret_cast<const float*>(g)[i];
}

struct AdamwArgs {
  float* p;
  const void* g;
  float* m;
  float* v;
  const uint8_t* wd_flags;  // one flag per 128 elements: weight decay applies
  int64_t n;
  int g_bf16;
  float lr, b1, b2, eps, wd, bc1, bc2;
  int decoupled;
  float clip;
  const float* norm;         // global gradient norm (device scalar) or null
  __nv_bfloat16* p_bf16;     // optional bf16 copy of the updated weights
};

// AdamW over elements [0, n) spread over `nthreads` threads (this thread is number `tid`); one thread handles 4 consecutive
// elements at a time (16-byte accesses on p, m, v and fp32 g)
__device__ __forceinline__ void adamw_update_range(const AdamwArgs& a_, int64_t tid, int64_t nthreads) {
  float* __restrict__ p = a_.p;
  const void* __restrict__ g = a_.g;
  float* __restrict__ m = a_.m;
  float* __restrict__ v = a_.v;
  const uint8_t* __restrict__ wd_flags = a_.wd_flags;
  const int64_t n = a_.n;
  const int g_bf16 = a_.g_bf16, decoupled = a_.decoupled;
  const float lr = a_.lr, b1 = a_.b1, b2 = a_.b2, eps = a_.eps, wd = a_.wd, bc1 = a_.bc1, bc2 = a_.bc2, clip = a_.clip;
  const float* __restrict__ norm = a_.norm;
  __nv_bfloat16* __restrict__ p_bf16 = a_.p_bf16;
  float scale = 1.f;
  if (norm != nullptr && clip > 0.f) scale = fminf(1.f, clip / (norm[0] + 1e-6f));
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (int64_t i4 = tid * 4; i4 < n; i4 += nthreads * 4) {
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

