// Softmax cross entropy with label smoothing over a large vocabulary.
// One CTA per row; online softmax (running max and sum) in one pass over the logits; backward recomputes
// p = exp(x - lse) and writes dlogits = dloss * (p - q) with q the smoothed target distribution.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ld(const void* x, int64_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]) : reinterpret_cast<const float*>(x)[i];
}

__global__ void __launch_bounds__(256)
ce_fwd_kernel(const void* __restrict__ logits, const int* __restrict__ tgt, float* __restrict__ loss, float* __restrict__ lse_out,
              int v, float smoothing, int is_bf16) {
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)v;
  float mx = -INFINITY, sum = 0.f, tot = 0.f;
  const int v8 = ((base & 7) == 0) ? (v & ~7) : 0;  // vector path only when the row start is 16-byte aligned
  for (int c = threadIdx.x * 8; c < v8; c += blockDim.x * 8) {
    F8 a = load8(logits, base + c, is_bf16);
    float lm = a.v[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, a.v[k]);
    float nm = fmaxf(mx, lm);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      s += __expf(a.v[k] - nm);
      tot += a.v[k];
    }
    sum = sum * __expf(mx - nm) + s;
    mx = nm;
  }
  for (int c = v8 + threadIdx.x; c < v; c += blockDim.x) {
    float a = ld(logits, base + c, is_bf16);
    float nm = fmaxf(mx, a);
    sum = sum * __expf(mx - nm) + __expf(a - nm);
    mx = nm;
    tot += a;
  }
  __shared__ float sh_m[8], sh_s[8], sh_t[8];
  float wm = warp_max(mx);
  float ws = warp_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - wm));
  float wt = warp_sum(tot);
  if ((threadIdx.x & 31) == 0) {
    sh_m[threadIdx.x >> 5] = wm;
    sh_s[threadIdx.x >> 5] = ws;
    sh_t[threadIdx.x >> 5] = wt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = sh_m[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, sh_m[w]);
    float s = 0.f, t = 0.f;
    for (int w = 0; w < 8; ++w) {
      if (sh_m[w] != -INFINITY) s += sh_s[w] * __expf(sh_m[w] - m);
      t += sh_t[w];
    }
    float lse = m + logf(s);
    int y = tgt[row];
    float xy = (y >= 0 && y < v) ? ld(logits, base + y, is_bf16) : 0.f;
    float nll = lse - xy;
    float l = nll;
    if (smoothing > 0.f) {
      // other = mean over the v-1 non-target classes of (lse - x_c)
      float other = ((float)v * lse - t - nll) / (float)(v - 1);
      l = (1.f - smoothing) * nll + smoothing * other;
    }
    loss[row] = (y >= 0 && y < v) ? l : 0.f;
    lse_out[row] = lse;
  }
}

__global__ void __launch_bounds__(256)
ce_bwd_kernel(const void* __restrict__ logits, const int* __restrict__ tgt, const float* __restrict__ lse_in,
              const float* __restrict__ dloss, void* __restrict__ dlogits, int v, float smoothing, int is_bf16) {
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)v;
  const float lse = lse_in[row];
  const int y = tgt[row];
  const bool valid = y >= 0 && y < v;
  const float dl = valid ? dloss[row] : 0.f;
  const float q_other = smoothing > 0.f ? smoothing / (float)(v - 1) : 0.f;
  const float q_tgt = 1.f - smoothing;
  const int v8 = ((base & 7) == 0) ? (v & ~7) : 0;
  for (int c = threadIdx.x * 8; c < v8; c += blockDim.x * 8) {
    F8 a = load8(logits, base + c, is_bf16);
    F8 o;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(a.v[k] - lse);
      float q = (c + k == y) ? q_tgt : q_other;
      o.v[k] = dl * (p - q);
    }
    store8(dlogits, base + c, o, is_bf16);
  }
  for (int c = v8 + threadIdx.x; c < v; c += blockDim.x) {
    float p = __expf(ld(logits, base + c, is_bf16) - lse);
    float q = (c == y) ? q_tgt : q_other;
    float o = dl * (p - q);
    if (is_bf16) reinterpret_cast<__nv_bfloat16*>(dlogits)[base + c] = __float2bfloat16(o);
    else reinterpret_cast<float*>(dlogits)[base + c] = o;
  }
}

}  // namespace

RB_EXPORT int rb200_softmax_ce_fwd(const void* logits, const int* tgt, float* loss, float* lse, long long rows, int v, float smoothing,
                                   int is_bf16, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  if (v < 2) return RB_ERR_ARG;
  ce_fwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, loss, lse, v, smoothing, is_bf16);
  return rb_check_launch("softmax_ce_fwd");
}

RB_EXPORT int rb200_softmax_ce_bwd(const void* logits, const int* tgt, const float* lse, const float* dloss, void* dlogits,
                                   long long rows, int v, float smoothing, int is_bf16, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  ce_bwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, lse, dloss, dlogits, v, smoothing, is_bf16);
  return rb_check_launch("softmax_ce_bwd");
}
