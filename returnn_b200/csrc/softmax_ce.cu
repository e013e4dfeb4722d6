// Softmax cross entropy with label smoothing over a large vocabulary.
// One CTA per row; online softmax (running max and sum) in one pass over the logits; backward recomputes
// p = exp(x - lse) and writes dlogits = dloss * (p - q) with q the smoothed target distribution.
// mode 0: q = (1-s) one-hot + s/(V-1) on the other classes, the loss is the cross entropy against q.
// mode 1: the loss is the plain negative log likelihood and only the gradient is smoothed, uniformly over all V classes
//         (q = (1-s) one-hot + s/V): what an identity with a smoothing backward between log-softmax and the loss computes.
// The forward kernel optionally writes the arg max of each row (first index among equal maxima).
#include "common.cuh"

namespace {

__device__ __forceinline__ float ld(const void* x, int64_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]) : reinterpret_cast<const float*>(x)[i];
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
ce_fwd_kernel(const void* __restrict__ logits, const int* __restrict__ tgt, float* __restrict__ loss, float* __restrict__ lse_out,
              int v, float smoothing, int mode, int* __restrict__ argmax_out) {
  constexpr int is_bf16 = kBf16 ? 1 : 0;
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)v;
  float mx = -INFINITY, sum = 0.f, tot = 0.f;
  int bi = 0x7fffffff;  // index of this thread's first maximum
  const int v8 = ((base & 7) == 0) ? (v & ~7) : 0;  // vector path only when the row start is 16-byte aligned
  // four independent 16-byte loads in flight per thread: the running max / sum chain is short, the loads are the latency
#pragma unroll 4
  for (int c = threadIdx.x * 8; c < v8; c += blockDim.x * 8) {
    F8 a = load8(logits, base + c, is_bf16);
    float lm = a.v[0];
    int li = 0;
#pragma unroll
    for (int k = 1; k < 8; ++k)
      if (a.v[k] > lm) {
        lm = a.v[k];
        li = k;
      }
    if (lm > mx) bi = c + li;
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
    if (a > mx) bi = c;
    float nm = fmaxf(mx, a);
    sum = sum * __expf(mx - nm) + __expf(a - nm);
    mx = nm;
    tot += a;
  }
  __shared__ float sh_m[8], sh_s[8], sh_t[8];
  __shared__ int sh_i[8];
  float wm = warp_max(mx);
  int wi = (mx == wm) ? bi : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wi = min(wi, __shfl_xor_sync(0xffffffffu, wi, o));
  float ws = warp_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - wm));
  float wt = warp_sum(tot);
  if ((threadIdx.x & 31) == 0) {
    sh_m[threadIdx.x >> 5] = wm;
    sh_s[threadIdx.x >> 5] = ws;
    sh_t[threadIdx.x >> 5] = wt;
    sh_i[threadIdx.x >> 5] = wi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = sh_m[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, sh_m[w]);
    float s = 0.f, t = 0.f;
    int am = 0x7fffffff;
    for (int w = 0; w < 8; ++w) {
      if (sh_m[w] != -INFINITY) s += sh_s[w] * __expf(sh_m[w] - m);
      t += sh_t[w];
      if (sh_m[w] == m) am = min(am, sh_i[w]);
    }
    if (argmax_out) argmax_out[row] = am < v ? am : 0;
    float lse = m + logf(s);
    int y = tgt[row];
    float xy = (y >= 0 && y < v) ? ld(logits, base + y, is_bf16) : 0.f;
    float nll = lse - xy;
    float l = nll;
    if (smoothing > 0.f && mode == 0) {
      // other = mean over the v-1 non-target classes of (lse - x_c)
      float other = ((float)v * lse - t - nll) / (float)(v - 1);
      l = (1.f - smoothing) * nll + smoothing * other;
    }
    loss[row] = (y >= 0 && y < v) ? l : 0.f;
    lse_out[row] = lse;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
ce_bwd_kernel(const void* __restrict__ logits, const int* __restrict__ tgt, const float* __restrict__ lse_in,
              const float* __restrict__ dloss, void* __restrict__ dlogits, int v, float smoothing, int mode) {
  constexpr int is_bf16 = kBf16 ? 1 : 0;
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)v;
  const float lse = lse_in[row];
  const int y = tgt[row];
  const bool valid = y >= 0 && y < v;
  const float dl = valid ? dloss[row] : 0.f;
  const float q_other = smoothing > 0.f ? smoothing / (float)(mode == 1 ? v : v - 1) : 0.f;
  const float q_tgt = 1.f - smoothing + (mode == 1 ? q_other : 0.f);
  const int v8 = ((base & 7) == 0) ? (v & ~7) : 0;
#pragma unroll 4
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
                                   int is_bf16, int mode, int* argmax_out, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  if (v < 2) return RB_ERR_ARG;
  if (is_bf16) ce_fwd_kernel<true><<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, loss, lse, v, smoothing, mode, argmax_out);
  else ce_fwd_kernel<false><<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, loss, lse, v, smoothing, mode, argmax_out);
  return rb_check_launch("softmax_ce_fwd");
}

RB_EXPORT int rb200_softmax_ce_bwd(const void* logits, const int* tgt, const float* lse, const float* dloss, void* dlogits,
                                   long long rows, int v, float smoothing, int is_bf16, int mode, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  if (is_bf16) ce_bwd_kernel<true><<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, lse, dloss, dlogits, v, smoothing, mode);
  else ce_bwd_kernel<false><<<(unsigned)rows, 256, 0, stream>>>(logits, tgt, lse, dloss, dlogits, v, smoothing, mode);
  return rb_check_launch("softmax_ce_bwd");
}
