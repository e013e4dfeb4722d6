// Attention of ONE query position per (hypothesis, head) over a key / value cache: the attention of a decoding step.
//   out[n, h, :] = softmax_t(scale * q[n, h, :] . K[n / group, h, t, :]) V[n / group, h, t, :],  t < valid(n)
// `group` consecutive hypotheses share one cache entry: in beam search the encoder keys / values of a sequence are the same for all its
// beam hypotheses, so the cross-attention cache is stored (and read) once per sequence instead of once per hypothesis.
// valid(n) = lens[n / group] (encoder lengths) or *pos + 1 (the device-side step counter of a self-attention cache, so that the launch
// can sit in a captured graph). One warp per (n, h); the lanes split the key positions, each keeps an online-softmax partial
// (max, sum, weighted value row) and the partials are merged with shuffles. The op is bound by reading the cache once.
// bf16 in / out, fp32 arithmetic; head dim 64 or 128.
#include "common.cuh"

namespace {

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(w[e] << 16);
    f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
}

template <int D>
__global__ void __launch_bounds__(256)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                        const int* __restrict__ lens, const long long* __restrict__ pos, int N, int H, int T, int group, float scale,
                        __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (n, h)
  if (w >= N * H) return;
  const int n = w / H, h = w - n * H;
  const int nk = n / group;
  int valid = lens ? lens[nk] : (int)(pos[0] + 1);
  valid = min(max(valid, 0), T);
  float qf[D];
  {
    const uint4* qp = reinterpret_cast<const uint4*>(q + ((size_t)n * H + h) * D);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) unpack8(__ldg(qp + i), qf + 8 * i);
  }
  const size_t base = ((size_t)nk * H + h) * T;
  float m = -INFINITY, l = 0.f;
  float acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.f;
  for (int t = lane; t < valid; t += 32) {
    const uint4* kp = reinterpret_cast<const uint4*>(k + (base + t) * D);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      float kf[8];
      unpack8(__ldg(kp + i), kf);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += qf[8 * i + e] * kf[e];
    }
    s *= scale;
    const float mn = fmaxf(m, s);
    const float f = __expf(m - mn), e = __expf(s - mn);  // m = -inf at the first key: f = 0
    l = l * f + e;
    const uint4* vp = reinterpret_cast<const uint4*>(v + (base + t) * D);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      float vf[8];
      unpack8(__ldg(vp + i), vf);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[8 * i + j] = acc[8 * i + j] * f + e * vf[j];
    }
    m = mn;
  }
  const float M = warp_max(m);
  const float f = (m == -INFINITY) ? 0.f : __expf(m - M);
  l = warp_sum(l * f);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* o = out + ((size_t)n * H + h) * D;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    const float total = warp_sum(acc[d] * f);
    if (lane == (d & 31)) o[d] = __float2bfloat16(total * inv);
  }
}

}  // namespace

// q [N, H, D], k / v [N / group, H, T, D], out [N, H, D], all bf16 contiguous; exactly one of lens [N / group] and pos [1] is given
RB_EXPORT int rb200_decode_attention(const void* q, const void* k, const void* v, const int* lens, const long long* pos, int N, int H, int T, int D,
                                     int group, float scale, void* out, cudaStream_t stream) {
  if (N <= 0 || H <= 0) return RB_OK;
  if ((D != 64 && D != 128) || group < 1 || N % group != 0 || (lens == nullptr) == (pos == nullptr)) {
    rb_set_error("decode_attention: head dim %d (64 or 128), group %d (must divide N = %d), one of lens / pos", D, group, N);
    return RB_ERR_UNSUPPORTED;
  }
  const int warps = N * H;
  const int blocks = (warps + 7) / 8;
  auto* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  auto* kk = reinterpret_cast<const __nv_bfloat16*>(k);
  auto* vv = reinterpret_cast<const __nv_bfloat16*>(v);
  auto* oo = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 64) decode_attention_kernel<64><<<blocks, 256, 0, stream>>>(qq, kk, vv, lens, pos, N, H, T, group, scale, oo);
  else decode_attention_kernel<128><<<blocks, 256, 0, stream>>>(qq, kk, vv, lens, pos, N, H, T, group, scale, oo);
  return rb_check_launch("decode_attention");
}
