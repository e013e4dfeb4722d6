// Scaled-dot-product attention for self, causal and cross attention (decoder layers, Transformer encoders): the softmax stage
// between the tcgen05 batched GEMMs  S = scale * Q K^T,  O = dropout(P) V  and, backward,  dP = dO V^T,  dQ = scale * dS K,
// dK = scale * dS^T Q,  dV = dropout(P)^T dO.
//
// Score buffers are [B*H, Tqp, Tkp] with Tqp, Tkp = the lengths rounded up to 64: the GEMMs contract over key positions
// (O, dQ) or query positions (dK, dV) in blocks of 64, so the margins [Tk, Tkp) and [Tq, Tqp) are written as zeros here and
// the buffers need no memset. A key j of batch entry b is visible to query i iff j < k_lens[b] (k_lens may be null: all Tk) and,
// for causal attention, j <= i + causal_shift (causal_shift = Tk - Tq: the last query sees all keys; 0 for self attention).
// One warp per query row. Scores (and, backward, the gradient w.r.t. the dropped probabilities) are bf16 as the GEMMs of an
// autocast region write them: a row of up to 1024 keys is read ONCE with 16-byte loads and kept in registers for max, sum and
// write (the *_vec kernels); longer rows and fp32 scores take the scalar three-pass kernels.
//
// Reference semantics: returnn/frontend/_backend.py:1575-1647 (scaled_dot_product_attention: matmul, mask, softmax, dropout,
// matmul; causal via a mask on the upper triangle).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t rng_u32(uint64_t seed, uint64_t idx) {
  uint4 r = philox4x32(make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)), make_uint4((uint32_t)(idx >> 2), (uint32_t)(idx >> 34), 0x51u, 0u));
  const uint32_t sel = (uint32_t)(idx & 3);
  return sel == 0 ? r.x : sel == 1 ? r.y : sel == 2 ? r.z : r.w;
}

__device__ __forceinline__ int visible_keys(int i, int tk, int klen, int causal, int causal_shift) {
  int n = klen < tk ? klen : tk;
  if (causal) {
    const int c = i + causal_shift + 1;
    n = c < n ? c : n;
  }
  return n < 0 ? 0 : n;
}

// s [BH, Tqp, Tkp] fp32 (rows < Tq, columns < Tk valid) -> p, pd [BH, Tqp, Tkp] bf16 (pd only with dropout)
__global__ void __launch_bounds__(128)
sdpa_softmax_fwd_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ p, __nv_bfloat16* __restrict__ pd,
                        const int* __restrict__ k_lens, int heads, int tq, int tk, int tqp, int tkp, int causal, int causal_shift,
                        float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  if (i >= tqp) return;
  const long long row = ((long long)z * tqp + i) * tkp;
  const bool drop = p_drop > 0.f;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  const int n = i < tq ? visible_keys(i, tk, k_lens ? k_lens[z / heads] : tk, causal, causal_shift) : 0;
  float mx = -INFINITY;
  for (int j = lane; j < n; j += 32) mx = fmaxf(mx, s[row + j]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < n; j += 32) sum += __expf(s[row + j] - mx);
  sum = warp_sum(sum);
  const float inv = n > 0 ? 1.f / sum : 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0, off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
  for (int j = lane; j < tkp; j += 32) {
    if (j < n) {
      const float pr = __expf(s[row + j] - mx) * inv;
      p[row + j] = __float2bfloat16(pr);
      if (drop) pd[row + j] = __float2bfloat16(rng_u32(sd, off + (uint64_t)(row + j)) >= thresh ? pr * keep_scale : 0.f);
    } else {
      p[row + j] = zero;
      if (drop) pd[row + j] = zero;
    }
  }
}

// p [BH, Tqp, Tkp] bf16, dpd fp32 (gradient w.r.t. the dropped probabilities) -> ds bf16 = p * (dp - sum_j p dp), dp = mask * dpd / (1-p)
__global__ void __launch_bounds__(128)
sdpa_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ dpd, __nv_bfloat16* __restrict__ ds,
                        const int* __restrict__ k_lens, int heads, int tq, int tk, int tqp, int tkp, int causal, int causal_shift,
                        float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  if (i >= tqp) return;
  const long long row = ((long long)z * tqp + i) * tkp;
  const bool drop = p_drop > 0.f;
  const int n = i < tq ? visible_keys(i, tk, k_lens ? k_lens[z / heads] : tk, causal, causal_shift) : 0;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0, off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
  auto dp_at = [&](int j) {
    float d = dpd[row + j];
    if (drop) d = rng_u32(sd, off + (uint64_t)(row + j)) >= thresh ? d * keep_scale : 0.f;
    return d;
  };
  float delta = 0.f;
  for (int j = lane; j < n; j += 32) delta += __bfloat162float(p[row + j]) * dp_at(j);
  delta = warp_sum(delta);
  for (int j = lane; j < tkp; j += 32) {
    float v = 0.f;
    if (j < n) v = __bfloat162float(p[row + j]) * (dp_at(j) - delta);
    ds[row + j] = __float2bfloat16(v);
  }
}

// ---- bf16 rows in registers. LPR lanes share a row (32 / LPR rows per warp, so that short rows keep every lane busy); lane l of the
// row holds elements [c * LPR * 8 + l * 8, + 8) for chunks c < CHUNKS (tkp <= CHUNKS * LPR * 8).
constexpr int kVecMaxKeys = 1024;

template <int LPR>
__device__ __forceinline__ float row_max(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8_bf16(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(w[e] << 16);
    f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack8_bf16(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    w[e] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// keep flags of 8 consecutive elements starting at idx (the same element -> random word mapping as rng_u32: counter idx >> 2, word idx & 3)
__device__ __forceinline__ uint32_t keep_mask8(uint64_t seed, uint64_t idx, uint32_t thresh) {
  uint32_t mask = 0;
  uint64_t have = ~0ull;
  uint4 r = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint64_t i = idx + e, c = i >> 2;
    if (c != have) {
      r = philox4x32(make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)), make_uint4((uint32_t)c, (uint32_t)(c >> 32), 0x51u, 0u));
      have = c;
    }
    const uint32_t sel = (uint32_t)(i & 3);
    const uint32_t word = sel == 0 ? r.x : sel == 1 ? r.y : sel == 2 ? r.z : r.w;
    mask |= (word >= thresh ? 1u : 0u) << e;
  }
  return mask;
}

template <int LPR, int CHUNKS>
__global__ void __launch_bounds__(128)
sdpa_softmax_fwd_vec_kernel(const __nv_bfloat16* __restrict__ s, __nv_bfloat16* __restrict__ p, __nv_bfloat16* __restrict__ pd,
                            const int* __restrict__ k_lens, int heads, int tq, int tk, int tqp, int tkp, int causal, int causal_shift,
                            float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  constexpr int RPW = 32 / LPR;  // rows per warp
  const int lane = threadIdx.x & (LPR - 1);
  const int i = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + (threadIdx.x & 31) / LPR;
  const int z = blockIdx.y;
  if (i >= tqp) return;  // whole warps only: tqp is a multiple of 64, a block covers 4 * RPW <= 16 rows
  const long long row = ((long long)z * tqp + i) * tkp;
  const bool drop = p_drop > 0.f;
  const int n = i < tq ? visible_keys(i, tk, k_lens ? k_lens[z / heads] : tk, causal, causal_shift) : 0;
  float v[CHUNKS][8];
  float mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int j0 = c * (LPR * 8) + lane * 8;
    if (j0 < n) {  // at least one visible key in this vector
      unpack8_bf16(*reinterpret_cast<const uint4*>(s + row + j0), v[c]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (j0 + e >= n) v[c][e] = -INFINITY;
        mx = fmaxf(mx, v[c][e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[c][e] = -INFINITY;
    }
  }
  mx = row_max<LPR>(mx);
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[c][e] = (n > 0 && v[c][e] > -INFINITY) ? __expf(v[c][e] - mx) : 0.f;
      sum += v[c][e];
    }
  }
  sum = row_sum<LPR>(sum);
  const float inv = n > 0 ? 1.f / sum : 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0, off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int j0 = c * (LPR * 8) + lane * 8;
    if (j0 >= tkp) continue;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[c][e] *= inv;
    *reinterpret_cast<uint4*>(p + row + j0) = pack8_bf16(v[c]);
    if (drop) {
      const uint32_t keep = j0 < n ? keep_mask8(sd, off + (uint64_t)(row + j0), thresh) : 0u;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[c][e] = (keep >> e) & 1u ? v[c][e] * keep_scale : 0.f;
      *reinterpret_cast<uint4*>(pd + row + j0) = pack8_bf16(v[c]);
    }
  }
}

template <int LPR, int CHUNKS>
__global__ void __launch_bounds__(128)
sdpa_softmax_bwd_vec_kernel(const __nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ dpd, __nv_bfloat16* __restrict__ ds,
                            const int* __restrict__ k_lens, int heads, int tq, int tk, int tqp, int tkp, int causal, int causal_shift,
                            float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  constexpr int RPW = 32 / LPR;  // rows per warp
  const int lane = threadIdx.x & (LPR - 1);
  const int i = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + (threadIdx.x & 31) / LPR;
  const int z = blockIdx.y;
  if (i >= tqp) return;  // whole warps only: tqp is a multiple of 64, a block covers 4 * RPW <= 16 rows
  const long long row = ((long long)z * tqp + i) * tkp;
  const bool drop = p_drop > 0.f;
  const int n = i < tq ? visible_keys(i, tk, k_lens ? k_lens[z / heads] : tk, causal, causal_shift) : 0;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0, off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
  float pv[CHUNKS][8], dv[CHUNKS][8];
  float delta = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int j0 = c * (LPR * 8) + lane * 8;
    if (j0 < n) {
      unpack8_bf16(*reinterpret_cast<const uint4*>(p + row + j0), pv[c]);
      unpack8_bf16(*reinterpret_cast<const uint4*>(dpd + row + j0), dv[c]);
      const uint32_t keep = drop ? keep_mask8(sd, off + (uint64_t)(row + j0), thresh) : 0xffu;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (j0 + e >= n) {
          pv[c][e] = 0.f;
          dv[c][e] = 0.f;
        } else if (drop) {
          dv[c][e] = (keep >> e) & 1u ? dv[c][e] * keep_scale : 0.f;
        }
        delta += pv[c][e] * dv[c][e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) pv[c][e] = dv[c][e] = 0.f;
    }
  }
  delta = row_sum<LPR>(delta);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int j0 = c * (LPR * 8) + lane * 8;
    if (j0 >= tkp) continue;
#pragma unroll
    for (int e = 0; e < 8; ++e) dv[c][e] = pv[c][e] * (dv[c][e] - delta);
    *reinterpret_cast<uint4*>(ds + row + j0) = pack8_bf16(dv[c]);
  }
}

}  // namespace

RB_EXPORT int rb200_sdpa_softmax_fwd(const float* s, void* p, void* pd, const int* k_lens, int batch, int heads, int tq, int tk, int tqp, int tkp,
                                     int causal, int causal_shift, float p_drop, const long long* seed, const long long* offset,
                                     cudaStream_t stream) {
  if (batch <= 0 || tqp <= 0) return RB_OK;
  if (tqp % 64 || tkp % 64 || tq > tqp || tk > tkp || (p_drop > 0.f && (!seed || !offset || !pd || !(p_drop < 1.f)))) {
    rb_set_error("sdpa_softmax_fwd: padded extents must be multiples of 64 (tq %d/%d tk %d/%d); dropout needs seed, offset and pd", tq, tqp, tk, tkp);
    return RB_ERR_ARG;
  }
  dim3 grid((tqp + 3) / 4, batch * heads);
  rb_launch_pdl(sdpa_softmax_fwd_kernel, grid, dim3(128), 0, stream, s, (__nv_bfloat16*)p, (__nv_bfloat16*)pd, k_lens, heads, tq, tk, tqp, tkp, causal,
                causal_shift, p_drop, seed, offset);
  return rb_check_launch("sdpa_softmax_fwd");
}

RB_EXPORT int rb200_sdpa_softmax_bwd(const void* p, const float* dpd, void* ds, const int* k_lens, int batch, int heads, int tq, int tk, int tqp,
                                     int tkp, int causal, int causal_shift, float p_drop, const long long* seed, const long long* offset,
                                     cudaStream_t stream) {
  if (batch <= 0 || tqp <= 0) return RB_OK;
  if (tqp % 64 || tkp % 64 || tq > tqp || tk > tkp || (p_drop > 0.f && (!seed || !offset || !(p_drop < 1.f)))) {
    rb_set_error("sdpa_softmax_bwd: padded extents must be multiples of 64 (tq %d/%d tk %d/%d)", tq, tqp, tk, tkp);
    return RB_ERR_ARG;
  }
  dim3 grid((tqp + 3) / 4, batch * heads);
  rb_launch_pdl(sdpa_softmax_bwd_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)p, dpd, (__nv_bfloat16*)ds, k_lens, heads, tq, tk, tqp, tkp,
                causal, causal_shift, p_drop, seed, offset);
  return rb_check_launch("sdpa_softmax_bwd");
}

// bf16 scores / gradients; rows of at most 1024 (padded) keys
RB_EXPORT int rb200_sdpa_softmax_fwd_bf16(const void* s, void* p, void* pd, const int* k_lens, int batch, int heads, int tq, int tk, int tqp, int tkp,
                                          int causal, int causal_shift, float p_drop, const long long* seed, const long long* offset,
                                          cudaStream_t stream) {
  if (batch <= 0 || tqp <= 0) return RB_OK;
  if (tqp % 64 || tkp % 64 || tkp > kVecMaxKeys || tq > tqp || tk > tkp || (p_drop > 0.f && (!seed || !offset || !pd || !(p_drop < 1.f)))) {
    rb_set_error("sdpa_softmax_fwd_bf16: padded extents must be multiples of 64, keys at most %d (tq %d/%d tk %d/%d); dropout needs seed, offset and pd",
                 kVecMaxKeys, tq, tqp, tk, tkp);
    return RB_ERR_ARG;
  }
#define SDPA_FWD(LPR, CH)                                                                                                                  \
  rb_launch_pdl(sdpa_softmax_fwd_vec_kernel<LPR, CH>, dim3(tqp / (4 * (32 / LPR)), batch * heads), dim3(128), 0, stream, (const __nv_bfloat16*)s, \
                (__nv_bfloat16*)p, (__nv_bfloat16*)pd, k_lens, heads, tq, tk, tqp, tkp, causal, causal_shift, p_drop, seed, offset)
  if (tkp <= 64) SDPA_FWD(8, 1);
  else if (tkp <= 128) SDPA_FWD(16, 1);
  else if (tkp <= 256) SDPA_FWD(32, 1);
  else if (tkp <= 512) SDPA_FWD(32, 2);
  else SDPA_FWD(32, 4);
#undef SDPA_FWD
  return rb_check_launch("sdpa_softmax_fwd_bf16");
}

RB_EXPORT int rb200_sdpa_softmax_bwd_bf16(const void* p, const void* dpd, void* ds, const int* k_lens, int batch, int heads, int tq, int tk, int tqp,
                                          int tkp, int causal, int causal_shift, float p_drop, const long long* seed, const long long* offset,
                                          cudaStream_t stream) {
  if (batch <= 0 || tqp <= 0) return RB_OK;
  if (tqp % 64 || tkp % 64 || tkp > kVecMaxKeys || tq > tqp || tk > tkp || (p_drop > 0.f && (!seed || !offset || !(p_drop < 1.f)))) {
    rb_set_error("sdpa_softmax_bwd_bf16: padded extents must be multiples of 64, keys at most %d (tq %d/%d tk %d/%d)", kVecMaxKeys, tq, tqp, tk, tkp);
    return RB_ERR_ARG;
  }
#define SDPA_BWD(LPR, CH)                                                                                                                  \
  rb_launch_pdl(sdpa_softmax_bwd_vec_kernel<LPR, CH>, dim3(tqp / (4 * (32 / LPR)), batch * heads), dim3(128), 0, stream, (const __nv_bfloat16*)p, \
                (const __nv_bfloat16*)dpd, (__nv_bfloat16*)ds, k_lens, heads, tq, tk, tqp, tkp, causal, causal_shift, p_drop, seed, offset)
  if (tkp <= 64) SDPA_BWD(8, 1);
  else if (tkp <= 128) SDPA_BWD(16, 1);
  else if (tkp <= 256) SDPA_BWD(32, 1);
  else if (tkp <= 512) SDPA_BWD(32, 2);
  else SDPA_BWD(32, 4);
#undef SDPA_BWD
  return rb_check_launch("sdpa_softmax_bwd_bf16");
}
