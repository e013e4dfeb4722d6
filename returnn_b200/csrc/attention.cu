// Relative-position self-attention on packed sequences: the non-GEMM stages.
//
// The contraction stages (Qu·K^T, Qv·P^T, W·V and the six backward products) run on the batched tcgen05 GEMM
// (gemm_tcgen05.cu) over zero-padded per-sequence buffers; the kernels here do the rest:
//   att_prepare      packed qkv [N, H*3*D] -> padded Qu = q+u, Qv = q+v, K, V  [B*Lp, H*D]
//   att_softmax_fwd  scores = S_ac[i,j] + G[i, j-i+center] (the Transformer-XL shift as an index), masked softmax over the
//                    valid keys, dropout with a replayable counter-based RNG; writes probabilities W and dropped Wd
//   att_softmax_bwd  dS = W * (dW - delta) with the exact delta = sum_j W*dW, and dG = the un-shifted dS
//   att_pack_dqkv    padded dQu+dQv, dK, dV -> packed dqkv [N, H*3*D]
// Row length (keys per query) is limited to 512: one warp holds a row in registers.
#include "common.cuh"

namespace {

__device__ __forceinline__ float score_f(float x) { return x; }
__device__ __forceinline__ float score_f(__nv_bfloat16 x) { return __bfloat162float(x); }

constexpr int kMaxPerLane = 16;  // 32 lanes * 16 = 512 keys

__global__ void __launch_bounds__(256)
att_prepare_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ u, const float* __restrict__ v,
                   const int* __restrict__ row_batch, const int* __restrict__ row_pos, __nv_bfloat16* __restrict__ qu,
                   __nv_bfloat16* __restrict__ qv, __nv_bfloat16* __restrict__ kk, __nv_bfloat16* __restrict__ vv,
                   int n_rows, int heads, int dim, int lp) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  // one thread per 8 consecutive elements of one of q/k/v of one head of one row
  const int groups_per_part = dim / 8;
  const int groups_per_row = heads * 3 * groups_per_part;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_rows * groups_per_row) return;
  const int row = (int)(gid / groups_per_row);
  int g = (int)(gid % groups_per_row);
  const int h = g / (3 * groups_per_part);
  g -= h * 3 * groups_per_part;
  const int part = g / groups_per_part;
  const int d0 = (g % groups_per_part) * 8;
  const int hd = heads * dim;
  F8 x = load8(qkv, (long long)row * 3 * hd + (long long)h * 3 * dim + part * dim + d0, 1);
  const long long dst = ((long long)row_batch[row] * lp + row_pos[row]) * hd + h * dim + d0;
  if (part == 0) {
    F8 a, b;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a.v[i] = x.v[i] + (u ? u[h * dim + d0 + i] : 0.f);
      b.v[i] = x.v[i] + (v ? v[h * dim + d0 + i] : 0.f);
    }
    store8(qu, dst, a, 1);
    store8(qv, dst, b, 1);
  } else if (part == 1) {
    store8(kk, dst, x, 1);
  } else {
    store8(vv, dst, x, 1);
  }
}

__device__ __forceinline__ uint32_t rng_u32(uint64_t seed, uint64_t idx) {
  uint4 r = philox4x32(make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)), make_uint4((uint32_t)(idx >> 2), (uint32_t)(idx >> 34), 0x51u, 0u));
  const uint32_t sel = (uint32_t)(idx & 3);
  return sel == 0 ? r.x : sel == 1 ? r.y : sel == 2 ? r.z : r.w;
}

// grid: (ceil(Lp / warps_per_cta), B*H); one warp per query row
template <typename TS>
__global__ void __launch_bounds__(128)
att_softmax_fwd_kernel(const TS* __restrict__ s_ac, const TS* __restrict__ g, __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ wd, const int* __restrict__ lens, int batch, int heads, int lp, int rp, int center,
                       float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  const int b = z / heads, h = z % heads;
  const int len = lens[b];
  // the GEMMs that consume w / wd contract over rows or columns up to the next multiple of 64: that margin is zeroed here,
  // nothing beyond it is ever read, so the buffers need no memset
  const int len64 = min(lp, (len + 63) & ~63);
  if (i >= len64) return;
  const long long srow = ((long long)z * lp + i) * lp;
  if (i >= len) {
    const __nv_bfloat16 zero = __float2bfloat16(0.f);
    for (int j = lane; j < len64; j += 32) {
      w[srow + j] = zero;
      if (p_drop > 0.f) wd[srow + j] = zero;
    }
    return;
  }
  const long long grow = (((long long)h * batch + b) * lp + i) * rp;
  float x[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int t = 0; t < kMaxPerLane; ++t) {
    const int j = lane + 32 * t;
    if (j < len) {
      x[t] = score_f(s_ac[srow + j]) + score_f(g[grow + (j - i + center)]);
      mx = fmaxf(mx, x[t]);
    } else {
      x[t] = -INFINITY;
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int t = 0; t < kMaxPerLane; ++t) {
    x[t] = (lane + 32 * t < len) ? __expf(x[t] - mx) : 0.f;
    sum += x[t];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  const bool drop = p_drop > 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0;
  const uint64_t off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
#pragma unroll
  for (int t = 0; t < kMaxPerLane; ++t) {
    const int j = lane + 32 * t;
    if (j < len64) {
      const float pr = j < len ? x[t] * inv : 0.f;
      w[srow + j] = __float2bfloat16(pr);
      if (drop) {
        const bool keep = rng_u32(sd, off + (uint64_t)(srow + j)) >= thresh;
        wd[srow + j] = __float2bfloat16(keep ? pr * keep_scale : 0.f);
      }
    }
  }
}

template <typename TS>
__global__ void __launch_bounds__(128)
att_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ w, const TS* __restrict__ dwd, __nv_bfloat16* __restrict__ ds,
                       __nv_bfloat16* __restrict__ dg, const int* __restrict__ lens, int batch, int heads, int lp, int rp, int center,
                       float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  const int b = z / heads, h = z % heads;
  const int len = lens[b];
  const int len64 = min(lp, (len + 63) & ~63);  // see the forward kernel
  if (i >= len64) return;
  const long long srow = ((long long)z * lp + i) * lp;
  if (i >= len) {
    for (int j = lane; j < len64; j += 32) ds[srow + j] = __float2bfloat16(0.f);
    return;
  }
  const long long grow = (((long long)h * batch + b) * lp + i) * rp;
  const bool drop = p_drop > 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0;
  const uint64_t off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
  float pw[kMaxPerLane], dw[kMaxPerLane];
  float delta = 0.f;
#pragma unroll
  for (int t = 0; t < kMaxPerLane; ++t) {
    const int j = lane + 32 * t;
    if (j < len) {
      pw[t] = __bfloat162float(w[srow + j]);
      float d = score_f(dwd[srow + j]);
      if (drop) d = (rng_u32(sd, off + (uint64_t)(srow + j)) >= thresh) ? d * keep_scale : 0.f;
      dw[t] = d;
      delta += pw[t] * d;
    } else {
      pw[t] = 0.f;
      dw[t] = 0.f;
    }
  }
  delta = warp_sum(delta);
#pragma unroll
  for (int t = 0; t < kMaxPerLane; ++t) {
    const int j = lane + 32 * t;
    if (j < len) {
      const __nv_bfloat16 o = __float2bfloat16(pw[t] * (dw[t] - delta));
      ds[srow + j] = o;
      dg[grow + (j - i + center)] = o;
    } else if (j < len64) {
      ds[srow + j] = __float2bfloat16(0.f);
    }
  }
}

// ---- bf16-score versions with 16-byte accesses: a lane owns 8 consecutive keys per step (two steps cover 512 keys), one
// philox call serves 4 keys (the scalar kernels above draw one per key and use a quarter of it). Same arithmetic, same dropout
// counters, so forward and backward (and the scalar kernels) agree on the mask.
__device__ __forceinline__ void rng8(uint64_t seed, uint64_t idx0, uint32_t (&r)[8]) {
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const uint64_t b0 = idx0 >> 2;  // idx0 is a multiple of 8
  const uint4 a = philox4x32(key, make_uint4((uint32_t)b0, (uint32_t)(b0 >> 32), 0x51u, 0u));
  const uint4 b = philox4x32(key, make_uint4((uint32_t)(b0 + 1), (uint32_t)((b0 + 1) >> 32), 0x51u, 0u));
  r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w; r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 p = __bfloat1622float2(h[q]);
    f[2 * q] = p.x;
    f[2 * q + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
  return u;
}

constexpr int kVecSteps = 2;  // 2 * 32 lanes * 8 keys = 512

__global__ void __launch_bounds__(128)
att_softmax_fwd_vec_kernel(const __nv_bfloat16* __restrict__ s_ac, const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ w,
                           __nv_bfloat16* __restrict__ wd, const int* __restrict__ lens, int batch, int heads, int lp, int rp, int center,
                           float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  const int b = z / heads, h = z % heads;
  const int len = lens[b];
  const int len64 = min(lp, (len + 63) & ~63);
  if (i >= len64) return;
  const long long srow = ((long long)z * lp + i) * lp;
  const bool drop = p_drop > 0.f;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  if (i >= len) {
    for (int j0 = lane * 8; j0 < len64; j0 += 256) {
      *reinterpret_cast<uint4*>(w + srow + j0) = zero4;
      if (drop) *reinterpret_cast<uint4*>(wd + srow + j0) = zero4;
    }
    return;
  }
  const long long grow = (((long long)h * batch + b) * lp + i) * rp + (center - i);
  float x[kVecSteps][8];
  float mx = -INFINITY;
#pragma unroll
  for (int t = 0; t < kVecSteps; ++t) {
    const int j0 = (t * 32 + lane) * 8;
    if (j0 < len) {
      float a[8];
      unpack8(*reinterpret_cast<const uint4*>(s_ac + srow + j0), a);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int j = j0 + e;
        x[t][e] = j < len ? a[e] + __bfloat162float(g[grow + j]) : -INFINITY;
        mx = fmaxf(mx, x[t][e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[t][e] = -INFINITY;
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int t = 0; t < kVecSteps; ++t)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      x[t][e] = x[t][e] > -INFINITY ? __expf(x[t][e] - mx) : 0.f;
      sum += x[t][e];
    }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0;
  const uint64_t off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
#pragma unroll
  for (int t = 0; t < kVecSteps; ++t) {
    const int j0 = (t * 32 + lane) * 8;
    if (j0 < len64) {
      float pr[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) pr[e] = x[t][e] * inv;  // zero beyond len
      *reinterpret_cast<uint4*>(w + srow + j0) = pack8(pr);
      if (drop) {
        uint32_t r[8];
        rng8(sd, off + (uint64_t)(srow + j0), r);
#pragma unroll
        for (int e = 0; e < 8; ++e) pr[e] = r[e] >= thresh ? pr[e] * keep_scale : 0.f;
        *reinterpret_cast<uint4*>(wd + srow + j0) = pack8(pr);
      }
    }
  }
}

__global__ void __launch_bounds__(128)
att_softmax_bwd_vec_kernel(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dwd, __nv_bfloat16* __restrict__ ds,
                           __nv_bfloat16* __restrict__ dg, const int* __restrict__ lens, int batch, int heads, int lp, int rp, int center,
                           float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  rb_pdl_wait();
  rb_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  const int b = z / heads, h = z % heads;
  const int len = lens[b];
  const int len64 = min(lp, (len + 63) & ~63);
  if (i >= len64) return;
  const long long srow = ((long long)z * lp + i) * lp;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  if (i >= len) {
    for (int j0 = lane * 8; j0 < len64; j0 += 256) *reinterpret_cast<uint4*>(ds + srow + j0) = zero4;
    return;
  }
  const long long grow = (((long long)h * batch + b) * lp + i) * rp + (center - i);
  const bool drop = p_drop > 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0;
  const uint64_t off = drop ? (uint64_t)offset[0] : 0;
  const uint32_t thresh = drop ? (uint32_t)(p_drop * 4294967296.0) : 0u;
  const float keep_scale = drop ? 1.f / (1.f - p_drop) : 1.f;
  float pw[kVecSteps][8], dw[kVecSteps][8];
  float delta = 0.f;
#pragma unroll
  for (int t = 0; t < kVecSteps; ++t) {
    const int j0 = (t * 32 + lane) * 8;
    if (j0 < len) {
      unpack8(*reinterpret_cast<const uint4*>(w + srow + j0), pw[t]);
      unpack8(*reinterpret_cast<const uint4*>(dwd + srow + j0), dw[t]);
      uint32_t r[8];
      if (drop) rng8(sd, off + (uint64_t)(srow + j0), r);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (j0 + e >= len) {
          pw[t][e] = 0.f;
          dw[t][e] = 0.f;
        } else if (drop) {
          dw[t][e] = r[e] >= thresh ? dw[t][e] * keep_scale : 0.f;
        }
        delta += pw[t][e] * dw[t][e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) pw[t][e] = dw[t][e] = 0.f;
    }
  }
  delta = warp_sum(delta);
#pragma unroll
  for (int t = 0; t < kVecSteps; ++t) {
    const int j0 = (t * 32 + lane) * 8;
    if (j0 < len64) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = pw[t][e] * (dw[t][e] - delta);  // zero beyond len
      const uint4 packed = pack8(o);
      *reinterpret_cast<uint4*>(ds + srow + j0) = packed;
      const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(&packed);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (j0 + e < len) dg[grow + j0 + e] = ob[e];
    }
  }
}

// wd = dropout(w) with the mask of the forward pass (same seed, same offset)
__global__ void __launch_bounds__(128)
att_redrop_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ wd, const int* __restrict__ lens, int heads, int lp,
                  float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int z = blockIdx.y;
  const int len = lens[z / heads];
  if (i >= len) return;
  const long long srow = ((long long)z * lp + i) * lp;
  const uint64_t sd = (uint64_t)seed[0], off = (uint64_t)offset[0];
  const uint32_t thresh = (uint32_t)(p_drop * 4294967296.0);
  const float keep_scale = 1.f / (1.f - p_drop);
  for (int j = lane; j < len; j += 32) {
    const bool keep = rng_u32(sd, off + (uint64_t)(srow + j)) >= thresh;
    wd[srow + j] = __float2bfloat16(keep ? __bfloat162float(w[srow + j]) * keep_scale : 0.f);
  }
}

__global__ void __launch_bounds__(256)
att_pack_dqkv_kernel(const __nv_bfloat16* __restrict__ dqu, const __nv_bfloat16* __restrict__ dqv, const __nv_bfloat16* __restrict__ dk,
                     const __nv_bfloat16* __restrict__ dv, const int* __restrict__ row_batch, const int* __restrict__ row_pos,
                     __nv_bfloat16* __restrict__ dqkv, int n_rows, int heads, int dim, int lp) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const int groups_per_part = dim / 8;
  const int groups_per_row = heads * 3 * groups_per_part;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_rows * groups_per_row) return;
  const int row = (int)(gid / groups_per_row);
  int g = (int)(gid % groups_per_row);
  const int h = g / (3 * groups_per_part);
  g -= h * 3 * groups_per_part;
  const int part = g / groups_per_part;
  const int d0 = (g % groups_per_part) * 8;
  const int hd = heads * dim;
  const long long src = ((long long)row_batch[row] * lp + row_pos[row]) * hd + h * dim + d0;
  F8 x;
  if (part == 0) {
    F8 a = load8(dqu, src, 1), b = load8(dqv, src, 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) x.v[i] = a.v[i] + b.v[i];
  } else if (part == 1) {
    x = load8(dk, src, 1);
  } else {
    x = load8(dv, src, 1);
  }
  store8(dqkv, (long long)row * 3 * hd + (long long)h * 3 * dim + part * dim + d0, x, 1);
}

// rows [B*Lp, HD] padded <-> packed [N, HD]
__global__ void __launch_bounds__(256)
att_rows_gather_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, const int* __restrict__ row_batch,
                       const int* __restrict__ row_pos, int n_rows, int width, int lp, int to_padded) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  const int groups = width / 8;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_rows * groups) return;
  const int row = (int)(gid / groups);
  const int c0 = (int)(gid % groups) * 8;
  const long long padded = ((long long)row_batch[row] * lp + row_pos[row]) * width + c0;
  const long long packed = (long long)row * width + c0;
  if (to_padded) store8(dst, padded, load8(src, packed, 1), 1);
  else store8(dst, packed, load8(src, padded, 1), 1);
}

}  // namespace

RB_EXPORT int rb200_att_prepare(const void* qkv, const float* u, const float* v, const int* row_batch, const int* row_pos, void* qu,
                                void* qv, void* k, void* vv, int n_rows, int heads, int dim, int lp, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  if (dim % 8) {
    rb_set_error("att_prepare: head dim %d must be a multiple of 8", dim);
    return RB_ERR_ARG;
  }
  long long total = (long long)n_rows * heads * 3 * (dim / 8);
  rb_launch_pdl(att_prepare_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 
      (const __nv_bfloat16*)qkv, u, v, row_batch, row_pos, (__nv_bfloat16*)qu, (__nv_bfloat16*)qv, (__nv_bfloat16*)k, (__nv_bfloat16*)vv,
      n_rows, heads, dim, lp);
  return rb_check_launch("att_prepare");
}

// scores_bf16: s_ac and g are bf16 (what the batched GEMMs write on the training path) instead of fp32
RB_EXPORT int rb200_att_softmax_fwd_ex(const void* s_ac, const void* g, int scores_bf16, void* w, void* wd, const int* lens, int batch, int heads,
                                       int lp, int rp, int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream) {
  if (lp > 32 * kMaxPerLane) {
    rb_set_error("att_softmax: padded length %d > %d", lp, 32 * kMaxPerLane);
    return RB_ERR_UNSUPPORTED;
  }
  dim3 grid((lp + 3) / 4, batch * heads);
  if (scores_bf16 && lp <= 512 && lp % 64 == 0 && rp % 8 == 0)
    rb_launch_pdl(att_softmax_fwd_vec_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)s_ac, (const __nv_bfloat16*)g, (__nv_bfloat16*)w,
                  (__nv_bfloat16*)wd, lens, batch, heads, lp, rp, center, p_drop, seed, offset);
  else if (scores_bf16)
    rb_launch_pdl(att_softmax_fwd_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, stream, (const __nv_bfloat16*)s_ac, (const __nv_bfloat16*)g, (__nv_bfloat16*)w,
                                                                    (__nv_bfloat16*)wd, lens, batch, heads, lp, rp, center, p_drop, seed, offset);
  else
  rb_launch_pdl(att_softmax_fwd_kernel<float>, dim3(grid), dim3(128), 0, stream, (const float*)s_ac, (const float*)g, (__nv_bfloat16*)w, (__nv_bfloat16*)wd, lens, batch, heads, lp, rp, center, p_drop,
                                                   seed, offset);
  return rb_check_launch("att_softmax_fwd");
}

RB_EXPORT int rb200_att_softmax_bwd_ex(const void* w, const void* dwd, int dwd_bf16, void* ds, void* dg, const int* lens, int batch, int heads, int lp,
                                       int rp, int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream) {
  if (lp > 32 * kMaxPerLane) return RB_ERR_UNSUPPORTED;
  dim3 grid((lp + 3) / 4, batch * heads);
  if (dwd_bf16 && lp <= 512 && lp % 64 == 0 && rp % 8 == 0)
    rb_launch_pdl(att_softmax_bwd_vec_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dwd, (__nv_bfloat16*)ds,
                  (__nv_bfloat16*)dg, lens, batch, heads, lp, rp, center, p_drop, seed, offset);
  else if (dwd_bf16)
    rb_launch_pdl(att_softmax_bwd_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, stream, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dwd, (__nv_bfloat16*)ds,
                                                                    (__nv_bfloat16*)dg, lens, batch, heads, lp, rp, center, p_drop, seed, offset);
  else
    rb_launch_pdl(att_softmax_bwd_kernel<float>, dim3(grid), dim3(128), 0, stream, (const __nv_bfloat16*)w, (const float*)dwd, (__nv_bfloat16*)ds, (__nv_bfloat16*)dg, lens,
                                                            batch, heads, lp, rp, center, p_drop, seed, offset);
  return rb_check_launch("att_softmax_bwd");
}

RB_EXPORT int rb200_att_softmax_fwd(const float* s_ac, const float* g, void* w, void* wd, const int* lens, int batch, int heads, int lp, int rp,
                                    int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream) {
  return rb200_att_softmax_fwd_ex(s_ac, g, 0, w, wd, lens, batch, heads, lp, rp, center, p_drop, seed, offset, stream);
}

RB_EXPORT int rb200_att_softmax_bwd(const void* w, const float* dwd, void* ds, void* dg, const int* lens, int batch, int heads, int lp, int rp,
                                    int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream) {
  return rb200_att_softmax_bwd_ex(w, dwd, 0, ds, dg, lens, batch, heads, lp, rp, center, p_drop, seed, offset, stream);
}

RB_EXPORT int rb200_att_redrop(const void* w, void* wd, const int* lens, int batch, int heads, int lp, float p_drop, const long long* seed,
                               const long long* offset, cudaStream_t stream) {
  dim3 grid((lp + 3) / 4, batch * heads);
  att_redrop_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)wd, lens, heads, lp, p_drop, seed, offset);
  return rb_check_launch("att_redrop");
}

RB_EXPORT int rb200_att_pack_dqkv(const void* dqu, const void* dqv, const void* dk, const void* dv, const int* row_batch, const int* row_pos,
                                  void* dqkv, int n_rows, int heads, int dim, int lp, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  long long total = (long long)n_rows * heads * 3 * (dim / 8);
  rb_launch_pdl(att_pack_dqkv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 
      (const __nv_bfloat16*)dqu, (const __nv_bfloat16*)dqv, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, row_batch, row_pos,
      (__nv_bfloat16*)dqkv, n_rows, heads, dim, lp);
  return rb_check_launch("att_pack_dqkv");
}

RB_EXPORT int rb200_att_rows_gather(const void* src, void* dst, const int* row_batch, const int* row_pos, int n_rows, int width, int lp,
                                    int to_padded, cudaStream_t stream) {
  if (n_rows <= 0) return RB_OK;
  if (width % 8) return RB_ERR_ARG;
  long long total = (long long)n_rows * (width / 8);
  rb_launch_pdl(att_rows_gather_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, row_batch, row_pos,
                                                                              n_rows, width, lp, to_padded);
  return rb_check_launch("att_rows_gather");
}
