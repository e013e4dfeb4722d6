// Element-wise kernels on bf16: dropout with a counter-based RNG whose seed and offset live in device memory
// (a CUDA-graph replay reads the current values, so every replay draws a fresh mask and backward re-creates the mask
// of its forward from the saved offset).
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int64_t n, float p,
               const int64_t* __restrict__ seed, const int64_t* __restrict__ offset) {
  const uint64_t sd = (uint64_t)seed[0];
  const uint64_t off = (uint64_t)offset[0];
  const float scale = 1.f / (1.f - p);
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  const int64_t n8 = n & ~(int64_t)7;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n8; i += (int64_t)gridDim.x * blockDim.x * 8) {
    uint64_t c = off + (uint64_t)i;
    uint4 r0 = philox4x32(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), make_uint4((uint32_t)c, (uint32_t)(c >> 32), 0u, 0u));
    uint4 r1 = philox4x32(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), make_uint4((uint32_t)c, (uint32_t)(c >> 32), 1u, 0u));
    uint32_t r[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    F8 a = load8(x, i, 1);
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] = r[k] >= thresh ? a.v[k] * scale : 0.f;
    store8(y, i, a, 1);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n - n8)) {
    int64_t i = n8 + threadIdx.x;
    uint64_t c = off + (uint64_t)n8;
    uint4 r0 = philox4x32(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), make_uint4((uint32_t)c, (uint32_t)(c >> 32), 0u, 0u));
    uint4 r1 = philox4x32(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), make_uint4((uint32_t)c, (uint32_t)(c >> 32), 1u, 0u));
    uint32_t r[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    float v = __bfloat162float(x[i]);
    y[i] = __float2bfloat16(r[threadIdx.x] >= thresh ? v * scale : 0.f);
  }
}

}  // namespace

RB_EXPORT int rb200_dropout_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, float p, const long long* seed,
                                 const long long* offset, cudaStream_t stream) {
  if (n <= 0) return RB_OK;
  if (!(p >= 0.f && p < 1.f)) {
    rb_set_error("dropout: p=%f out of [0,1)", p);
    return RB_ERR_ARG;
  }
  int grid = (int)((n / 8 + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 148 * 8) grid = 148 * 8;
  dropout_kernel<<<grid, 256, 0, stream>>>(x, y, n, p, (const int64_t*)seed, (const int64_t*)offset);
  return rb_check_launch("dropout");
}
