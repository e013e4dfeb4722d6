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
  const uint32_t thresh = rb_dropout_thresh16(p);
  const uint2 key = make_uint2((uint32_t)sd, (uint32_t)(sd >> 32));
  const int64_t n8 = n & ~(int64_t)7;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n8; i += (int64_t)gridDim.x * blockDim.x * 8) {
    F8 a = load8(x, i, 1);
    rb_dropout_apply8(key, off + (uint64_t)i, thresh, scale, a.v);
    store8(y, i, a, 1);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n - n8)) {
    // the last, incomplete group: the same 16-bit values as a complete group starting at n8 would use
    int64_t i = n8 + threadIdx.x;
    const uint4 r = rb_dropout_bits8(key, off + (uint64_t)n8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    const uint32_t bits = (threadIdx.x & 1) ? (w[threadIdx.x >> 1] >> 16) : (w[threadIdx.x >> 1] & 0xFFFFu);
    float v = __bfloat162float(x[i]);
    y[i] = __float2bfloat16(bits >= thresh ? v * scale : 0.f);
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
