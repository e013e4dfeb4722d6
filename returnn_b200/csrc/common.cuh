// Shared device helpers for the sm_100a kernels of returnn_b200.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RB_EXPORT extern "C" __attribute__((visibility("default")))

// status codes returned by every entry point
enum { RB_OK = 0, RB_ERR_ARG = 1, RB_ERR_LAUNCH = 2, RB_ERR_UNSUPPORTED = 3, RB_ERR_TIMEOUT = 4 };

void rb_set_error(const char* fmt, ...);

static inline int rb_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    rb_set_error("%s: %s", what, cudaGetErrorString(e));
    return RB_ERR_LAUNCH;
  }
  return RB_OK;
}

// ---- programmatic dependent launch -----------------------------------------------------------------------------------
// Kernels that follow each other on a stream leave the GPU idle for a few microseconds at every boundary (the last CTAs of
// one drain, then the next is launched). A kernel launched through rb_launch_pdl may be scheduled while its predecessor
// still runs: it does the part of its prologue that touches no global memory, then calls rb_pdl_wait(), which returns once
// the predecessor grid has completed and its writes are visible. Every kernel launched this way MUST call rb_pdl_wait()
// before its first global-memory access; rb_pdl_launch() (right after it) lets the successor start being scheduled in turn.
// Launched the ordinary way, both calls do nothing. RETURNN_B200_PDL=0 turns the attribute off.
__device__ __forceinline__ void rb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rb_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool rb_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t rb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = rb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 8 consecutive elements as floats, from bf16 (16-byte load) or fp32 (two 16-byte loads)
struct F8 {
  float v[8];
};
__device__ __forceinline__ F8 load8(const void* base, int64_t idx, int is_bf16) {
  F8 r;
  if (is_bf16) {
    uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      r.v[2 * i] = f.x;
      r.v[2 * i + 1] = f.y;
    }
  } else {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    float4 a = p[0], b = p[1];
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  }
  return r;
}
__device__ __forceinline__ void store8(void* base, int64_t idx, const F8& r, int is_bf16) {
  if (is_bf16) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(r.v[2 * i], r.v[2 * i + 1]);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = u;
  } else {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx);
    p[0] = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    p[1] = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
  }
}

// counter-based RNG: philox4x32 with ROUNDS rounds, keyed on (seed, counter)
template <int ROUNDS>
__device__ __forceinline__ uint4 philox4x32_rounds(uint2 key, uint4 ctr) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < ROUNDS; ++i) {
    uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ uint4 philox4x32(uint2 key, uint4 ctr) { return philox4x32_rounds<10>(key, ctr); }

// Dropout mask of 8 consecutive elements (a 16-byte group of bf16 values), used alike by every kernel that applies or replays
// the mask of a linear layer's output (GEMM epilogues, the dropout kernels, the column-sum kernel of the backward pass):
// ONE philox4x32-7 call (7 rounds pass the statistical test batteries; the mask needs no more) keyed on the seed, with the
// element offset of the group's first element as counter, gives 128 bits = 16 bits per element. Element i is kept when its 16
// bits are >= thresh16 = floor(p * 65536): the drop probability is p to within 1/65536.
// Returns the 8 random 16-bit values packed as {e0 | e1 << 16, e2 | e3 << 16, ...}.
__device__ __forceinline__ uint4 rb_dropout_bits8(uint2 key, uint64_t counter) {
  return philox4x32_rounds<7>(key, make_uint4((uint32_t)counter, (uint32_t)(counter >> 32), 0xD0u, 0u));
}
__device__ __forceinline__ uint32_t rb_dropout_thresh16(float p) { return (uint32_t)(p * 65536.0f); }
// v[0..7] -> kept values times `scale`, dropped values 0
__device__ __forceinline__ void rb_dropout_apply8(uint2 key, uint64_t counter, uint32_t thresh16, float scale, float* v) {
  const uint4 r = rb_dropout_bits8(key, counter);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = (w[i] & 0xFFFFu) >= thresh16 ? v[2 * i] * scale : 0.f;
    v[2 * i + 1] = (w[i] >> 16) >= thresh16 ? v[2 * i + 1] * scale : 0.f;
  }
}
