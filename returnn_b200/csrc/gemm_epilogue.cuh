// Epilogue and work-unit decoding shared by the persistent tcgen05 GEMM kernels (one-CTA and CTA-pair variants).
#pragma once
#include "tcgen05.cuh"
#include "gemm.h"

namespace rbg {

using namespace rbt;

constexpr int BK = 64;

struct Params {
  RbGemm g;
  int tiles_m, tiles_n, split, kb_per_split, num_kb, units;
  int vec_ok;    // all epilogue pointers 16-byte aligned and ldc % 8 == 0
  int bias_vec;  // fp32 bias, 16-byte aligned: read as two float4
  int tma_store; // the output leaves through shared memory and bulk tensor stores (tensor maps of c / c2 passed to the kernel)
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float act_grad(float z, int act) {
  if (act == 1) return z > 0.f ? 1.f : 0.f;
  if (act == 2) {
    float s = __fdividef(1.f, 1.f + __expf(-z));
    return s * (1.f + z * (1.f - s));
  }
  if (act == 3) {
    float cdf = 0.5f * (1.f + erff(z * 0.70710678118654752f));
    float pdf = __expf(-0.5f * z * z) * 0.3989422804014327f;
    return cdf + z * pdf;
  }
  return 1.f;
}

// The activation (or its derivative) on 8 values. The kind is uniform over the kernel: it is tested ONCE per group, outside the
// element loops, so that the cheap kinds do not carry the instructions of the expensive one (erf) as predicated code.
__device__ __forceinline__ float silu_tanh(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return x * (0.5f + 0.5f * t);  // x * sigmoid(x), sigmoid(x) = (1 + tanh(x / 2)) / 2: one special-function instruction
}
__device__ __forceinline__ void act8(float* v, int act) {
  if (act == 2) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = silu_tanh(v[i]);
  } else if (act == 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.f);
  } else if (act == 3) {
#pragma unroll  // no rolled loop here: a dynamically indexed v[] would move the array, for every kind, from registers to local memory
    for (int i = 0; i < 8; ++i) v[i] = 0.5f * v[i] * (1.f + erff(v[i] * 0.70710678118654752f));
  }
}
__device__ __forceinline__ void act_grad8(float* v, const float* z, int act) {
  if (act == 2) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * z[i]));
      const float s = 0.5f + 0.5f * t;
      v[i] *= s * (1.f + z[i] * (1.f - s));
    }
  } else if (act == 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = z[i] > 0.f ? v[i] : 0.f;
  } else if (act == 3) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= act_grad(z[i], 3);
  }
}

__device__ __forceinline__ void load8_bf16(const void* base, size_t off, bool vec, int nvalid, float* out) {
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(base) + off;
  if (vec) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = i < nvalid ? __bfloat162float(p[i]) : 0.f;
  }
}

__device__ __forceinline__ void store8_bf16(void* base, size_t off, bool vec, int nvalid, const float* v) {
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(base) + off;
  if (vec) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < nvalid) p[i] = __float2bfloat16(v[i]);
  }
}

// one lane's share of the epilogue: 8 consecutive columns [col, col+8) of one output row.
// FULL = false compiles the common case only (scale, bias, activation, store): no activation gradient, dropout or residual,
// which keeps the instruction stream of the epilogue warps short.
template <bool FULL>
__device__ __forceinline__ void epilogue_group(const Params& p, int row, int col, int n_extent, size_t c_off, float* v) {
  const RbGemm& g = p.g;
  const int nvalid = min(8, n_extent - col);
  const bool vec = p.vec_ok && nvalid == 8 && (c_off & 7) == 0;
  const size_t off = c_off + (size_t)row * g.ldc + col;
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= g.alpha;
  if (g.bias && p.bias_vec && nvalid == 8) {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g.bias) + col));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g.bias) + col) + 1);
    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
    v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
  } else if (g.bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < nvalid) {
        v[i] += g.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g.bias)[col + i])
                            : __ldg(reinterpret_cast<const float*>(g.bias) + col + i);
      }
    }
  }
  float pre[8];
  if (FULL && g.dact_z) {
    float z[8];
    load8_bf16(g.dact_z, off, vec, nvalid, z);
    act_grad8(v, z, g.act);
  } else if (g.act) {
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = v[i];
    act8(v, g.act);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = v[i];
  }
  if (FULL && g.drop_p > 0.f) {
    const uint64_t sd = (uint64_t)g.seed[0];
    const uint64_t c = (uint64_t)g.offset[0] + g.drop_site + (uint64_t)off;
    rb_dropout_apply8(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), c, rb_dropout_thresh16(g.drop_p), 1.f / (1.f - g.drop_p), v);
  }
  if (FULL && g.resid) {
    float rs[8];
    load8_bf16(g.resid, off, vec, nvalid, rs);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = rs[i] + g.res_scale * v[i];
  }
  if (g.out_fp32) {
    float* c = reinterpret_cast<float*>(g.c) + off;
    if (g.accumulate == 2) {
      if (vec) {
        atomicAdd(reinterpret_cast<float4*>(c), make_float4(v[0], v[1], v[2], v[3]));
        atomicAdd(reinterpret_cast<float4*>(c) + 1, make_float4(v[4], v[5], v[6], v[7]));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < nvalid) atomicAdd(c + i, v[i]);
      }
    } else if (vec) {
      float4 a = make_float4(v[0], v[1], v[2], v[3]), b = make_float4(v[4], v[5], v[6], v[7]);
      if (g.accumulate == 1) {
        float4 oa = reinterpret_cast<float4*>(c)[0], ob = reinterpret_cast<float4*>(c)[1];
        a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
        b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
      }
      reinterpret_cast<float4*>(c)[0] = a;
      reinterpret_cast<float4*>(c)[1] = b;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < nvalid) c[i] = g.accumulate == 1 ? c[i] + v[i] : v[i];
    }
  } else if (g.c2) {
    store8_bf16(g.c, off, vec, nvalid, pre);
    store8_bf16(g.c2, off, vec, nvalid, v);
  } else {
    store8_bf16(g.c, off, vec, nvalid, v);
  }
}

// one work unit: output tile (m0, n0) of problem z, K blocks [kb0, kb1)
struct Unit {
  int m0, n0, kb0, kb1, M, N;
  int a_r0, a_c0, b_r0, b_c0;
  size_t c_off;
  bool valid;
};

template <int BM, int BN>
__device__ __forceinline__ Unit decode_unit(const Params& p, int u) {
  const RbGemm& g = p.g;
  Unit w;
  const int tiles = p.tiles_m * p.tiles_n;
  if (g.batch > 0) {
    const int z = u / tiles, t = u % tiles;
    const int zb = z / g.heads, zh = z % g.heads;
    const int len = g.lens ? g.lens[zb] : 0;
    w.M = g.m_from_lens ? len : g.m;
    w.N = g.n_from_lens ? len : g.n;
    const int K = g.k_from_lens ? len : g.k;
    w.m0 = (t / p.tiles_n) * BM;
    w.n0 = (t % p.tiles_n) * BN;
    w.kb0 = 0;
    w.kb1 = K > 0 ? (K + BK - 1) / BK : 0;
    w.a_r0 = (int)(zb * g.a_rb + zh * g.a_rh); w.a_c0 = (int)(zb * g.a_cb + zh * g.a_ch);
    w.b_r0 = (int)(zb * g.b_rb + zh * g.b_rh); w.b_c0 = (int)(zb * g.b_cb + zh * g.b_ch);
    w.c_off = (size_t)zb * g.c_sb + (size_t)zh * g.c_sh;
    w.valid = w.m0 < w.M && w.n0 < w.N && w.kb1 > 0;
  } else {
    const int sp = u / tiles, t = u % tiles;
    w.M = g.m; w.N = g.n;
    w.m0 = (t / p.tiles_n) * BM;
    w.n0 = (t % p.tiles_n) * BN;
    w.kb0 = sp * p.kb_per_split;
    w.kb1 = min(p.num_kb, w.kb0 + p.kb_per_split);
    w.a_r0 = w.a_c0 = w.b_r0 = w.b_c0 = 0;
    w.c_off = 0;
    w.valid = true;
  }
  return w;
}

// Epilogue of the accumulator columns [c_begin, c_end) of one 128-row tile by one warp (TMEM lane quarter q), in chunks of 16
// columns: tcgen05.ld -> registers -> this warp's 2 KB staging area (fp32 rows of 64 bytes, 16-byte chunk index xor-swizzled with
// the row so that neither direction has bank conflicts) -> every lane owns 8 consecutive columns of one row -> epilogue_group.
// `arrive` is called by lane 0 once the warp's last read of the accumulator has completed (hands the TMEM buffer back to the
// MMA issuer). Many narrow warps rather than few wide ones: the epilogue is latency-bound per warp (measured about 6 stall
// cycles per issued instruction), so its throughput scales with the number of warps the schedulers can switch between.
template <bool FULL, typename Arrive>
__device__ __forceinline__ void epilogue_columns(const Params& p, const Unit& w, int m0, int n0, uint32_t t_addr, int c_begin, int c_end, float* stg,
                                                 int lane, int q, Arrive arrive) {
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 16) {
    uint32_t r[16];
    tmem_ld16(t_addr + (uint32_t)c0, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (c0 + 16 >= c_end) {
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) arrive();
    }
    float4* srow = reinterpret_cast<float4*>(stg + lane * 16);
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      srow[j ^ sw] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
    }
    __syncwarp();
    const int cg = lane & 1;
    const int col = n0 + c0 + cg * 8;
#pragma unroll
    for (int itr = 0; itr < 2; ++itr) {
      const int rl = itr * 16 + (lane >> 1);
      const int row = m0 + q * 32 + rl;
      const float4* rrow = reinterpret_cast<const float4*>(stg + rl * 16);
      const int sr = (rl >> 1) & 3;
      const float4 a = rrow[(2 * cg) ^ sr], b = rrow[(2 * cg + 1) ^ sr];
      if (row < w.M && col < w.N) {
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        epilogue_group<FULL>(p, row, col, w.N, w.c_off, v);
      }
    }
    __syncwarp();
  }
}

// ---- row-owner epilogue with bulk tensor stores ---------------------------------------------------------------------------------
// Every lane owns ONE accumulator row (TMEM lane = row) and reads W consecutive columns of it with one or two tcgen05.ld.x32, so
// the accumulator buffer is handed back to the MMA issuer as soon as the values are in registers. Bias, activation, activation
// gradient, dropout and residual are computed on groups of 8 consecutive columns (the same grouping and dropout counters as
// epilogue_group). The results go to this warp's 4 KB box in shared memory in the swizzled layout of the output tensor map (rows
// of 128 bytes: 64 bf16 or 32 fp32 columns; 16-byte chunk j of row r sits at chunk position j ^ (r & 7), which also keeps the
// 32 lanes' 16-byte writes on distinct banks), and ONE bulk tensor store (or bulk reduce-add for accumulate != 0) per box moves
// them to global memory: full-line writes, no st.global from the warps, rows and columns outside the matrix clipped by the TMA
// unit. The next box is written only after the previous store has finished reading shared memory (wait_group.read).

// v[8] (accumulator values of columns col .. col+7 of `row`) -> final values in v, pre-activation in pre. Loads of dact_z / resid
// only for valid elements. Same order of operations as epilogue_group.
__device__ __forceinline__ void unpack8_bf16(const uint4& u, float* out) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// The epilogue's global input (dact_z if there is one, else resid) for the 16 columns col0 .. col0+15 of `row`, fetched into
// registers one phase ahead of its use: the first phase BEFORE the warp waits for the accumulator (the loads are in flight while
// the MMAs of the tile still run), every later phase before the arithmetic of the phase before it. Groups that are not completely
// inside the matrix are left to the in-line path of epilogue_math8 (their slot stays zero and is not used).
__device__ __forceinline__ void epilogue_prefetch16(const Params& p, int M, int N, int row, int col0, uint4& a, uint4& b) {
  const RbGemm& g = p.g;
  const void* src = g.dact_z ? g.dact_z : g.resid;
  a = make_uint4(0u, 0u, 0u, 0u);
  b = a;
  if (src == nullptr || row >= M) return;
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(src) + (size_t)row * g.ldc + col0;
  if (col0 + 8 <= N) a = *reinterpret_cast<const uint4*>(base);
  if (col0 + 16 <= N) b = *reinterpret_cast<const uint4*>(base + 8);
}

// in8 / in_valid: the group's prefetched input (see epilogue_prefetch_half), passed by value so that it stays in registers
template <bool FULL>
__device__ __forceinline__ void epilogue_math8(const Params& p, int row, int col, bool row_ok, int n_extent, float* v, float* pre,
                                               const uint4 in8 = make_uint4(0u, 0u, 0u, 0u), bool in_valid = false) {
  const RbGemm& g = p.g;
  const int nvalid = row_ok ? max(0, min(8, n_extent - col)) : 0;
  const bool have_in = FULL && in_valid && nvalid == 8;
  const size_t off = (size_t)row * g.ldc + col;
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= g.alpha;
  if (g.bias && nvalid == 8) {
    if (p.bias_vec) {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g.bias) + col));
      const float4 b1 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g.bias) + col) + 1);
      v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
      v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] += g.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g.bias)[col + i])
                            : __ldg(reinterpret_cast<const float*>(g.bias) + col + i);
      }
    }
  } else if (g.bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < nvalid) {
        v[i] += g.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g.bias)[col + i])
                            : __ldg(reinterpret_cast<const float*>(g.bias) + col + i);
      }
    }
  }
  if (FULL && g.dact_z) {
    float z[8];
    if (have_in) unpack8_bf16(in8, z);
    else load8_bf16(g.dact_z, off, nvalid == 8, nvalid, z);
    act_grad8(v, z, g.act);
  } else if (g.act) {
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = v[i];
    act8(v, g.act);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = v[i];
  }
  if (FULL && g.drop_p > 0.f) {
    const uint64_t sd = (uint64_t)g.seed[0];
    const uint64_t c = (uint64_t)g.offset[0] + g.drop_site + (uint64_t)off;
    rb_dropout_apply8(make_uint2((uint32_t)sd, (uint32_t)(sd >> 32)), c, rb_dropout_thresh16(g.drop_p), 1.f / (1.f - g.drop_p), v);
  }
  if (FULL && g.resid) {
    float rs[8];
    if (have_in && g.dact_z == nullptr) unpack8_bf16(in8, rs);
    else load8_bf16(g.resid, off, nvalid == 8, nvalid, rs);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = rs[i] + g.res_scale * v[i];
  }
}

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

// One warp's share of a tile: rows m0 + q*32 .. +31 (lane = row), accumulator columns [c_begin, c_begin + 64) at TMEM address
// t_addr (lane quarter already applied). box: this warp's 4 KB of shared memory, 1024-byte aligned. tm_c / tm_c2: tensor maps of the
// outputs with boxes of 32 rows x 128 bytes (64 bf16 or 32 fp32 columns; with a second output c2: 32 rows x 64 bytes, 64-byte swizzle). `arrive` hands the accumulator buffer back (lane 0).
// One warp's share of a tile in four phases of 16 columns (a rolled loop: the body is small enough to stay in the instruction
// cache, which an unrolled 64-column body is not; with 16 warps walking through it once per tile, instruction fetch was the
// largest stall reason of the unrolled form). A phase: tcgen05.ld of 16 accumulator values, request of the NEXT phase's global
// input (full epilogue), arithmetic on two groups of 8 columns, 16-byte writes into the box. The accumulator buffer is released
// after the last phase's tcgen05.ld. A box is handed to the TMA unit when it is complete: after 64 bf16 columns (one output),
// after 32 columns for fp32 outputs and for two outputs (then a pair of boxes with 64-byte rows, 64-byte swizzle: chunk j of row r
// at position j ^ ((r >> 1) & 3)), and it is written again only after that store has finished reading it.
// in_a / in_b: the prefetched input of phase 0 (valid if have_in).
template <bool FULL, typename Arrive>
__device__ __forceinline__ void epilogue_rows_tma(const Params& p, const Unit& w, int m0, int n0, uint32_t t_addr, int c_begin, uint8_t* box,
                                                  const CUtensorMap* tm_c, const CUtensorMap* tm_c2, int lane, int q, Arrive arrive,
                                                  uint4 in_a, uint4 in_b, bool have_in) {
  const RbGemm& g = p.g;
  const int row0 = m0 + q * 32;
  const int row = row0 + lane;
  const bool row_ok = row < w.M;
  const int col0 = n0 + c_begin;
  auto release = [&]() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) arrive();
  };
  if (row0 >= w.M || col0 >= w.N) {  // nothing of this warp's box lies inside the matrix (warp-uniform): nothing to read
    release();
    return;
  }
  const bool two_out = g.c2 != nullptr;
  const bool fp32 = g.out_fp32 != 0;
  const bool half_boxes = two_out || fp32;  // a box (or pair of boxes) is complete after 32 columns
  uint8_t* my_row = box + lane * 128;
  uint8_t* row_pre = box + lane * 64;
  uint8_t* row_fin = box + 2048 + lane * 64;
  const int sw = lane & 7, sw64 = (lane >> 1) & 3;
#pragma unroll 1
  for (int ph = 0; ph < 4; ++ph) {
    uint32_t r[16];
    tmem_ld16(t_addr + (uint32_t)(c_begin + 16 * ph), r);
    uint4 nx_a = make_uint4(0u, 0u, 0u, 0u), nx_b = nx_a;
    if (FULL && ph < 3 && have_in) epilogue_prefetch16(p, w.M, w.N, row, col0 + 16 * (ph + 1), nx_a, nx_b);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (ph == 3) release();
    if (ph == 0 || (half_boxes && ph == 2)) {
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
    }
    const bool cols_in = col0 + 16 * ph < w.N;
#pragma unroll
    for (int gi = 0; gi < 2; ++gi) {
      float v[8], pre[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[8 * gi + i]);
      epilogue_math8<FULL>(p, row, col0 + 16 * ph + 8 * gi, row_ok && cols_in, w.N, v, pre, gi == 0 ? in_a : in_b, have_in);
      if (fp32) {
        const int c8 = 4 * (ph & 1) + 2 * gi;  // 16-byte chunk within the 32-column box
        *reinterpret_cast<float4*>(my_row + ((c8 ^ sw) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(my_row + (((c8 + 1) ^ sw) << 4)) = make_float4(v[4], v[5], v[6], v[7]);
      } else if (two_out) {
        const int c4 = 2 * (ph & 1) + gi;
        *reinterpret_cast<uint4*>(row_pre + ((c4 ^ sw64) << 4)) = pack8_bf16(pre);
        *reinterpret_cast<uint4*>(row_fin + ((c4 ^ sw64) << 4)) = pack8_bf16(v);
      } else {
        *reinterpret_cast<uint4*>(my_row + (((2 * ph + gi) ^ sw) << 4)) = pack8_bf16(v);
      }
    }
    in_a = nx_a;
    in_b = nx_b;
    if (ph == 3 || (half_boxes && ph == 1)) {
      const int cbox = half_boxes ? col0 + 32 * (ph >> 1) : col0;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && cbox < w.N) {
        if (fp32 && g.accumulate) {
          tma_reduce_add_2d(tm_c, cbox, row0, box);
        } else {
          tma_store_2d(tm_c, cbox, row0, box);
          if (two_out) tma_store_2d(tm_c2, cbox, row0, box + 2048);
        }
        tma_store_commit();
      }
    }
  }
}

constexpr int kEpilogueWarps = 16;                        // four per TMEM lane quarter: each takes a quarter of the tile's columns
constexpr int kGemmThreads = 64 + kEpilogueWarps * 32;    // + TMA producer warp + MMA warp
constexpr int kStagingBytesPerWarp = 32 * 16 * 4;
constexpr int kStoreBoxBytesPerWarp = 32 * 128;           // row-owner epilogue: one box of 32 rows x 128 bytes per warp

}  // namespace rbg
