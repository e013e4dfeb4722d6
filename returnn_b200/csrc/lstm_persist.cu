// Persistent LSTM recurrence: ONE kernel runs all T steps of a direction. The recurrent matrix never leaves the chip: CTA c
// keeps the rows of W_rec that produce the four gates of its kUnits hidden units in shared memory (forward), or the columns
// that those units feed (backward), for the whole sequence. Per step a CTA multiplies the small [B, K] activation matrix (read
// from L2, where the other CTAs wrote it in the previous step) with its resident slice on the tensor cores, applies the cell
// for its units, publishes its slice of h_t (or dz_t) and meets the other CTAs at a grid barrier. The per-step executor in
// lstm.cu needs two launches of latency-bound kernels per step (about 22 us); here a step is a barrier plus about 100 KB of L2
// reads per CTA.
//
// The step product has only B <= 48 rows: the warp-level mma (m16n8k16, bf16 -> fp32) fits this shape (three 16-row tiles);
// a tcgen05 tile is at least 64 rows by one CTA and its operands would have to be re-staged through TMA every step. The eight
// warps of a CTA split the contraction; their partial sums meet in shared memory.
//
// Launched cooperatively (all CTAs resident). Every barrier wait is bounded: a CTA that gives up raises the abort word, all
// CTAs leave the time loop, and the host reports RB_ERR_TIMEOUT.
//
// Semantics, gate order (i, f, g, o), masking and the tensors saved for backward are those of lstm.cu
// (reference: returnn/native_op.py:1029-1179 NativeLstm2, returnn/torch/frontend/_backend.py:2796-2810).
#include "common.cuh"
#include "gemm.h"
#include <cooperative_groups.h>

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kUnits = 8;      // hidden units per CTA (H = 1024 -> 128 CTAs)
constexpr int kMaxRows = 48;   // batch rows (three m16 tiles)
constexpr int kThreads = 256;  // eight warps: each takes one eighth of the contraction
constexpr int kPad = 32;       // row padding of the resident slice: pitch = 64 bytes mod 128 (conflict-free 16-byte fragment loads)
constexpr int kRedPad = 8;      // row padding of the partial-sum slots
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// all CTAs of the grid; false (for every thread of every CTA, eventually) when someone timed out
__device__ bool grid_barrier(uint32_t* counter, uint32_t target, int* abort_word, int* status) {
  __shared__ int sh_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    int ok = 1;
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_gpu(counter) - target) < 0) {
      if (++spins > kSpinLimit || *reinterpret_cast<volatile int*>(abort_word)) {
        ok = 0;
        atomicExch(abort_word, 1);
        if (status) atomicCAS(status, 0, (5 << 24) | (int)(blockIdx.x & 0xFFFF));
        break;
      }
      __nanosleep(64);
    }
    __threadfence();
    sh_ok = ok;
  }
  __syncthreads();
  return sh_ok != 0;
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// red[row][n] += sum_k A[row][k] * Bs[n][k] for rows < n_rows; A in global (written by other CTAs: read through L2), Bs resident
// in shared memory with row pitch K + kPad. The contraction is cut into blocks of 32 k; the warp w takes the blocks
// [w*nblk/8, (w+1)*nblk/8).
//
// Operand fetch: all CTAs read the same small A matrix at the same time, so the number of L2 requests, not the bytes, sets the
// step time. A lane therefore fetches 16 contiguous bytes (8 k) per row and block instead of four 4-byte fragment words: the
// order of the k inside a block is free as long as A and B agree, so the lane t of a quad owns k [8t, 8t+8) of the block, its
// words 0/1 feed the first m16n8k16 (as the fragment halves "k 2t.." and "k 2t+8..") and its words 2/3 the second one. The B
// fragments come from shared memory with the same 16-byte pattern (row pitch = 64 bytes mod 128: conflict-free quarter warps).
template <int NOUT, int kPrefetch>
__device__ __forceinline__ void step_matmul(const bf16* __restrict__ A, int n_rows, int K, const bf16* __restrict__ Bs, float* __restrict__ red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int pitch = K + kPad;
  float acc[3][NOUT / 8][4];
#pragma unroll
  for (int m = 0; m < 3; ++m)
#pragma unroll
    for (int n = 0; n < NOUT / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;
  const int m_tiles = (n_rows + 15) / 16;
  auto load_a = [&](int k0, uint4 (&a)[3][2]) {
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      const int r0 = m * 16 + g, r1 = r0 + 8;
      a[m][0] = r0 < n_rows ? __ldcg(reinterpret_cast<const uint4*>(A + (size_t)r0 * K + k0 + 8 * t)) : make_uint4(0u, 0u, 0u, 0u);
      a[m][1] = r1 < n_rows ? __ldcg(reinterpret_cast<const uint4*>(A + (size_t)r1 * K + k0 + 8 * t)) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  // chunks of kPrefetch blocks: all operand loads of a chunk are issued before its first multiply, so a chunk costs one L2 round
  // trip (kPrefetch = 4: the forward contraction of H = 1024 is a single chunk per warp; the two-direction kernels use 2 to stay
  // within 128 registers, so that two CTAs share an SM and cover each other's round trips)
  const int nblk = K >> 5;
  const int b_begin = warp * nblk / 8, b_end = (warp + 1) * nblk / 8;
  for (int bc = b_begin; bc < b_end; bc += kPrefetch) {
    uint4 a[kPrefetch][3][2];
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i)
      if (bc + i < b_end) load_a((bc + i) << 5, a[i]);
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i) {
      if (bc + i >= b_end) break;
      const int k0 = (bc + i) << 5;
#pragma unroll
      for (int n = 0; n < NOUT / 8; ++n) {
        const uint4 b = *reinterpret_cast<const uint4*>(Bs + (size_t)(n * 8 + g) * pitch + k0 + 8 * t);
#pragma unroll
        for (int m = 0; m < 3; ++m) {
          if (m >= m_tiles) continue;
          const uint32_t f0[4] = {a[i][m][0].x, a[i][m][1].x, a[i][m][0].y, a[i][m][1].y};
          mma16816(acc[m][n], f0, b.x, b.y);
          const uint32_t f1[4] = {a[i][m][0].z, a[i][m][1].z, a[i][m][0].w, a[i][m][1].w};
          mma16816(acc[m][n], f1, b.z, b.w);
        }
      }
    }
  }
  // The partial sums of the eight warps meet in shared memory without atomics (eight warps adding 48 values per lane onto the
  // same words was the largest batch-dependent part of a forward step): warps 4..7 store theirs into slot (warp - 4), warps
  // 0..3 add their own onto that slot, the caller sums the four slots (red_sum). Row pitch NOUT + 8 floats: the 8-byte accesses
  // of a half warp fall on distinct banks.
  constexpr int RP = NOUT + kRedPad;
  float* slot = red + (warp & 3) * (kMaxRows * RP);
  if (warp >= 4) {
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      if (m >= m_tiles) continue;
      const int r0 = m * 16 + g, r1 = r0 + 8;
#pragma unroll
      for (int n = 0; n < NOUT / 8; ++n) {
        const int c = n * 8 + 2 * t;
        *reinterpret_cast<float2*>(&slot[r0 * RP + c]) = make_float2(acc[m][n][0], acc[m][n][1]);
        *reinterpret_cast<float2*>(&slot[r1 * RP + c]) = make_float2(acc[m][n][2], acc[m][n][3]);
      }
    }
  }
  __syncthreads();
  if (warp < 4) {
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      if (m >= m_tiles) continue;
      const int r0 = m * 16 + g, r1 = r0 + 8;
#pragma unroll
      for (int n = 0; n < NOUT / 8; ++n) {
        const int c = n * 8 + 2 * t;
        float2* q0 = reinterpret_cast<float2*>(&slot[r0 * RP + c]);
        float2* q1 = reinterpret_cast<float2*>(&slot[r1 * RP + c]);
        const float2 v0 = *q0, v1 = *q1;
        *q0 = make_float2(v0.x + acc[m][n][0], v0.y + acc[m][n][1]);
        *q1 = make_float2(v1.x + acc[m][n][2], v1.y + acc[m][n][3]);
      }
    }
  }
}

// sum over the four slots that step_matmul leaves (after a __syncthreads)
template <int NOUT>
__device__ __forceinline__ float red_sum(const float* __restrict__ red, int row, int col) {
  constexpr int RP = NOUT + kRedPad;
  const float* q = red + row * RP + col;
  return (q[0] + q[kMaxRows * RP]) + (q[2 * kMaxRows * RP] + q[3 * kMaxRows * RP]);
}

struct FwdArgs {
  const bf16* z_in;     // [T,B,4H]
  const bf16* w_rec;    // [4H,H]
  const int* lens;      // [B] or null
  const float *h0, *c0; // [B,H]
  int T, B, H, reverse;
  bf16* y;              // [T,B,H]
  float* c_all;         // [T,B,H]
  bf16* gates;          // [T,B,4H]
  bf16* hprev_all;      // [T,B,H]
  float *h_final, *c_final;
  bf16* hbuf;           // [2,B,H] exchange buffer of the hidden state
  uint32_t* counter;    // zeroed before the launch
  int* abort_word;      // zeroed before the launch
  int* status;          // receives (5 << 24) | cta when a barrier wait ran out
};

template <int kPrefetch>
__device__ __forceinline__ void fwd_body(const FwdArgs& p, const int cta, const uint32_t n_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B;
  const int pitch = H + kPad;
  bf16* Ws = reinterpret_cast<bf16*>(smem_raw);                                 // [4*kUnits][H+kPad]: row q*kUnits+u = W_rec[q*H + j0 + u]
  float* red = reinterpret_cast<float*>(Ws + (size_t)4 * kUnits * pitch);       // [4 slots][48][4*kUnits + kRedPad]
  float* cst = red + 4 * kMaxRows * (4 * kUnits + kRedPad);                                     // [48][kUnits] cell state
  float* hst = cst + kMaxRows * kUnits;                                         // [48][kUnits] own slice of h (fp32)
  const int j0 = cta * kUnits;
  // resident slice: 4*kUnits rows of H elements, 16-byte copies
  for (int idx = threadIdx.x; idx < 4 * kUnits * (H / 8); idx += kThreads) {
    const int r = idx / (H / 8), v = idx % (H / 8);
    const int q = r / kUnits, u = r % kUnits;
    *reinterpret_cast<uint4*>(Ws + (size_t)r * pitch + v * 8) = *reinterpret_cast<const uint4*>(p.w_rec + ((size_t)q * H + j0 + u) * H + v * 8);
  }
  for (int idx = threadIdx.x; idx < kMaxRows * kUnits; idx += kThreads) {
    const int b = idx / kUnits, u = idx % kUnits;
    float c = 0.f, h = 0.f;
    if (b < B) {
      c = p.c0[(size_t)b * H + j0 + u];
      h = p.h0[(size_t)b * H + j0 + u];
      p.hbuf[(size_t)b * H + j0 + u] = __float2bfloat16(h);
    }
    cst[idx] = c;
    hst[idx] = __bfloat162float(__float2bfloat16(h));
  }
  // every thread owns up to kSlots (row, unit) pairs; their input projections z_in[t] are fetched one step ahead (they come from
  // DRAM) so that the cell does not wait for them after the barrier
  constexpr int kSlots = (kMaxRows * kUnits + kThreads - 1) / kThreads;
  float zin[kSlots][4];
  auto fetch_zin = [&](int t) {
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < B * kUnits) {
        const int b = idx / kUnits, u = idx % kUnits;
        const bf16* z = p.z_in + ((size_t)t * B + b) * 4 * H + j0 + u;
#pragma unroll
        for (int q = 0; q < 4; ++q) zin[i][q] = __bfloat162float(z[(size_t)q * H]);
      }
    }
  };
  if (p.T > 0) fetch_zin(p.reverse ? p.T - 1 : 0);
  uint32_t n_bar = 0;
  bool ok = grid_barrier(p.counter, (++n_bar) * n_cta, p.abort_word, p.status);
  for (int s = 0; s < p.T && ok; ++s) {
    const int t = p.reverse ? p.T - 1 - s : s;
    const bf16* h_cur = p.hbuf + (size_t)(s & 1) * B * H;
    bf16* h_nxt = p.hbuf + (size_t)((s + 1) & 1) * B * H;
    step_matmul<4 * kUnits, kPrefetch>(h_cur, B, H, Ws, red);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx >= B * kUnits) continue;
      const int b = idx / kUnits, u = idx % kUnits;
      const size_t o = ((size_t)t * B + b) * H + j0 + u;
      const size_t zo = ((size_t)t * B + b) * 4 * H + j0 + u;
      const bool valid = !p.lens || t < p.lens[b];
      const float hp = hst[idx], cp = cst[idx];
      p.hprev_all[o] = __float2bfloat16(hp);
      if (!valid) {
        p.y[o] = __float2bfloat16(0.f);
        p.c_all[o] = cp;
        p.gates[zo] = p.gates[zo + H] = p.gates[zo + 2 * H] = p.gates[zo + 3 * H] = __float2bfloat16(0.f);
        h_nxt[(size_t)b * H + j0 + u] = __float2bfloat16(hp);
        continue;
      }
      const float gi = sigm(red_sum<4 * kUnits>(red, b, u) + zin[i][0]);
      const float gf = sigm(red_sum<4 * kUnits>(red, b, kUnits + u) + zin[i][1]);
      const float gg = tanhf(red_sum<4 * kUnits>(red, b, 2 * kUnits + u) + zin[i][2]);
      const float go = sigm(red_sum<4 * kUnits>(red, b, 3 * kUnits + u) + zin[i][3]);
      const float c = gf * cp + gi * gg;
      const bf16 hb = __float2bfloat16(go * tanhf(c));
      cst[idx] = c;
      hst[idx] = __bfloat162float(hb);
      p.c_all[o] = c;
      p.y[o] = hb;
      h_nxt[(size_t)b * H + j0 + u] = hb;
      p.gates[zo] = __float2bfloat16(gi);
      p.gates[zo + H] = __float2bfloat16(gf);
      p.gates[zo + 2 * H] = __float2bfloat16(gg);
      p.gates[zo + 3 * H] = __float2bfloat16(go);
    }
    if (s + 1 < p.T) fetch_zin(p.reverse ? p.T - 2 - s : s + 1);
    ok = grid_barrier(p.counter, (++n_bar) * n_cta, p.abort_word, p.status);
  }
  for (int idx = threadIdx.x; idx < B * kUnits; idx += kThreads) {
    const int b = idx / kUnits, u = idx % kUnits;
    p.h_final[(size_t)b * H + j0 + u] = hst[idx];
    p.c_final[(size_t)b * H + j0 + u] = cst[idx];
  }
}

__global__ void __launch_bounds__(kThreads, 1) lstm_persist_fwd_kernel(FwdArgs p) { fwd_body<4>(p, blockIdx.x, gridDim.x); }

// Both directions of a bidirectional layer in one launch: the first half of the grid runs d[0], the second half d[1], each with
// its own barrier words. Two CTAs share an SM (128 registers per thread), so the two recurrences, each bound by the latency of
// its grid barrier and L2 round trip per step, overlap instead of running one after the other.
struct FwdPair {
  FwdArgs d[2];
};

__global__ void __launch_bounds__(kThreads, 2) lstm_persist_fwd_pair_kernel(const __grid_constant__ FwdPair pp) {
  const int half = gridDim.x / 2;
  if ((int)blockIdx.x < half) fwd_body<2>(pp.d[0], blockIdx.x, half);
  else fwd_body<2>(pp.d[1], blockIdx.x - half, half);
}

struct BwdArgs {
  const bf16* dy;        // [T,B,H] or null
  const float *dh_final, *dc_final;  // [B,H] or null
  const bf16* w_rec;     // [4H,H]
  const int* lens;
  const bf16* gates;     // [T,B,4H]
  const float *c_all, *c0;
  int T, B, H, reverse;
  bf16* dz;              // [T,B,4H]: output and per-step exchange buffer
  float *dh0, *dc0;      // [B,H] outputs
  uint32_t* counter;
  int* abort_word;
  int* status;
};

template <int kPrefetch>
__device__ __forceinline__ void bwd_body(const BwdArgs& p, const int cta, const uint32_t n_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B, K = 4 * p.H;
  const int pitch = K + kPad;
  bf16* Wt = reinterpret_cast<bf16*>(smem_raw);                      // [kUnits][4H+kPad]: Wt[u][n] = W_rec[n][j0+u]
  float* red = reinterpret_cast<float*>(Wt + (size_t)kUnits * pitch);  // [4 slots][48][kUnits + kRedPad]
  float* dhs = red + 4 * kMaxRows * (kUnits + kRedPad);                              // [48][16] gradient arriving at h_t
  float* dcs = dhs + kMaxRows * kUnits;                              // [48][16] gradient arriving at c_t
  const int j0 = cta * kUnits;
  for (int idx = threadIdx.x; idx < K * (kUnits / 8); idx += kThreads) {
    // row n of W_rec, units j0 .. j0 + kUnits - 1, in 16-byte pieces
    const int n = idx / (kUnits / 8), piece = idx % (kUnits / 8);
    const uint4 v = *reinterpret_cast<const uint4*>(p.w_rec + (size_t)n * H + j0 + piece * 8);
    const bf16* e = reinterpret_cast<const bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) Wt[(size_t)(piece * 8 + i) * pitch + n] = e[i];
  }
  for (int idx = threadIdx.x; idx < kMaxRows * kUnits; idx += kThreads) {
    const int b = idx / kUnits, u = idx % kUnits;
    dhs[idx] = (b < B && p.dh_final) ? p.dh_final[(size_t)b * H + j0 + u] : 0.f;
    dcs[idx] = (b < B && p.dc_final) ? p.dc_final[(size_t)b * H + j0 + u] : 0.f;
  }
  __syncthreads();
  uint32_t n_bar = 0;
  bool ok = true;
  for (int s = p.T - 1; s >= 0 && ok; --s) {
    const int t = p.reverse ? p.T - 1 - s : s;
    const int t_prev = p.reverse ? t + 1 : t - 1;
    bf16* dz_t = p.dz + (size_t)t * B * K;
    for (int idx = threadIdx.x; idx < B * kUnits; idx += kThreads) {
      const int b = idx / kUnits, u = idx % kUnits;
      const size_t o = ((size_t)t * B + b) * H + j0 + u;
      const size_t zo = (size_t)b * K + j0 + u;
      const bool valid = !p.lens || t < p.lens[b];
      if (!valid) {
        dz_t[zo] = dz_t[zo + H] = dz_t[zo + 2 * H] = dz_t[zo + 3 * H] = __float2bfloat16(0.f);
        continue;  // state was carried: dh and dc pass through
      }
      const float dh = dhs[idx] + (p.dy ? __bfloat162float(p.dy[o]) : 0.f);
      const bf16* gt = p.gates + ((size_t)t * B + b) * K + j0 + u;
      const float gi = __bfloat162float(gt[0]), gf = __bfloat162float(gt[H]), gg = __bfloat162float(gt[2 * H]), go = __bfloat162float(gt[3 * H]);
      const float tc = tanhf(p.c_all[o]);
      const float cprev = s > 0 ? p.c_all[((size_t)t_prev * B + b) * H + j0 + u] : p.c0[(size_t)b * H + j0 + u];
      const float dc = dcs[idx] + dh * go * (1.f - tc * tc);
      dz_t[zo] = __float2bfloat16(dc * gg * gi * (1.f - gi));
      dz_t[zo + H] = __float2bfloat16(dc * cprev * gf * (1.f - gf));
      dz_t[zo + 2 * H] = __float2bfloat16(dc * gi * (1.f - gg * gg));
      dz_t[zo + 3 * H] = __float2bfloat16(dh * tc * go * (1.f - go));
      dcs[idx] = dc * gf;
      dhs[idx] = 0.f;
    }
    ok = grid_barrier(p.counter, (++n_bar) * n_cta, p.abort_word, p.status);  // all slices of dz_t are written
    if (!ok) break;
    step_matmul<kUnits, kPrefetch>(dz_t, B, K, Wt, red);
    __syncthreads();
    for (int idx = threadIdx.x; idx < B * kUnits; idx += kThreads) dhs[idx] += red_sum<kUnits>(red, idx / kUnits, idx % kUnits);
    __syncthreads();
  }
  for (int idx = threadIdx.x; idx < B * kUnits; idx += kThreads) {
    const int b = idx / kUnits, u = idx % kUnits;
    p.dh0[(size_t)b * H + j0 + u] = dhs[idx];
    p.dc0[(size_t)b * H + j0 + u] = dcs[idx];
  }
}

__global__ void __launch_bounds__(kThreads, 1) lstm_persist_bwd_kernel(BwdArgs p) { bwd_body<4>(p, blockIdx.x, gridDim.x); }

struct BwdPair {
  BwdArgs d[2];
};

__global__ void __launch_bounds__(kThreads, 2) lstm_persist_bwd_pair_kernel(const __grid_constant__ BwdPair pp) {
  const int half = gridDim.x / 2;
  if ((int)blockIdx.x < half) bwd_body<2>(pp.d[0], blockIdx.x, half);
  else bwd_body<2>(pp.d[1], blockIdx.x - half, half);
}

// barrier words of the calls in flight: 64 slots of (counter, abort word), handed out round robin
constexpr int kSyncSlots = 64;
static __device__ unsigned int g_lstm_sync[kSyncSlots * 2];

unsigned int* sync_slot() {
  static unsigned int* base[64] = {nullptr};
  static unsigned next = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!base[dev]) {
    unsigned int* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_lstm_sync) != cudaSuccess) return nullptr;
    base[dev] = ptr;
  }
  return base[dev] + 2 * (next++ % kSyncSlots);
}

size_t fwd_smem(int H) {
  return (size_t)4 * kUnits * (H + kPad) * sizeof(bf16) + (size_t)kMaxRows * (4 * (4 * kUnits + kRedPad) + 2 * kUnits) * sizeof(float);
}
size_t bwd_smem(int H) {
  return (size_t)kUnits * (4 * H + kPad) * sizeof(bf16) + (size_t)kMaxRows * (4 * (kUnits + kRedPad) + 2 * kUnits) * sizeof(float);
}

bool enabled() {
  static const bool on = [] {
    const char* v = getenv("RETURNN_B200_LSTM_PERSIST");
    return !(v && v[0] == '0');
  }();
  return on;
}

}  // namespace

// whether the persistent kernels take this problem (else the per-step executor runs)
bool rb_lstm_persist_supported(int T, int B, int H) {
  if (!enabled() || T <= 0 || B <= 0 || B > kMaxRows || H % 128 || H / kUnits > 148) return false;
  return fwd_smem(H) <= 220 * 1024 && bwd_smem(H) <= 220 * 1024;
}

// scratch: hbuf 2*B*H bf16 provided by the caller, contents arbitrary
int rb_lstm_persist_fwd(const void* z_in, const void* w_rec, const int* lens, const float* h0, const float* c0, int T, int B, int H, int reverse,
                        void* y, float* c_all, void* gates, void* hprev_all, float* h_final, float* c_final, void* hbuf, int* status,
                        cudaStream_t stream) {
  unsigned int* sync_words = sync_slot();
  if (!sync_words) {
    rb_set_error("lstm_persist_fwd: no barrier words");
    return RB_ERR_LAUNCH;
  }
  FwdArgs a;
  a.z_in = (const bf16*)z_in; a.w_rec = (const bf16*)w_rec; a.lens = lens; a.h0 = h0; a.c0 = c0;
  a.T = T; a.B = B; a.H = H; a.reverse = reverse;
  a.y = (bf16*)y; a.c_all = c_all; a.gates = (bf16*)gates; a.hprev_all = (bf16*)hprev_all; a.h_final = h_final; a.c_final = c_final;
  a.hbuf = (bf16*)hbuf; a.counter = sync_words; a.abort_word = reinterpret_cast<int*>(sync_words + 1); a.status = status;
  cudaMemsetAsync(sync_words, 0, 2 * sizeof(unsigned int), stream);
  const size_t smem = fwd_smem(H);
  cudaError_t e = cudaFuncSetAttribute(lstm_persist_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  void* args[] = {&a};
  if (e == cudaSuccess) e = cudaLaunchCooperativeKernel((const void*)lstm_persist_fwd_kernel, dim3(H / kUnits), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) {
    rb_set_error("lstm_persist_fwd: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return RB_ERR_LAUNCH;
  }
  return RB_OK;
}

int rb_lstm_persist_bwd(const void* dy, const float* dh_final, const float* dc_final, const void* w_rec, const int* lens, const void* gates,
                        const float* c_all, const float* c0, int T, int B, int H, int reverse, void* dz, float* dh0, float* dc0, int* status,
                        cudaStream_t stream) {
  unsigned int* sync_words = sync_slot();
  if (!sync_words) {
    rb_set_error("lstm_persist_bwd: no barrier words");
    return RB_ERR_LAUNCH;
  }
  BwdArgs a;
  a.dy = (const bf16*)dy; a.dh_final = dh_final; a.dc_final = dc_final; a.w_rec = (const bf16*)w_rec; a.lens = lens; a.gates = (const bf16*)gates;
  a.c_all = c_all; a.c0 = c0; a.T = T; a.B = B; a.H = H; a.reverse = reverse; a.dz = (bf16*)dz; a.dh0 = dh0; a.dc0 = dc0;
  a.counter = sync_words; a.abort_word = reinterpret_cast<int*>(sync_words + 1); a.status = status;
  cudaMemsetAsync(sync_words, 0, 2 * sizeof(unsigned int), stream);
  const size_t smem = bwd_smem(H);
  cudaError_t e = cudaFuncSetAttribute(lstm_persist_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  void* args[] = {&a};
  if (e == cudaSuccess) e = cudaLaunchCooperativeKernel((const void*)lstm_persist_bwd_kernel, dim3(H / kUnits), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) {
    rb_set_error("lstm_persist_bwd: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return RB_ERR_LAUNCH;
  }
  return RB_OK;
}

// ---- both directions of a bidirectional layer in one cooperative launch -------------------------------------------------

// whether the two-direction kernels take this problem: the single-direction conditions, and both grids co-resident (two CTAs
// per SM: checked through the occupancy of the pair kernels on the current device)
RB_EXPORT int rb200_blstm_supported(int T, int B, int H) {
  if (!rb_lstm_persist_supported(T, B, H)) return 0;
  static int sm_count = 0, occ_fwd[2] = {-1, 0}, occ_bwd[2] = {-1, 0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (!sm_count && cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (occ_fwd[0] != H) {
    const size_t sf = fwd_smem(H), sb = bwd_smem(H);
    if (cudaFuncSetAttribute(lstm_persist_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sf) != cudaSuccess ||
        cudaFuncSetAttribute(lstm_persist_bwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sb) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_fwd[1], lstm_persist_fwd_pair_kernel, kThreads, sf) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_bwd[1], lstm_persist_bwd_pair_kernel, kThreads, sb) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    occ_fwd[0] = occ_bwd[0] = H;
  }
  const int need = 2 * (H / kUnits);
  return occ_fwd[1] * sm_count >= need && occ_bwd[1] * sm_count >= need;
}

// ptrs[d * 11 + i] for direction d (0: forward in time, 1: reversed):
//   0 z_in [T,B,4H] bf16, 1 w_rec [4H,H] bf16, 2 h0, 3 c0 [B,H] fp32, 4 y [T,B,H] bf16, 5 c_all [T,B,H] fp32, 6 gates [T,B,4H] bf16,
//   7 hprev_all [T,B,H] bf16, 8 h_final, 9 c_final [B,H] fp32, 10 hbuf (scratch, 2*B*H bf16)
RB_EXPORT int rb200_blstm_fwd(void* const* ptrs, const int* lens, int T, int B, int H, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return RB_OK;
  if (!rb200_blstm_supported(T, B, H)) {
    rb_set_error("blstm_fwd: shape T=%d B=%d H=%d is not supported by the two-direction kernel", T, B, H);
    return RB_ERR_UNSUPPORTED;
  }
  FwdPair pp;
  for (int d = 0; d < 2; ++d) {
    unsigned int* sync_words = sync_slot();
    if (!sync_words) {
      rb_set_error("blstm_fwd: no barrier words");
      return RB_ERR_LAUNCH;
    }
    void* const* q = ptrs + d * 11;
    FwdArgs& a = pp.d[d];
    a.z_in = (const bf16*)q[0]; a.w_rec = (const bf16*)q[1]; a.lens = lens; a.h0 = (const float*)q[2]; a.c0 = (const float*)q[3];
    a.T = T; a.B = B; a.H = H; a.reverse = d;
    a.y = (bf16*)q[4]; a.c_all = (float*)q[5]; a.gates = (bf16*)q[6]; a.hprev_all = (bf16*)q[7]; a.h_final = (float*)q[8]; a.c_final = (float*)q[9];
    a.hbuf = (bf16*)q[10]; a.counter = sync_words; a.abort_word = reinterpret_cast<int*>(sync_words + 1); a.status = status;
    cudaMemsetAsync(sync_words, 0, 2 * sizeof(unsigned int), stream);
  }
  const size_t smem = fwd_smem(H);
  void* args[] = {&pp};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_persist_fwd_pair_kernel, dim3(2 * (H / kUnits)), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) {
    rb_set_error("blstm_fwd: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return RB_ERR_LAUNCH;
  }
  return RB_OK;
}

// ptrs[d * 12 + i]: 0 dy [T,B,H] bf16 or null, 1 dh_final, 2 dc_final [B,H] fp32 or null, 3 w_rec bf16, 4 gates, 5 c_all, 6 c0, 7 hprev_all,
//   8 dz [T,B,4H] bf16 (out), 9 dw_rec [4H,H] fp32 (accumulated into; may be null), 10 dh0, 11 dc0 [B,H] fp32 (out)
RB_EXPORT int rb200_blstm_bwd(void* const* ptrs, const int* lens, int T, int B, int H, int* status, int* n_launch, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return RB_OK;
  if (!rb200_blstm_supported(T, B, H)) {
    rb_set_error("blstm_bwd: shape T=%d B=%d H=%d is not supported by the two-direction kernel", T, B, H);
    return RB_ERR_UNSUPPORTED;
  }
  BwdPair pp;
  for (int d = 0; d < 2; ++d) {
    unsigned int* sync_words = sync_slot();
    if (!sync_words) {
      rb_set_error("blstm_bwd: no barrier words");
      return RB_ERR_LAUNCH;
    }
    void* const* q = ptrs + d * 12;
    BwdArgs& a = pp.d[d];
    a.dy = (const bf16*)q[0]; a.dh_final = (const float*)q[1]; a.dc_final = (const float*)q[2]; a.w_rec = (const bf16*)q[3]; a.lens = lens;
    a.gates = (const bf16*)q[4]; a.c_all = (const float*)q[5]; a.c0 = (const float*)q[6]; a.T = T; a.B = B; a.H = H; a.reverse = d;
    a.dz = (bf16*)q[8]; a.dh0 = (float*)q[10]; a.dc0 = (float*)q[11];
    a.counter = sync_words; a.abort_word = reinterpret_cast<int*>(sync_words + 1); a.status = status;
    cudaMemsetAsync(sync_words, 0, 2 * sizeof(unsigned int), stream);
  }
  const size_t smem = bwd_smem(H);
  void* args[] = {&pp};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_persist_bwd_pair_kernel, dim3(2 * (H / kUnits)), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) {
    rb_set_error("blstm_bwd: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return RB_ERR_LAUNCH;
  }
  int launches = 3;
  for (int d = 0; d < 2; ++d) {
    void* const* q = ptrs + d * 12;
    if (!q[9]) continue;
    // dW_rec[4H,H] += dz^T [4H, T*B] . h_prev [T*B, H]
    RbGemm g;
    g.a = q[8]; g.b = q[7]; g.c = q[9]; g.m = 4 * H; g.n = H; g.k = T * B; g.lda = 4 * H; g.ldb = H; g.ldc = H;
    g.a_mn_major = 1; g.b_mn_major = 1; g.out_fp32 = 1; g.accumulate = 2; g.status = status;
    int st = rb_gemm(g, stream);
    if (st) return st;
    ++launches;
  }
  if (n_launch) *n_launch = launches;
  return rb_check_launch("blstm_bwd");
}
