// Persistent bf16 GEMM on the 5th-generation tensor cores (sm_100a) with a fused epilogue.
//
//   D[M,N] = epilogue(alpha * op(A)·op(B)),   fp32 accumulation in tensor memory
//
// One CTA per SM walks a list of work units (128 x BN output tile, BN = 256 or 128, optionally one slice of K):
//   warp 0   TMA producer: cp.async.bulk.tensor (128-byte swizzle, no cluster multicast) into a shared-memory ring that keeps
//            running across units, so the loads of the next tile are in flight while the current one is still multiplied
//   warp 1   MMA issuer: one thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x BN x 16); tcgen05.commit frees the ring
//            stage and, after the last K block, publishes the accumulator
//   warps 2-5 epilogue: tcgen05.ld (32x32b) -> registers -> per-warp shared staging (swizzled fp32) -> every lane then owns
//            8 consecutive columns of one row, so that bias, activation, activation gradient, dropout (counter-based),
//            residual add and the store are all 16-byte coalesced accesses
// The accumulator is double-buffered in tensor memory (2 x BN columns): the epilogue of unit i overlaps the MMAs of unit i+1.
//
// Split-K: with accumulate == 2 the launcher may cut K into slices; every slice adds its partial tile to the fp32 output
// with vector atomics. This is what the weight gradient dW += X^T·dY uses (few output tiles, long contraction).
//
// Every mbarrier wait is bounded. A wait that gives up raises the CTA's abort flag and writes a status word; all roles
// leave their loops, the CTA waits for its TMA copies in flight, frees its tensor memory and returns.
#include "gemm_epilogue.cuh"
#include <cstdlib>

using namespace rbt;
using namespace rbg;

namespace {

constexpr int BM = 128;
constexpr int kThreads = kGemmThreads;
constexpr int kRingBytes = 196608;      // operand ring: 4 stages (BN = 256) or 6 stages (BN = 128)
constexpr int kStagingBytes = kEpilogueWarps * kStagingBytesPerWarp;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kRingBytes + kStagingBytes + kBarrierBytes + 1024;
constexpr int kMaxStages = 6;

template <int BN, bool FULL>
__global__ void __launch_bounds__(kThreads, 1)
gemm_persist_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Params p) {
  constexpr int kTileBytesA = BM * BK * 2;
  constexpr int kTileBytesB = BN * BK * 2;
  constexpr int kStageBytes = kTileBytesA + kTileBytesB;
  constexpr int kStages = kRingBytes / kStageBytes;
  static_assert(kStages <= kMaxStages && kStages >= 2, "ring");
  constexpr uint32_t kTmemCols = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* staging = reinterpret_cast<float*>(smem + kRingBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kRingBytes + kStagingBytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const RbGemm& g = p.g;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kEpilogueWarps);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: it may overlap the tail of the preceding kernel
  rb_pdl_wait();
  rb_pdl_launch();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const Unit w = decode_unit<BM, BN>(p, u);
        if (!w.valid) continue;
        const int m0 = w.m0, n0 = w.n0;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            if (g.status) atomicCAS(g.status, 0, (1 << 24) | (kb & 0xFFFFFF));
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kTileBytesA;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          const int k0 = kb * BK;
          if (!g.a_mn_major) {
            tma_load_2d(sa, &tm_a, w.a_c0 + k0, w.a_r0 + m0, &full_bar[s]);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tm_a, w.a_c0 + m0 + 64 * j, w.a_r0 + k0, &full_bar[s]);
          }
          if (!g.b_mn_major) {
            tma_load_2d(sb, &tm_b, w.b_c0 + k0, w.b_r0 + n0, &full_bar[s]);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tm_b, w.b_c0 + n0 + 64 * j, w.b_r0 + k0, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t ab_fmt = g.ab_fp16 ? 0u : 1u;  // operand format field: 0 = fp16, 1 = bf16 (accumulator fp32 either way)
      const uint32_t idesc = (1u << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((uint32_t)(g.a_mn_major ? 1 : 0) << 15) |
                             ((uint32_t)(g.b_mn_major ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const Unit w = decode_unit<BM, BN>(p, u);
        if (!w.valid) continue;
        const int kb0 = w.kb0, kb1 = w.kb1;
        const uint32_t buf = t_local & 1u;
        if (!mbar_wait(&acc_empty[buf], ((t_local >> 1) & 1u) ^ 1u, abort_flag)) {
          *abort_flag = 1;
          if (g.status) atomicCAS(g.status, 0, (4 << 24) | (u & 0xFFFFFF));
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
            *abort_flag = 1;
            if (g.status) atomicCAS(g.status, 0, (2 << 24) | (kb & 0xFFFFFF));
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kTileBytesA;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major: 16 elements = 32 bytes along the swizzled row; MN-major: 16 K-rows of 128 bytes = 2 swizzle atoms,
            // 64-wide MN groups 8192 bytes apart
            const uint64_t adesc = g.a_mn_major ? make_desc(sa + kk * 2048, 8192, 1024) : make_desc(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = g.b_mn_major ? make_desc(sb + kk * 2048, 8192, 1024) : make_desc(sb + kk * 32, 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
        ++t_local;
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    float* stg = staging + (warp - 2) * (kStagingBytesPerWarp / 4);
    uint32_t t_local = 0;
    for (int u = blockIdx.x; u < p.units; u += gridDim.x) {
      const Unit w = decode_unit<BM, BN>(p, u);
      if (!w.valid) continue;
      const int m0 = w.m0, n0 = w.n0;
      const uint32_t buf = t_local & 1u;
      bool ok = mbar_wait(&acc_full[buf], (t_local >> 1) & 1u, abort_flag);
      if (!ok && lane == 0) {
        *abort_flag = 1;
        if (g.status) atomicCAS(g.status, 0, (3 << 24) | (u & 0xFFFFFF));
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      const int part = (warp - 2) >> 2;  // four warps per lane quarter, each with a quarter of the columns
      epilogue_columns<FULL>(p, w, m0, n0, t_addr, part * (BN / 4), (part + 1) * (BN / 4), stg, lane, q, [&]() { mbar_arrive(&acc_empty[buf]); });
      ++t_local;
    }
  }

  // ---------------- teardown ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // let copies that are still in flight land before the shared memory goes away (bounded: about 1 ms)
    for (uint32_t i = 0; i < (1u << 12); ++i) __nanosleep(256);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int BN>
int launch(const RbGemm& g, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_persist_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_persist_kernel<BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      rb_set_error("gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return RB_ERR_LAUNCH;
    }
    attr_set = true;
  }
  Params p;
  p.g = g;
  p.tiles_m = (g.m + BM - 1) / BM;
  p.tiles_n = (g.n + BN - 1) / BN;
  p.num_kb = (g.k + BK - 1) / BK;
  const int tiles = p.tiles_m * p.tiles_n;
  const int sms = num_sms();
  int split = 1;
  if (g.accumulate == 2) {
    split = g.split_k > 0 ? g.split_k : (tiles >= sms ? 1 : sms / tiles);
    const int max_split = p.num_kb >= 4 ? p.num_kb / 4 : 1;  // at least 4 K blocks per slice
    if (split > max_split) split = max_split;
    if (split < 1) split = 1;
  }
  p.kb_per_split = (p.num_kb + split - 1) / split;
  p.split = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty slices
  p.units = tiles * p.split;
  if (g.batch > 0) {
    p.split = 1;
    p.units = tiles * g.batch;
  }
  auto al16 = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  p.vec_ok = (g.ldc % 8 == 0) && al16(g.c) && al16(g.c2) && al16(g.resid) && al16(g.dact_z);
  p.bias_vec = g.bias != nullptr && !g.bias_bf16 && al16(g.bias);
  const bool full = g.dact_z != nullptr || g.drop_p > 0.f || g.resid != nullptr;
  CUtensorMap tm_a, tm_b;
  int st;
  long long a_rows = g.a_mn_major ? g.k : g.m, a_cols = g.a_mn_major ? g.m : g.k;
  long long b_rows = g.b_mn_major ? g.k : g.n, b_cols = g.b_mn_major ? g.n : g.k;
  if (g.batch > 0) {
    a_rows = g.a_rows; a_cols = g.a_cols; b_rows = g.b_rows; b_cols = g.b_cols;
  }
  st = g.a_mn_major ? make_map(&tm_a, g.a, a_cols, a_rows, g.lda, 64, BK) : make_map(&tm_a, g.a, a_cols, a_rows, g.lda, BK, BM);
  if (st) return st;
  st = g.b_mn_major ? make_map(&tm_b, g.b, b_cols, b_rows, g.ldb, 64, BK) : make_map(&tm_b, g.b, b_cols, b_rows, g.ldb, BK, BN);
  if (st) return st;
  int grid = p.units < sms ? p.units : sms;
  {
    // tuning knob: cap the number of CTAs (for bandwidth / latency experiments)
    static int cap = -1;
    if (cap < 0) {
      const char* e = getenv("RETURNN_B200_GEMM_MAX_CTAS");
      cap = e ? atoi(e) : 0;
    }
    if (cap > 0 && grid > cap) grid = cap;
  }
  if (full) rb_launch_pdl(gemm_persist_kernel<BN, true>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_a, tm_b, p);
  else rb_launch_pdl(gemm_persist_kernel<BN, false>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_a, tm_b, p);
  return rb_check_launch("gemm_persist");
}

}  // namespace

int rb_gemm(const RbGemm& g, cudaStream_t stream) {
  if (g.m <= 0 || g.n <= 0) return RB_OK;
  if (g.k <= 0 && !(g.batch > 0 && g.k_from_lens)) {
    rb_set_error("gemm: k=%d", g.k);
    return RB_ERR_ARG;
  }
  if (g.batch > 0 && (g.accumulate == 2 || g.split_k > 1 || g.a_rows <= 0 || g.a_cols <= 0 || g.b_rows <= 0 || g.b_cols <= 0)) {
    rb_set_error("gemm: the batched form needs the stored extents and supports no split-K");
    return RB_ERR_ARG;
  }
  if ((g.lda % 8) || (g.ldb % 8) || (reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) {
    rb_set_error("gemm: operands need 16-byte aligned bases and pitches that are multiples of 8 elements (lda %d ldb %d)", g.lda, g.ldb);
    return RB_ERR_ARG;
  }
  if (g.accumulate && !g.out_fp32) {
    rb_set_error("gemm: accumulate needs fp32 output");
    return RB_ERR_ARG;
  }
  if (g.out_fp32 && (g.c2 || g.resid)) {
    rb_set_error("gemm: second output / residual need bf16 output");
    return RB_ERR_ARG;
  }
  if (g.drop_p > 0.f && (!g.seed || !g.offset || (g.ldc % 8) || !(g.drop_p < 1.f))) {
    rb_set_error("gemm: dropout epilogue needs seed/offset pointers, ldc %% 8 == 0 and p < 1 (ldc %d, p %f)", g.ldc, g.drop_p);
    return RB_ERR_ARG;
  }
  if (g.split_k > 1 && g.accumulate != 2) {
    rb_set_error("gemm: split_k needs accumulate == 2");
    return RB_ERR_ARG;
  }
  if (rb_gemm_pair_wanted(g)) return rb_gemm_pair(g, stream);
  if (g.n > 128) return launch<256>(g, stream);
  return launch<128>(g, stream);
}

// C entry points with the full epilogue (see gemm.h for the meaning of the arguments); the second reads A and B as fp16
static int gemm_ex(const void* a, const void* b, void* c, void* c2, const void* bias, int m, int n, int k, int lda, int ldb, int ldc, int a_mn_major,
                   int b_mn_major, int bias_bf16, int act, int out_fp32, int accumulate, float alpha, const void* dact_z, float drop_p,
                   const long long* seed, const long long* offset, unsigned long long drop_site, const void* resid, float res_scale, int split_k,
                   int* status, int ab_fp16, cudaStream_t stream) {
  RbGemm g;
  g.a = a; g.b = b; g.c = c; g.c2 = c2; g.bias = bias; g.bias_bf16 = bias_bf16;
  g.m = m; g.n = n; g.k = k; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.a_mn_major = a_mn_major; g.b_mn_major = b_mn_major; g.ab_fp16 = ab_fp16;
  g.act = act; g.out_fp32 = out_fp32; g.accumulate = accumulate; g.alpha = alpha;
  g.dact_z = dact_z; g.drop_p = drop_p; g.seed = seed; g.offset = offset; g.drop_site = drop_site;
  g.resid = resid; g.res_scale = res_scale; g.split_k = split_k; g.status = status;
  return rb_gemm(g, stream);
}

RB_EXPORT int rb200_gemm_bf16_ex(const void* a, const void* b, void* c, void* c2, const void* bias, int m, int n, int k, int lda, int ldb,
                                 int ldc, int a_mn_major, int b_mn_major, int bias_bf16, int act, int out_fp32, int accumulate, float alpha,
                                 const void* dact_z, float drop_p, const long long* seed, const long long* offset,
                                 unsigned long long drop_site, const void* resid, float res_scale, int split_k, int* status,
                                 cudaStream_t stream) {
  return gemm_ex(a, b, c, c2, bias, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, bias_bf16, act, out_fp32, accumulate, alpha, dact_z, drop_p, seed,
                 offset, drop_site, resid, res_scale, split_k, status, 0, stream);
}

RB_EXPORT int rb200_gemm_fp16_ex(const void* a, const void* b, void* c, void* c2, const void* bias, int m, int n, int k, int lda, int ldb,
                                 int ldc, int a_mn_major, int b_mn_major, int bias_bf16, int act, int out_fp32, int accumulate, float alpha,
                                 const void* dact_z, float drop_p, const long long* seed, const long long* offset,
                                 unsigned long long drop_site, const void* resid, float res_scale, int split_k, int* status,
                                 cudaStream_t stream) {
  return gemm_ex(a, b, c, c2, bias, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, bias_bf16, act, out_fp32, accumulate, alpha, dact_z, drop_p, seed,
                 offset, drop_site, resid, res_scale, split_k, status, 1, stream);
}
