// bf16 GEMM on the 5th-generation tensor cores (sm_100a): D[M,N] = A · B (+ bias) (activation), fp32 accumulation in TMEM.
//
//   - operands arrive in shared memory through TMA (cp.async.bulk.tensor, 128-byte swizzle) into a 3-stage ring;
//     no cluster multicast: every CTA loads its own tiles
//   - one elected thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x 128 x 16 per instruction),
//     accumulator = 128 lanes x 128 fp32 columns of tensor memory
//   - tcgen05.commit arrives on mbarriers: "stage free" for the producer, "accumulator ready" for the epilogue
//   - 4 epilogue warps read their 32 TMEM lanes with tcgen05.ld (32x32b.x32), apply bias / activation, write bf16 or fp32
//
// Operand layouts ("major"): a K-major operand is stored [rows = M or N][K contiguous]; an MN-major operand is stored
// [K][M or N contiguous]. All four combinations are supported, which covers forward (X·W), data gradient (dY·W^T) and
// weight gradient (X^T·dY) of a linear layer with row-major tensors and no transposes in memory.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the kernel raises an abort flag (shared), writes a status word
// to global memory, waits for its own TMA copies with a second bound, frees its tensor memory and returns.
#include "tcgen05.cuh"
#include "gemm.h"
#include <cstdlib>
#include <cstring>

using namespace rbt;

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 3;
constexpr int kTileBytesA = BM * BK * 2;  // 16 KB
constexpr int kTileBytesB = BN * BK * 2;  // 16 KB
constexpr int kStageBytes = kTileBytesA + kTileBytesB;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr int kThreads = 192;  // warp 0: TMA producer, warp 1: MMA issuer + TMEM owner, warps 2..5: epilogue
constexpr uint32_t kTmemCols = 128;

struct GemmParams {
  void* c;            // [M, ldc]
  void* c2;           // optional second output: the activated value (c then holds the pre-activation)
  const void* bias;   // [N] or null
  int m, n, k;
  int ldc;            // elements
  int a_mn_major, b_mn_major;
  int bias_bf16;
  int act;            // 0 none, 1 relu, 2 silu, 3 gelu(erf)
  int out_fp32;       // c dtype
  int accumulate;     // fp32 out only: c += result
  float alpha;        // result scale (applied before bias)
  int* status;        // device word: 0 ok, else (code << 24 | detail)
  // batching: blockIdx.z = b * heads + h; operand origins (in stored-matrix rows / columns) and output offset per (b, h)
  int heads;
  long long a_rb, a_rh, a_cb, a_ch;
  long long b_rb, b_rh, b_cb, b_ch;
  long long c_sb, c_sh;   // element offsets into c / c2
  const int* lens;        // per-b length, or null
  int m_from_lens, n_from_lens, k_from_lens;  // take the extent from lens[b] instead of m / n / k
};

__global__ void __launch_bounds__(kThreads, 2)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_bar = empty_bar + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const int zb = (int)blockIdx.z / p.heads, zh = (int)blockIdx.z % p.heads;
  const int len_b = p.lens ? p.lens[zb] : 0;
  const int M = p.m_from_lens ? len_b : p.m;
  const int N = p.n_from_lens ? len_b : p.n;
  const int K = p.k_from_lens ? len_b : p.k;
  if (m0 >= M || n0 >= N) return;  // uniform for the whole CTA, before any barrier or TMEM use
  const int a_r0 = (int)(zb * p.a_rb + zh * p.a_rh), a_c0 = (int)(zb * p.a_cb + zh * p.a_ch);
  const int b_r0 = (int)(zb * p.b_rb + zh * p.b_rh), b_c0 = (int)(zb * p.b_cb + zh * p.b_ch);
  const size_t c_off = (size_t)zb * p.c_sb + (size_t)zh * p.c_sh;
  const int num_kb = K > 0 ? (K + BK - 1) / BK : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        const uint32_t round = kb / kStages;
        if (round > 0) {
          if (!mbar_wait(&empty_bar[s], (round - 1) & 1u, abort_flag)) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, (1 << 24) | kb);
            break;
          }
        }
        uint8_t* sa = smem + s * kStageBytes;
        uint8_t* sb = sa + kTileBytesA;
        mbar_expect_tx(&full_bar[s], kStageBytes);
        const int k0 = kb * BK;
        if (!p.a_mn_major) {
          tma_load_2d(sa, &tm_a, a_c0 + k0, a_r0 + m0, &full_bar[s]);
        } else {
          tma_load_2d(sa, &tm_a, a_c0 + m0, a_r0 + k0, &full_bar[s]);
          tma_load_2d(sa + kTileBytesA / 2, &tm_a, a_c0 + m0 + 64, a_r0 + k0, &full_bar[s]);
        }
        if (!p.b_mn_major) {
          tma_load_2d(sb, &tm_b, b_c0 + k0, b_r0 + n0, &full_bar[s]);
        } else {
          tma_load_2d(sb, &tm_b, b_c0 + n0, b_r0 + k0, &full_bar[s]);
          tma_load_2d(sb + kTileBytesB / 2, &tm_b, b_c0 + n0 + 64, b_r0 + k0, &full_bar[s]);
        }
        ++issued;
      }
      (void)issued;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      // instruction descriptor: fp32 accumulate, bf16 A and B, majors, N/8, M/16
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn_major ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn_major ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kStages;
        const uint32_t round = kb / kStages;
        if (!mbar_wait(&full_bar[s], round & 1u, abort_flag)) {
          *abort_flag = 1;
          if (p.status) atomicCAS(p.status, 0, (2 << 24) | kb);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(smem + s * kStageBytes);
        const uint32_t sb = sa + kTileBytesA;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          // K-major: 16 elements = 32 bytes along the swizzled row; MN-major: 16 K-rows of 128 bytes = 2 swizzle atoms
          const uint64_t adesc = p.a_mn_major ? make_desc(sa + kk * 2048, /*lbo=*/kTileBytesA / 2, /*sbo=*/1024)
                                              : make_desc(sa + kk * 32, /*lbo=*/16, /*sbo=*/1024);
          const uint64_t bdesc = p.b_mn_major ? make_desc(sb + kk * 2048, /*lbo=*/kTileBytesB / 2, /*sbo=*/1024)
                                              : make_desc(sb + kk * 32, /*lbo=*/16, /*sbo=*/1024);
          umma_f16(tmem_base, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
      }
      if (ok) umma_commit(acc_bar);  // accumulator complete (with num_kb == 0 this arrives at once; the epilogue then writes zeros)
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    bool ok = mbar_wait(acc_bar, 0, abort_flag);
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.status) atomicCAS(p.status, 0, (3 << 24));
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < M;
      const bool vec_ok = (p.ldc % 8) == 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (!row_ok) continue;
        const int col0 = n0 + c0;
        if (col0 >= N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = num_kb > 0 ? __uint_as_float(r[j]) * p.alpha : 0.f;
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            int col = col0 + j;
            if (col < N) {
              v[j] += p.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col])
                                  : reinterpret_cast<const float*>(p.bias)[col];
            }
          }
        }
        const size_t off = c_off + (size_t)row * p.ldc + col0;
        if (p.out_fp32) {
          float* c = reinterpret_cast<float*>(p.c) + off;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < N) {
              float val = apply_act(v[j], p.act);
              c[j] = p.accumulate ? c[j] + val : val;
            }
          }
        } else {
          __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.c) + off;
          __nv_bfloat16* c2 = p.c2 ? reinterpret_cast<__nv_bfloat16*>(p.c2) + off : nullptr;
          if (vec_ok && col0 + 32 <= N && (c_off % 8) == 0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 u, u2;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
              __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u2);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float a = v[g * 8 + 2 * j], b = v[g * 8 + 2 * j + 1];
                if (c2) {
                  h[j] = __floats2bfloat162_rn(a, b);
                  h2[j] = __floats2bfloat162_rn(apply_act(a, p.act), apply_act(b, p.act));
                } else {
                  h[j] = __floats2bfloat162_rn(apply_act(a, p.act), apply_act(b, p.act));
                }
              }
              *reinterpret_cast<uint4*>(c + g * 8) = u;
              if (c2) *reinterpret_cast<uint4*>(c2 + g * 8) = u2;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < N) {
                if (c2) {
                  c[j] = __float2bfloat16(v[j]);
                  c2[j] = __float2bfloat16(apply_act(v[j], p.act));
                } else {
                  c[j] = __float2bfloat16(apply_act(v[j], p.act));
                }
              }
            }
          }
        }
      }
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

// ---- host side ----------------------------------------------------------------------------------------------------

}  // namespace

static int launch_gemm(const void* a, const void* b, long long a_rows, long long a_cols, long long b_rows, long long b_cols, int lda, int ldb,
                       GemmParams p, int grid_m, int grid_n, int batch, cudaStream_t stream) {
  if ((lda % 8) || (ldb % 8) || (((uintptr_t)a) & 15) || (((uintptr_t)b) & 15)) {
    rb_set_error("gemm: operands need 16-byte aligned bases and pitches that are multiples of 8 elements (lda %d ldb %d)", lda, ldb);
    return RB_ERR_ARG;
  }
  if (p.accumulate && !p.out_fp32) {
    rb_set_error("gemm: accumulate needs fp32 output");
    return RB_ERR_ARG;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      rb_set_error("gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return RB_ERR_LAUNCH;
    }
    attr_set = true;
  }
  CUtensorMap tm_a, tm_b;
  int st;
  // stored matrices: [a_rows][a_cols] and [b_rows][b_cols]; K-major box = {64 (k), 128 rows}; MN-major box = {64 (m/n), 64 k-rows}
  if (!p.a_mn_major) st = make_map(&tm_a, a, a_cols, a_rows, lda, BK, BM);
  else st = make_map(&tm_a, a, a_cols, a_rows, lda, 64, BK);
  if (st) return st;
  if (!p.b_mn_major) st = make_map(&tm_b, b, b_cols, b_rows, ldb, BK, BN);
  else st = make_map(&tm_b, b, b_cols, b_rows, ldb, 64, BK);
  if (st) return st;
  dim3 grid(grid_n, grid_m, batch);
  gemm_bf16_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tm_a, tm_b, p);
  return rb_check_launch("gemm_bf16");
}

// Batched form. Operands are 2-D stored matrices (rows x cols, row pitch ld*); problem z = b * heads + h reads A from the
// stored origin (b*a_rb + h*a_rh, b*a_cb + h*a_ch), B likewise, and writes C at element offset b*c_sb + h*c_sh.
// Extents m / n / k are fixed, or lens[b] where the corresponding *_from_lens flag is set. Tiles beyond a problem's
// extents exit at once. Stored data beyond an extent in the contraction direction must be zero (or finite on the other operand).
RB_EXPORT int rb200_gemm_bf16_batched(const void* a, const void* b, void* c, const void* bias, long long a_rows, long long a_cols,
                                      long long b_rows, long long b_cols, int lda, int ldb, int ldc, int m, int n, int k,
                                      int a_mn_major, int b_mn_major, int bias_bf16, int act, int out_fp32, int accumulate, float alpha,
                                      int batch, int heads, const long long* offs /*a_rb,a_rh,a_cb,a_ch,b_rb,b_rh,b_cb,b_ch,c_sb,c_sh*/,
                                      const int* lens, int m_from_lens, int n_from_lens, int k_from_lens, int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || batch <= 0) return RB_OK;
  static int legacy = -1;
  if (legacy < 0) {
    const char* e = getenv("RETURNN_B200_GEMM_KERNEL");
    legacy = (e && strcmp(e, "legacy") == 0) ? 1 : 0;
  }
  if (!legacy) {
    RbGemm g;
    g.a = a; g.b = b; g.c = c; g.bias = bias; g.bias_bf16 = bias_bf16;
    g.m = m; g.n = n; g.k = k; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
    g.a_mn_major = a_mn_major; g.b_mn_major = b_mn_major; g.act = act; g.out_fp32 = out_fp32; g.accumulate = accumulate; g.alpha = alpha;
    g.status = status;
    g.batch = batch; g.heads = heads > 0 ? heads : 1;
    g.a_rb = offs[0]; g.a_rh = offs[1]; g.a_cb = offs[2]; g.a_ch = offs[3];
    g.b_rb = offs[4]; g.b_rh = offs[5]; g.b_cb = offs[6]; g.b_ch = offs[7];
    g.c_sb = offs[8]; g.c_sh = offs[9];
    g.a_rows = a_rows; g.a_cols = a_cols; g.b_rows = b_rows; g.b_cols = b_cols;
    g.lens = lens; g.m_from_lens = m_from_lens; g.n_from_lens = n_from_lens; g.k_from_lens = k_from_lens;
    return rb_gemm(g, stream);
  }
  GemmParams p;
  p.c = c;
  p.c2 = nullptr;
  p.bias = bias;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = ldc;
  p.a_mn_major = a_mn_major;
  p.b_mn_major = b_mn_major;
  p.bias_bf16 = bias_bf16;
  p.act = act;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.alpha = alpha;
  p.status = status;
  p.heads = heads > 0 ? heads : 1;
  p.a_rb = offs[0]; p.a_rh = offs[1]; p.a_cb = offs[2]; p.a_ch = offs[3];
  p.b_rb = offs[4]; p.b_rh = offs[5]; p.b_cb = offs[6]; p.b_ch = offs[7];
  p.c_sb = offs[8]; p.c_sh = offs[9];
  p.lens = lens;
  p.m_from_lens = m_from_lens;
  p.n_from_lens = n_from_lens;
  p.k_from_lens = k_from_lens;
  return launch_gemm(a, b, a_rows, a_cols, b_rows, b_cols, lda, ldb, p, (m + BM - 1) / BM, (n + BN - 1) / BN, batch, stream);
}

// D[m,n] = alpha * op(A)·op(B) (+bias)(act).
//   a_mn_major = 0: A stored [m][k] with row pitch lda;  1: A stored [k][m] with row pitch lda
//   b_mn_major = 0: B stored [n][k] with row pitch ldb;  1: B stored [k][n] with row pitch ldb
// Requirements: base pointers 16-byte aligned, pitches multiples of 8 elements.
RB_EXPORT int rb200_gemm_bf16(const void* a, const void* b, void* c, void* c2, const void* bias, int m, int n, int k, int lda, int ldb,
                              int ldc, int a_mn_major, int b_mn_major, int bias_bf16, int act, int out_fp32, int accumulate, float alpha,
                              int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return RB_OK;
  if (k <= 0) {
    rb_set_error("gemm: k=%d", k);
    return RB_ERR_ARG;
  }
  GemmParams p;
  p.c = c;
  p.c2 = c2;
  p.bias = bias;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = ldc;
  p.a_mn_major = a_mn_major;
  p.b_mn_major = b_mn_major;
  p.bias_bf16 = bias_bf16;
  p.act = act;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.alpha = alpha;
  p.status = status;
  p.heads = 1;
  p.a_rb = p.a_rh = p.a_cb = p.a_ch = 0;
  p.b_rb = p.b_rh = p.b_cb = p.b_ch = 0;
  p.c_sb = p.c_sh = 0;
  p.lens = nullptr;
  p.m_from_lens = p.n_from_lens = p.k_from_lens = 0;
  long long a_rows = a_mn_major ? k : m, a_cols = a_mn_major ? m : k;
  long long b_rows = b_mn_major ? k : n, b_cols = b_mn_major ? n : k;
  return launch_gemm(a, b, a_rows, a_cols, b_rows, b_cols, lda, ldb, p, (m + BM - 1) / BM, (n + BN - 1) / BN, 1, stream);
}
