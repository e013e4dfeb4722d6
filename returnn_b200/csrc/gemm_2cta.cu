// CTA-pair variant of the persistent bf16 GEMM: two CTAs of a cluster (two SMs) compute one 256 x 256 output tile with
// tcgen05.mma.cta_group::2. Each CTA loads its own 128 rows of A and half of the B tile, so a pair moves 64 KB per K block for
// 256 x 256 x 64 multiply-adds: two thirds of the L2->SM operand traffic per flop of the one-CTA kernel (128 x 256 tiles, 48 KB per
// CTA and K block), which is what bounds that kernel (measured: time per K block independent of the tile width, scaling with the
// number of active SMs).
//
// Roles per CTA: warp 0 = TMA producer (loads with .cta_group::2 and no multicast; they complete on the *leader's* full barrier,
// which is armed for the bytes of both CTAs), warp 1 = TMEM allocation, and in the leader CTA (cluster rank 0) the MMA issuer,
// warps 2-17 = epilogue of the CTA's own 128 accumulator rows (tensor memory is per SM): every lane owns one row, reads 64 columns of
// it from tensor memory, and the results leave through a swizzled box in shared memory and one bulk tensor store per warp (bulk
// reduce-add for the accumulating fp32 outputs of the weight gradients); see epilogue_rows_tma. Outputs that a tensor map cannot
// describe (unaligned pitch or base) take the per-lane st.global path. tcgen05.commit with a cluster
// multicast mask releases a ring stage / publishes an accumulator in both CTAs at once; the epilogue warps of both CTAs arrive on
// the leader's "accumulator free" barrier. All waits are bounded; a CTA never exits before its peer (cluster barrier at the end),
// because the leader's MMAs read the peer's shared memory.
#include "gemm_epilogue.cuh"
#include <cstdlib>
#include <cstring>

using namespace rbt;
using namespace rbg;

namespace {

constexpr int BM = 256;              // per pair; 128 per CTA
constexpr int BN = 256;
constexpr int kThreads = kGemmThreads;
constexpr int kTileBytesA = 128 * BK * 2;        // 16 KB: this CTA's rows of A
constexpr int kTileBytesB = (BN / 2) * BK * 2;   // 16 KB: this CTA's half of B
constexpr int kStageBytes = kTileBytesA + kTileBytesB;
constexpr int kStages = 5;
constexpr int kRingBytes = kStages * kStageBytes;  // 160 KB
constexpr int kStagingBytes = kEpilogueWarps * kStoreBoxBytesPerWarp;  // 64 KB: one 4 KB store box per epilogue warp (1024-byte aligned)
static_assert(kStoreBoxBytesPerWarp >= kStagingBytesPerWarp, "the st.global path stages in the same area");
constexpr int kSmemBytes = kRingBytes + kStagingBytes + 256 + 1024;
constexpr uint32_t kTmemCols = 2 * BN;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs once the pair's MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

template <bool FULL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                 const __grid_constant__ CUtensorMap tm_c2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* staging = reinterpret_cast<float*>(smem + kRingBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kRingBytes + kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const RbGemm& g = p.g;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);   // leader: one expect_tx arrival per use, both CTAs' bytes
      mbar_init(&empty_bar[s], 1);  // one multicast commit per use
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * kEpilogueWarps);  // leader: the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // barriers of both CTAs are initialised before anyone signals across
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: it may overlap the tail of the preceding kernel
  rb_pdl_wait();
  rb_pdl_launch();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (both CTAs) ----------------
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < p.units && ok; u += n_pairs) {
        const Unit w = decode_unit<BM, BN>(p, u);
        if (!w.valid) continue;
        const int m0 = w.m0 + (int)rank * 128;
        const int n0 = w.n0 + (int)rank * (BN / 2);
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
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);  // the leader's barrier collects both CTAs' bytes
          if (leader) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);
          const int k0 = kb * BK;
          if (!g.a_mn_major) {
            tma_load_2d_pair(sa, &tm_a, k0, m0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &tm_a, m0 + 64 * j, k0, bar);
          }
          if (!g.b_mn_major) {
            tma_load_2d_pair(sb, &tm_b, k0, n0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * 8192, &tm_b, n0 + 64 * j, k0, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (leader CTA only) ----------------
      const uint32_t ab_fmt = g.ab_fp16 ? 0u : 1u;  // operand format field: 0 = fp16, 1 = bf16 (accumulator fp32 either way)
      const uint32_t idesc = (1u << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((uint32_t)(g.a_mn_major ? 1 : 0) << 15) |
                             ((uint32_t)(g.b_mn_major ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int u = pair; u < p.units && ok; u += n_pairs) {
        const Unit w = decode_unit<BM, BN>(p, u);
        if (!w.valid) continue;
        const uint32_t buf = t_local & 1u;
        if (!mbar_wait(&acc_empty[buf], ((t_local >> 1) & 1u) ^ 1u, abort_flag)) {
          *abort_flag = 1;
          if (g.status) atomicCAS(g.status, 0, (4 << 24) | (u & 0xFFFFFF));
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
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
            const uint64_t adesc = g.a_mn_major ? make_desc(sa + kk * 2048, 8192, 1024) : make_desc(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = g.b_mn_major ? make_desc(sb + kk * 2048, 8192, 1024) : make_desc(sb + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s]);
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
        ++t_local;
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 rows ----------------
    const int q = warp & 3;
    uint8_t* box = reinterpret_cast<uint8_t*>(staging) + (warp - 2) * kStoreBoxBytesPerWarp;
    float* stg = reinterpret_cast<float*>(box);
    uint32_t t_local = 0;
    for (int u = pair; u < p.units; u += n_pairs) {
      const Unit w = decode_unit<BM, BN>(p, u);
      if (!w.valid) continue;
      const int m0 = w.m0 + (int)rank * 128, n0 = w.n0;
      const uint32_t buf = t_local & 1u;
      const int part = (warp - 2) >> 2;  // four warps per lane quarter, each with a quarter of the columns
      // the epilogue's global input of this lane's row (first 16 columns) is requested before the wait: it arrives while the tile is
      // still multiplied
      uint4 in_a = make_uint4(0u, 0u, 0u, 0u), in_b = in_a;
      const bool prefetched = FULL && p.tma_store && (g.dact_z != nullptr || g.resid != nullptr);
      if (prefetched) epilogue_prefetch16(p, w.M, w.N, m0 + q * 32 + lane, n0 + part * (BN / 4), in_a, in_b);
      bool ok = mbar_wait(&acc_full[buf], (t_local >> 1) & 1u, abort_flag);
      if (!ok && lane == 0) {
        *abort_flag = 1;
        if (g.status) atomicCAS(g.status, 0, (3 << 24) | (u & 0xFFFFFF));
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      auto release = [&]() { mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0)); };
      if (p.tma_store) epilogue_rows_tma<FULL>(p, w, m0, n0, t_addr, part * (BN / 4), box, &tm_c, &tm_c2, lane, q, release, in_a, in_b, prefetched);
      else epilogue_columns<FULL>(p, w, m0, n0, t_addr, part * (BN / 4), (part + 1) * (BN / 4), stg, lane, q, release);
      ++t_local;
    }
    // the bulk stores read this CTA's shared memory: the reads must have finished before the CTA exits and its shared memory is
    // handed to another CTA (the writes themselves complete like any other store of the grid)
    if (p.tma_store && lane == 0) tma_store_wait_read();
  }

  // ---------------- teardown ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (uint32_t i = 0; i < (1u << 12); ++i) __nanosleep(256);
  }
  __syncthreads();
  cluster_sync();  // the peer's MMAs and barrier signals may still touch this CTA's shared memory until here
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

}  // namespace

// whether rb_gemm should route this problem to the CTA-pair kernel
bool rb_gemm_pair_wanted(const RbGemm& g) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("RETURNN_B200_GEMM_2CTA");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  return enabled && g.batch == 0 && g.m > 128 && g.n > 128;
}

int rb_gemm_pair(const RbGemm& g, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      rb_set_error("gemm (pair): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
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
  const int pairs_max = num_sms() / 2;
  int split = 1;
  if (g.accumulate == 2) {
    split = g.split_k > 0 ? g.split_k : (tiles >= pairs_max ? 1 : pairs_max / tiles);
    const int max_split = p.num_kb >= 4 ? p.num_kb / 4 : 1;
    if (split > max_split) split = max_split;
    if (split < 1) split = 1;
  }
  p.kb_per_split = (p.num_kb + split - 1) / split;
  p.split = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.units = tiles * p.split;
  auto al16 = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  p.vec_ok = (g.ldc % 8 == 0) && al16(g.c) && al16(g.c2) && al16(g.resid) && al16(g.dact_z);
  p.bias_vec = g.bias != nullptr && !g.bias_bf16 && al16(g.bias);
  const bool full = g.dact_z != nullptr || g.drop_p > 0.f || g.resid != nullptr;
  static int tma_store_enabled = -1;
  if (tma_store_enabled < 0) {
    const char* e = getenv("RETURNN_B200_GEMM_TMA_STORE");
    tma_store_enabled = (e && e[0] == '0') ? 0 : 1;
  }
  // bulk tensor stores need what a tensor map needs: 16-byte aligned base, row pitch a multiple of 16 bytes
  p.tma_store = tma_store_enabled && p.vec_ok && g.c != nullptr && (g.out_fp32 ? true : (g.ldc % 8 == 0));
  CUtensorMap tm_a, tm_b, tm_c, tm_c2;
  memset(&tm_c, 0, sizeof(tm_c));
  memset(&tm_c2, 0, sizeof(tm_c2));
  int st;
  if (p.tma_store) {
    // boxes of 32 rows x 128 bytes: 64 bf16 or 32 fp32 columns; with a second output, 32 rows x 64 bytes (32 bf16 columns) each
    if (g.c2) {
      st = make_map(&tm_c, g.c, g.n, g.m, g.ldc, 32, 32, false, true);
      if (st) return st;
      st = make_map(&tm_c2, g.c2, g.n, g.m, g.ldc, 32, 32, false, true);
    } else {
      st = make_map(&tm_c, g.c, g.n, g.m, g.ldc, g.out_fp32 ? 32 : 64, 32, g.out_fp32 != 0);
    }
    if (st) return st;
  }
  const long long a_rows = g.a_mn_major ? g.k : g.m, a_cols = g.a_mn_major ? g.m : g.k;
  const long long b_rows = g.b_mn_major ? g.k : g.n, b_cols = g.b_mn_major ? g.n : g.k;
  st = g.a_mn_major ? make_map(&tm_a, g.a, a_cols, a_rows, g.lda, 64, BK) : make_map(&tm_a, g.a, a_cols, a_rows, g.lda, BK, 128);
  if (st) return st;
  st = g.b_mn_major ? make_map(&tm_b, g.b, b_cols, b_rows, g.ldb, 64, BK) : make_map(&tm_b, g.b, b_cols, b_rows, g.ldb, BK, BN / 2);
  if (st) return st;
  int pairs = p.units < pairs_max ? p.units : pairs_max;
  if (full) rb_launch_pdl(gemm_pair_kernel<true>, dim3(2 * pairs), dim3(kThreads), kSmemBytes, stream, tm_a, tm_b, tm_c, tm_c2, p);
  else rb_launch_pdl(gemm_pair_kernel<false>, dim3(2 * pairs), dim3(kThreads), kSmemBytes, stream, tm_a, tm_b, tm_c, tm_c2, p);
  return rb_check_launch("gemm_pair");
}
