// Fused gradient all-reduce over NVLink peer memory for one node (2..8 GPUs, one process per GPU).
//
// One kernel per bucket does what otherwise takes a scale kernel, an NCCL all-reduce and a norm kernel:
//   1. entry barrier between the same-numbered CTAs of all ranks (flags in symmetric memory, release/acquire at system scope)
//   2. every rank owns one slice of the bucket: it sums that slice over all ranks
//        - plain path: 16-byte loads from each peer's buffer (peer pointers), rotated so that the ranks do not all hit
//          the same peer at once
//        - multimem path: one multimem.ld_reduce through the NVSwitch multicast mapping (the switch adds)
//      scales by 1/world, accumulates the sum of squares, and writes the result into every rank's buffer
//      (peer stores, or one multimem.st)
//   3. the sum of squares of the slice is added (system-scope atomics) to a norm accumulator on every rank, so that after the
//      last bucket every rank holds the squared global gradient norm without another pass or collective
//   4. exit barrier: all pushes have landed before any rank's next kernel reads its buffer
//
// Every wait is bounded twice over: by a time limit read from the GPU's global timer (rb200_collective_set_wait_ms, default 20 s:
// long enough for a peer that is late because of a lazy initialisation or a data stall, short enough that a dead peer does not
// hold the GPU) and by a poll count that follows from it. A CTA that gives up writes a status word and skips its data phase;
// the context stays usable and the host raises an error when it reads the word (once per training step, with the losses).
//
// Parameter-averaging mode (AdamW update, then average): the slices are interleaved instead of contiguous. With G = grid size
// x 512 threads, float4 number i is updated on every rank by CTA (i mod G) / 512, and it is reduced by rank (i / G) mod world,
// again in CTA (i mod G) / 512. So everything a CTA reads in the averaging phase, locally and on the peers, was written by
// the same-numbered CTA of that rank before that CTA signalled the entry barrier: the barrier between same-numbered CTAs is
// all the synchronisation the two phases need.
#include "common.cuh"
#include "adamw.cuh"
#include <cstring>

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 256;
constexpr int kThreads = 512;

// wait limit of the cross-rank barriers in nanoseconds (process-wide; set through rb200_collective_set_wait_ms)
unsigned long long g_wait_ns = 20ull * 1000 * 1000 * 1000;

struct ArParams {
  float* bufs[kMaxWorld];       // the gradient arena of every rank (bufs[rank] is local)
  uint32_t* flags[kMaxWorld];   // [world][kMaxBlocks] per rank: flags[dst][src * kMaxBlocks + block]
  float* norm[kMaxWorld];       // norm accumulator of every rank
  float* mc;                    // multicast mapping of the arena, or null
  int world, rank;
  long long lo, n;              // element range of the bucket
  float scale;
  uint32_t epoch;               // barrier values epoch (entry) and epoch + 1 (exit); grows by 2 per call on all ranks alike
  int norm_slot;
  int interleaved;              // 1: rank r owns float4 i with (i / G) % world == r (parameter-averaging mode), 0: contiguous slices
  unsigned long long wait_ns;   // time limit of a barrier wait
  int* status;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// barrier between CTA blockIdx.x of all ranks; false = a peer did not arrive in time
__device__ bool cta_barrier(const ArParams& p, uint32_t val, int* sh_fail, int code) {
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(p.flags[peer] + (size_t)p.rank * kMaxBlocks + blockIdx.x, val);
    const uint32_t* mine = p.flags[p.rank] + (size_t)peer * kMaxBlocks + blockIdx.x;
    bool ok = false;
    const unsigned long long t0 = global_timer_ns();
    // every poll after the first 64 sleeps about a microsecond: the poll count bounds the wait even if the timer stood still
    const unsigned long long max_polls = 64 + p.wait_ns / 500;
    for (unsigned long long i = 0; i < max_polls; ++i) {
      if ((int32_t)(ld_acquire_sys(mine) - val) >= 0) {
        ok = true;
        break;
      }
      if (i >= 64 && global_timer_ns() - t0 > p.wait_ns) break;
      __nanosleep(i < 64 ? 32 : 1000);
    }
    if (!ok) {
      *sh_fail = 1;
      if (p.status) atomicCAS(p.status, 0, (code << 24) | (peer << 16) | (int)(blockIdx.x & 0xFFFF));
    }
  }
  __syncthreads();
  return *sh_fail == 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce(const float* addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// With `adam` set (adam.p != null) the kernel first runs this rank's AdamW update over its whole parameter arena (p.bufs[rank] is
// then the parameter arena, not the gradient arena), and only then averages: the entry barrier doubles as "every rank has
// finished its update". This is the parameter-averaging mode (local steps, sync every N): update + average in one launch.
// T threads per CTA. The 128-thread form is capped at 80 registers: four such warps fit into what a resident GEMM CTA of the
// backward pass (18 warps x 96 registers, ~200 KB shared memory) leaves free on an SM, so a bucket reduction running next to the
// backward pass does not keep the CTAs of the next persistent GEMM off its SMs.
template <int U, int T>
__global__ void __launch_bounds__(T, T == 128 ? 6 : 1)
fused_allreduce_kernel(const ArParams p, const AdamwArgs adam) {
  constexpr int kThreads = T;  // shadows the file-level default inside this kernel
  __shared__ int sh_fail;
  __shared__ float sh_red[kThreads / 32];
  if (threadIdx.x == 0) sh_fail = 0;
  if (adam.p != nullptr) {
    adamw_update_range(adam, (int64_t)blockIdx.x * kThreads + threadIdx.x, (int64_t)gridDim.x * kThreads);
  }
  if (!cta_barrier(p, p.epoch, &sh_fail, 1)) return;

  // slices of whole float4s; the tail (n % 4 elements) belongs to the last rank
  const long long n4 = p.n / 4;
  const long long per = (n4 + p.world - 1) / p.world;
  const long long grid_threads = (long long)gridDim.x * kThreads;
  // contiguous mode: this rank's slice [s0, s1), consecutive iterations one grid apart
  // interleaved mode: grid-sized chunks dealt out to the ranks in turn, consecutive iterations `world` grids apart
  const long long s0 = p.interleaved ? (long long)p.rank * grid_threads : (per * p.rank < n4 ? per * p.rank : n4);
  const long long s1 = p.interleaved ? n4 : (s0 + per < n4 ? s0 + per : n4);
  float ssq = 0.f;
  const long long stride = p.interleaved ? grid_threads * p.world : grid_threads;
  // U float4 per thread and iteration: all loads of an iteration are issued before the first use, which keeps enough bytes in
  // flight to cover the NVLink round trip. A bucket reduction overlaps the backward pass and takes the SMs of its CTAs away from
  // it for its whole duration (it is bound by the link, not by the SM), so the deeper unroll with FEWER CTAs is the better
  // neighbour: the bytes in flight per GPU stay the same, on a quarter of the SMs.
  for (long long i0 = s0 + (long long)blockIdx.x * kThreads + threadIdx.x; i0 < s1; i0 += U * stride) {
    float4 acc[U];
    if (p.mc) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < s1) acc[u] = multimem_ld_reduce(p.mc + p.lo + i * 4);
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int k = 0; k < p.world; ++k) {
        const int peer = (p.rank + k) % p.world;
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          v[u] = i < s1 ? *reinterpret_cast<const float4*>(p.bufs[peer] + p.lo + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= s1) break;
      const long long e = p.lo + i * 4;
      float4 a = acc[u];
      a.x *= p.scale; a.y *= p.scale; a.z *= p.scale; a.w *= p.scale;
      ssq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      if (p.mc) {
        multimem_st(p.mc + e, a);
      } else {
#pragma unroll 1
        for (int k = 0; k < p.world; ++k) {
          const int peer = (p.rank + k) % p.world;
          *reinterpret_cast<float4*>(p.bufs[peer] + e) = a;
        }
      }
    }
  }
  if (p.rank == p.world - 1 && blockIdx.x == 0 && threadIdx.x < (p.n & 3)) {
    const long long e = p.lo + n4 * 4 + threadIdx.x;
    float acc = 0.f;
    for (int k = 0; k < p.world; ++k) acc += p.bufs[k][e];
    acc *= p.scale;
    ssq += acc * acc;
    for (int k = 0; k < p.world; ++k) p.bufs[k][e] = acc;
  }
  // sum of squares of this CTA's share -> every rank's accumulator
  ssq = warp_sum(ssq);
  if ((threadIdx.x & 31) == 0) sh_red[threadIdx.x >> 5] = ssq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? sh_red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0 && v != 0.f) {
      for (int k = 0; k < p.world; ++k) atomicAdd_system(p.norm[k] + p.norm_slot, v);
    }
  }
  cta_barrier(p, p.epoch + 1, &sh_fail, 2);
}

}  // namespace

// bufs / flags / norm: arrays of `world` device addresses (one per rank, index = rank). The flag buffers hold
// world * 256 zero-initialised uint32. epoch: 1, 3, 5, ... identical on all ranks for the same call.
RB_EXPORT int rb200_fused_allreduce(const long long* bufs, const long long* flags, const long long* norm, void* multicast, int world, int rank,
                                    long long lo, long long n, float scale, unsigned int epoch, int norm_slot, int blocks, int* status,
                                    cudaStream_t stream) {
  if (world < 2 || world > kMaxWorld || rank < 0 || rank >= world) {
    rb_set_error("fused_allreduce: world %d rank %d", world, rank);
    return RB_ERR_ARG;
  }
  if (n <= 0) return RB_OK;
  if (lo % 4) {
    rb_set_error("fused_allreduce: bucket start %lld must be a multiple of 4 elements", lo);
    return RB_ERR_ARG;
  }
  ArParams p;
  for (int i = 0; i < kMaxWorld; ++i) {
    p.bufs[i] = i < world ? reinterpret_cast<float*>(bufs[i]) : nullptr;
    p.flags[i] = i < world ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
    p.norm[i] = i < world ? reinterpret_cast<float*>(norm[i]) : nullptr;
  }
  p.mc = reinterpret_cast<float*>(multicast);
  p.world = world;
  p.rank = rank;
  p.lo = lo;
  p.n = n;
  p.scale = scale;
  p.epoch = epoch;
  p.norm_slot = norm_slot;
  p.interleaved = 0;
  p.wait_ns = g_wait_ns;
  p.status = status;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  AdamwArgs none;
  memset(&none, 0, sizeof(none));
  static int unroll = 0, threads = 0;
  if (!unroll) {
    const char* e = getenv("RETURNN_B200_ALLREDUCE_UNROLL");
    unroll = e ? atoi(e) : 4;
    if (unroll != 4 && unroll != 8 && unroll != 16) unroll = 4;
    const char* t = getenv("RETURNN_B200_ALLREDUCE_THREADS");
    threads = t && atoi(t) == 128 ? 128 : kThreads;
  }
  if (threads == 128) {
    if (unroll == 4) fused_allreduce_kernel<4, 128><<<blocks, 128, 0, stream>>>(p, none);
    else fused_allreduce_kernel<8, 128><<<blocks, 128, 0, stream>>>(p, none);
  } else if (unroll == 16) {
    fused_allreduce_kernel<16, kThreads><<<blocks, kThreads, 0, stream>>>(p, none);
  } else if (unroll == 8) {
    fused_allreduce_kernel<8, kThreads><<<blocks, kThreads, 0, stream>>>(p, none);
  } else {
    fused_allreduce_kernel<4, kThreads><<<blocks, kThreads, 0, stream>>>(p, none);
  }
  return rb_check_launch("fused_allreduce");
}

// Parameter averaging fused with the optimizer update: AdamW on this rank's parameters (arguments as rb200_adamw_arena), then the
// average over all ranks written to every rank. bufs: the parameter arenas (symmetric memory).
RB_EXPORT int rb200_fused_adamw_param_avg(const long long* bufs, const long long* flags, const long long* norm, void* multicast, int world, int rank,
                                          long long n, unsigned int epoch, int blocks, int* status, const void* g, float* m, float* v,
                                          const uint8_t* wd_flags, int g_bf16, float lr, float b1, float b2, float eps, float wd, float bc1,
                                          float bc2, int decoupled, float clip, const float* grad_norm, int do_update, cudaStream_t stream) {
  if (world < 2 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0 || n % 4 != 0) {
    rb_set_error("fused_adamw_param_avg: world %d rank %d n %lld (n must be a positive multiple of 4)", world, rank, n);
    return RB_ERR_ARG;
  }
  ArParams p;
  for (int i = 0; i < kMaxWorld; ++i) {
    p.bufs[i] = i < world ? reinterpret_cast<float*>(bufs[i]) : nullptr;
    p.flags[i] = i < world ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
    p.norm[i] = i < world ? reinterpret_cast<float*>(norm[i]) : nullptr;
  }
  p.mc = reinterpret_cast<float*>(multicast);
  p.world = world;
  p.rank = rank;
  p.lo = 0;
  p.n = n;
  p.scale = 1.f / (float)world;
  p.epoch = epoch;
  p.norm_slot = 7;  // unused accumulator slot
  p.interleaved = 1;
  p.wait_ns = g_wait_ns;
  p.status = status;
  AdamwArgs a;
  memset(&a, 0, sizeof(a));
  if (do_update) {
    a = AdamwArgs{p.bufs[rank], g, m, v, wd_flags, (int64_t)n, g_bf16, lr, b1, b2, eps, wd, bc1, bc2, decoupled, clip, grad_norm, nullptr};
  }
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  fused_allreduce_kernel<4, kThreads><<<blocks, kThreads, 0, stream>>>(p, a);
  return rb_check_launch("fused_adamw_param_avg");
}

RB_EXPORT int rb200_fused_allreduce_flag_words() { return kMaxWorld * kMaxBlocks; }

// Time limit of every cross-rank barrier wait of the kernels in this file, for launches made after this call (1 ms .. 10 min).
RB_EXPORT int rb200_collective_set_wait_ms(int ms) {
  if (ms < 1 || ms > 600000) {
    rb_set_error("collective_set_wait_ms: %d is outside 1..600000", ms);
    return RB_ERR_ARG;
  }
  g_wait_ns = (unsigned long long)ms * 1000000ull;
  return RB_OK;
}
