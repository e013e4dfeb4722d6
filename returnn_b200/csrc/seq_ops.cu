// Sequence-level utility kernels:
//   - device assert without a trap: a failed condition writes (code, index) to a status word that the host polls
//   - edit distance between batched label sequences (one warp per pair, anti-diagonal free: row DP in registers/shared)
//   - beam-search step: log-softmax over the vocabulary + accumulated scores + top-k over beam x vocabulary, one CTA per batch entry
//   - RNN-T loss (forward-backward over the T x U lattice, one CTA per sequence, anti-diagonal wavefront) with gradients
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------------------------
// device assert: status[0] = code, status[1] = first failing index (both stay 0 when everything holds)
__global__ void assert_kernel(const uint8_t* __restrict__ cond, long long n, int* __restrict__ status, int code) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if (!cond[i]) {
      if (atomicCAS(status, 0, code) == 0) status[1] = (int)(i < 0x7fffffff ? i : 0x7fffffff);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// edit distance: a [B, La] and b [B, Lb] int32 (padded), lengths per row; out [B] int32. One warp per pair: lane-strided over
// the columns of the DP row held in shared memory, row by row with a prefix-min fix-up for the insertion chain.
constexpr int kEdMaxLen = 2048;

__global__ void __launch_bounds__(128)
edit_distance_kernel(const int* __restrict__ a, const int* __restrict__ a_len, int lda, const int* __restrict__ b, const int* __restrict__ b_len,
                     int ldb, int* __restrict__ out, int batch) {
  extern __shared__ int sh[];  // per warp: 2 rows of (kEdMaxLen + 1)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (blockDim.x >> 5) + warp;
  if (pair >= batch) return;
  int* prev = sh + warp * 2 * (kEdMaxLen + 1);
  int* cur = prev + (kEdMaxLen + 1);
  const int n = a_len[pair], m = b_len[pair];
  const int* sa = a + (size_t)pair * lda;
  const int* sb = b + (size_t)pair * ldb;
  for (int j = lane; j <= m; j += 32) prev[j] = j;
  __syncwarp();
  for (int i = 1; i <= n; ++i) {
    const int ai = sa[i - 1];
    // substitution / deletion candidates are independent per column
    for (int j = lane; j <= m; j += 32) {
      int v = i;
      if (j > 0) {
        const int sub = prev[j - 1] + (ai == sb[j - 1] ? 0 : 1);
        const int del = prev[j] + 1;
        v = sub < del ? sub : del;
      }
      cur[j] = v;
    }
    __syncwarp();
    // insertion chain: cur[j] = min(cur[j], cur[j-1] + 1) is a prefix-min of (cur[j] - j) plus j
    int carry = INT_MAX / 2;
    for (int j0 = 0; j0 <= m; j0 += 32) {
      const int j = j0 + lane;
      int v = j <= m ? cur[j] - j : INT_MAX / 2;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o && u < v) v = u;
      }
      if (carry < v) v = carry;
      if (j <= m) cur[j] = v + j;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
    __syncwarp();
    int* t = prev;
    prev = cur;
    cur = t;
  }
  if (lane == 0) out[pair] = prev[m];
}

// ---------------------------------------------------------------------------------------------------------------------
// beam step. logits [B, beam, V] (fp32 or bf16, unnormalised unless normalized != 0), prev_scores [B, beam] fp32,
// finished [B, beam] uint8 (optional): a finished hypothesis only continues with eos, at unchanged score.
// out_scores [B, K] fp32, out_backref [B, K] int32 (beam index), out_label [B, K] int32; K <= 32.
constexpr int kTopkMaxK = 32;
constexpr int kTopkThreads = 256;

struct Cand {
  float s;
  int idx;
};

// Two kernels. (1) One CTA per hypothesis row [V] selects the row's K best logits and computes its log-sum-exp; the candidates
// leave as (prev + logit - lse, h * V + v), sorted. B * beam CTAs fill the machine where one CTA per batch entry left most SMs idle.
// Selection by threshold instead of by sorting: the 256 threads form K groups, every group finds the maximum of its elements; the
// smallest of these K maxima is a lower bound of the row's K-th largest element (K distinct elements are >= it), so only elements
// >= that bound can be among the K best. They are few (a few times K for unstructured data): the threads append them to a list in
// shared memory and the list is ranked by counting.
// A row where more than kTopkCap elements pass (many equal values) takes K rounds of a block-wide argmax instead.
// (2) One warp per batch entry merges the beam sorted lists.
constexpr int kTopkCap = 1024;

__device__ __forceinline__ bool cand_before(float sa, int ia, float sb, int ib) {  // order: score descending, index ascending
  return sa > sb || (sa == sb && ia < ib);
}

template <typename F>
__device__ __forceinline__ void for_each_in_row(const void* logits, int is_bf16, size_t row, int V, F&& visit) {
  if (is_bf16) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(logits) + row * V;
    const int mis = (int)((reinterpret_cast<uintptr_t>(p) & 15) >> 1);
    const int head = min(V, (8 - mis) & 7);  // elements before the first 16-byte boundary
    for (int v = threadIdx.x; v < head; v += kTopkThreads) visit(__bfloat162float(p[v]), v);
    const int n_vec = (V - head) >> 3;
    const uint4* pv = reinterpret_cast<const uint4*>(p + head);
    for (int q = threadIdx.x; q < n_vec; q += kTopkThreads) {
      const uint4 u = __ldg(pv + q);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        visit(__uint_as_float(w[e] << 16), head + q * 8 + 2 * e);
        visit(__uint_as_float(w[e] & 0xffff0000u), head + q * 8 + 2 * e + 1);
      }
    }
    for (int v = head + n_vec * 8 + threadIdx.x; v < V; v += kTopkThreads) visit(__bfloat162float(p[v]), v);
  } else {
    const float* p = reinterpret_cast<const float*>(logits) + row * V;
    const int mis = (int)((reinterpret_cast<uintptr_t>(p) & 15) >> 2);
    const int head = min(V, (4 - mis) & 3);
    for (int v = threadIdx.x; v < head; v += kTopkThreads) visit(p[v], v);
    const int n_vec = (V - head) >> 2;
    const float4* pv = reinterpret_cast<const float4*>(p + head);
    for (int q = threadIdx.x; q < n_vec; q += kTopkThreads) {
      const float4 u = __ldg(pv + q);
      visit(u.x, head + q * 4);
      visit(u.y, head + q * 4 + 1);
      visit(u.z, head + q * 4 + 2);
      visit(u.w, head + q * 4 + 3);
    }
    for (int v = head + n_vec * 4 + threadIdx.x; v < V; v += kTopkThreads) visit(p[v], v);
  }
}

__global__ void __launch_bounds__(kTopkThreads)
beam_topk_row_kernel(const void* __restrict__ logits, int is_bf16, int normalized, const float* __restrict__ prev_scores,
                     const uint8_t* __restrict__ finished, int beam, int V, int eos, int K, Cand* __restrict__ cands) {
  __shared__ float sh_m[kTopkThreads / 32], sh_s[kTopkThreads / 32];
  __shared__ float sh_gmax[kTopkMaxK];
  __shared__ Cand sh_c[kTopkCap];
  __shared__ float sh_lse;
  __shared__ int sh_cnt;
  __shared__ Cand sh_best[kTopkThreads / 32];
  const int row = blockIdx.x;  // b * beam + h
  const int h = row % beam;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Cand* out = cands + (size_t)row * K;
  const float prev = prev_scores[row];
  if (finished && finished[row]) {  // only continuation: eos at unchanged score
    if (threadIdx.x < K) {
      out[threadIdx.x].s = threadIdx.x == 0 ? prev : -INFINITY;
      out[threadIdx.x].idx = threadIdx.x == 0 ? h * V + eos : -1;
    }
    return;
  }
  // pass 1: this thread's maximum, and the log-sum-exp
  float mx = -INFINITY, sum = 0.f;
  for_each_in_row(logits, is_bf16, (size_t)row, V, [&](float x, int) {
    if (x > mx) {
      sum = sum * __expf(mx - x) + 1.f;
      mx = x;
    } else {
      sum += __expf(x - mx);
    }
  });
  {
    const int g = kTopkThreads / K;  // threads per group: 32, 16 or 8 (K is 8, 16 or 32), so a group lies within a warp
    float gm = mx;
    for (int o = g >> 1; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
    if ((threadIdx.x & (g - 1)) == 0) sh_gmax[threadIdx.x / g] = gm;
  }
  if (threadIdx.x == 0) sh_cnt = 0;
  float wm = mx, ws = sum;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, wm, o), os = __shfl_xor_sync(0xffffffffu, ws, o);
    const float nm = fmaxf(wm, om);
    ws = (wm == -INFINITY ? 0.f : ws * __expf(wm - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    wm = nm;
  }
  if (lane == 0) {
    sh_m[warp] = wm;
    sh_s[warp] = ws;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = sh_m[0], sm = sh_s[0];
    for (int w = 1; w < kTopkThreads / 32; ++w) {
      const float om = sh_m[w], os = sh_s[w];
      const float nm = fmaxf(m, om);
      sm = (m == -INFINITY ? 0.f : sm * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    sh_lse = normalized ? 0.f : m + __logf(sm);
  }
  __syncthreads();
  float theta = sh_gmax[0];
  for (int j = 1; j < K; ++j) theta = fminf(theta, sh_gmax[j]);
  // pass 2 (the row comes from L1 / L2 now): collect everything >= theta
  for_each_in_row(logits, is_bf16, (size_t)row, V, [&](float x, int v) {
    if (x >= theta) {
      const int pos = atomicAdd(&sh_cnt, 1);
      if (pos < kTopkCap) {
        sh_c[pos].s = x;
        sh_c[pos].idx = v;
      }
    }
  });
  __syncthreads();
  const int M = sh_cnt;
  const float lse = sh_lse;
  if (M <= kTopkCap) {
    for (int c = threadIdx.x; c < M; c += kTopkThreads) {
      const float x = sh_c[c].s;
      const int v = sh_c[c].idx;
      int before = 0;
      for (int j = 0; j < M; ++j) before += cand_before(sh_c[j].s, sh_c[j].idx, x, v) ? 1 : 0;
      if (before < K) {
        out[before].s = prev + x - lse;
        out[before].idx = h * V + v;
      }
    }
    for (int r = M + threadIdx.x; r < K; r += kTopkThreads) {  // fewer than K elements in the row
      out[r].s = -INFINITY;
      out[r].idx = -1;
    }
    return;
  }
  // many equal values: K rounds, each the best element that comes after the previous winner in (score desc, index asc) order
  float last_s = INFINITY;
  int last_i = -1;
  for (int r = 0; r < K; ++r) {
    float bs = -INFINITY;
    int bi = 0x7fffffff;
    for_each_in_row(logits, is_bf16, (size_t)row, V, [&](float x, int v) {
      const bool after_last = x < last_s || (x == last_s && v > last_i);
      if (after_last && cand_before(x, v, bs, bi)) {
        bs = x;
        bi = v;
      }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (cand_before(os, oi, bs, bi)) {
        bs = os;
        bi = oi;
      }
    }
    if (lane == 0) {
      sh_best[warp].s = bs;
      sh_best[warp].idx = bi;
    }
    __syncthreads();
    bs = sh_best[0].s;
    bi = sh_best[0].idx;
    for (int w = 1; w < kTopkThreads / 32; ++w) {
      if (cand_before(sh_best[w].s, sh_best[w].idx, bs, bi)) {
        bs = sh_best[w].s;
        bi = sh_best[w].idx;
      }
    }
    __syncthreads();
    const bool found = bi != 0x7fffffff;
    if (threadIdx.x == 0) {
      out[r].s = found ? prev + bs - lse : -INFINITY;
      out[r].idx = found ? h * V + bi : -1;
    }
    last_s = found ? bs : -INFINITY;
    last_i = found ? bi : 0x7fffffff;
  }
}

// one warp per batch entry: lane l owns the sorted lists of hypotheses l and l + 32; k_out rounds of a warp-wide argmax over the heads
__global__ void __launch_bounds__(32)
beam_topk_merge_kernel(const Cand* __restrict__ cands, int beam, int K, int V, float* __restrict__ out_scores, int* __restrict__ out_backref,
                       int* __restrict__ out_label, int k_out) {
  const int b = blockIdx.x, lane = threadIdx.x;
  const Cand* base = cands + (size_t)b * beam * K;
  int hd0 = 0, hd1 = 0;
  for (int r = 0; r < k_out; ++r) {
    float s0 = -INFINITY, s1 = -INFINITY;
    int i0 = -1, i1 = -1;
    if (lane < beam && hd0 < K) {
      const Cand c = base[(size_t)lane * K + hd0];
      s0 = c.s;
      i0 = c.idx;
    }
    if (lane + 32 < beam && hd1 < K) {
      const Cand c = base[(size_t)(lane + 32) * K + hd1];
      s1 = c.s;
      i1 = c.idx;
    }
    const bool second = i1 >= 0 && (i0 < 0 || s1 > s0);
    float ms = second ? s1 : s0;
    int mi = second ? i1 : i0;
    if (mi < 0) ms = -INFINITY;
    int ml = mi >= 0 ? lane : 64;
    float bs = ms;
    int bl = ml;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int ol = __shfl_xor_sync(0xffffffffu, bl, o);
      if (ol < 64 && (bl >= 64 || os > bs || (os == bs && ol < bl))) {
        bs = os;
        bl = ol;
      }
    }
    bs = __shfl_sync(0xffffffffu, bs, 0);
    bl = __shfl_sync(0xffffffffu, bl, 0);
    int widx = -1;
    if (bl < 64) {
      widx = __shfl_sync(0xffffffffu, mi, bl);
      if (lane == bl) {
        if (second) ++hd1; else ++hd0;
      }
    }
    if (lane == 0) {
      out_scores[(size_t)b * k_out + r] = widx >= 0 ? bs : -INFINITY;
      out_backref[(size_t)b * k_out + r] = widx >= 0 ? widx / V : 0;
      out_label[(size_t)b * k_out + r] = widx >= 0 ? widx % V : 0;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// RNN-T loss. lp_blank [B, T, U1] and lp_label [B, T, U1] fp32 log-probabilities of emitting blank / the next label at lattice
// node (t, u), U1 = max label length + 1 (lp_label[.., u] for u == len is ignored). One CTA per sequence; alpha and beta live in
// global scratch [B, T, U1] each; anti-diagonals are processed in parallel. Gradients w.r.t. both inputs are written when
// requested: d lp_blank(t,u) = -exp(alpha(t,u) + lp_blank(t,u) + beta(t+1,u) - logZ), likewise for labels.
__device__ __forceinline__ float log_add(float a, float b) {
  if (a == -INFINITY) return b;
  if (b == -INFINITY) return a;
  const float m = fmaxf(a, b);
  return m + __logf(__expf(a - m) + __expf(b - m));
}

__global__ void __launch_bounds__(256)
rnnt_kernel(const float* __restrict__ lp_blank, const float* __restrict__ lp_label, const int* __restrict__ t_lens, const int* __restrict__ u_lens,
            int T, int U1, float* __restrict__ alpha, float* __restrict__ beta, float* __restrict__ loss, float* __restrict__ d_blank,
            float* __restrict__ d_label) {
  const int b = blockIdx.x;
  const int Tb = t_lens[b], Ub = u_lens[b] + 1;  // lattice is Tb x Ub
  const size_t off = (size_t)b * T * U1;
  const float* pb = lp_blank + off;
  const float* pl = lp_label + off;
  float* al = alpha + off;
  float* be = beta + off;
  if (Tb <= 0) {
    if (threadIdx.x == 0) loss[b] = 0.f;
    return;
  }
  // The forward and the backward recursion are independent: they run at the same time in the two halves of the CTA, each half
  // with its own named barrier. A lattice node needs its two predecessors, which both lie on the previous anti-diagonal: that
  // diagonal is kept in shared memory (indexed by u), so the dependent chain of a step is shared memory -> log-add -> barrier and
  // global memory is only written inside the loops (and read for the log-probabilities, which do not depend on the chain).
  extern __shared__ float rsm[];  // [4][U1]: previous / current diagonal of alpha and of beta
  const int half = blockDim.x >> 1;
  const int dir = threadIdx.x >= half ? 1 : 0;
  const int lt = threadIdx.x - dir * half;
  float* prev = rsm + dir * 2 * U1;
  float* cur = prev + U1;
  for (int u = lt; u < U1; u += half) prev[u] = -INFINITY;
  asm volatile("bar.sync %0, %1;" ::"r"(1 + dir), "r"(half) : "memory");
  if (dir == 0) {
    for (int d = 0; d < Tb + Ub - 1; ++d) {
      for (int u = lt; u < Ub; u += half) {
        const int t = d - u;
        float v = -INFINITY;
        if (t >= 0 && t < Tb) {
          if (t == 0 && u == 0) v = 0.f;
          else {
            const float from_t = t > 0 ? prev[u] + pb[(size_t)(t - 1) * U1 + u] : -INFINITY;
            const float from_u = u > 0 ? prev[u - 1] + pl[(size_t)t * U1 + u - 1] : -INFINITY;
            v = log_add(from_t, from_u);
          }
          al[(size_t)t * U1 + u] = v;
        }
        cur[u] = v;
      }
      asm volatile("bar.sync 1, %0;" ::"r"(half) : "memory");
      float* tmp = prev;
      prev = cur;
      cur = tmp;
    }
  } else {
    for (int d = Tb + Ub - 2; d >= 0; --d) {
      for (int u = lt; u < Ub; u += half) {
        const int t = d - u;
        float v = -INFINITY;
        if (t >= 0 && t < Tb) {
          if (t == Tb - 1 && u == Ub - 1) v = pb[(size_t)t * U1 + u];
          else {
            const float to_t = t < Tb - 1 ? prev[u] + pb[(size_t)t * U1 + u] : -INFINITY;
            const float to_u = u < Ub - 1 ? prev[u + 1] + pl[(size_t)t * U1 + u] : -INFINITY;
            v = log_add(to_t, to_u);
          }
          be[(size_t)t * U1 + u] = v;
        }
        cur[u] = v;
      }
      asm volatile("bar.sync 2, %0;" ::"r"(half) : "memory");
      float* tmp = prev;
      prev = cur;
      cur = tmp;
    }
  }
  __syncthreads();  // both recursions are done and their global writes are visible to the whole CTA
  const float log_z = be[0];
  if (threadIdx.x == 0) loss[b] = -log_z;
  if (d_blank || d_label) {
    for (int i = threadIdx.x; i < T * U1; i += blockDim.x) {
      const int t = i / U1, u = i - t * U1;
      float gb = 0.f, gl = 0.f;
      if (t < Tb && u < Ub && log_z > -INFINITY) {
        const float a = al[i];
        const float nb = (t == Tb - 1) ? (u == Ub - 1 ? 0.f : -INFINITY) : be[(size_t)(t + 1) * U1 + u];
        gb = -__expf(a + pb[i] + nb - log_z);
        if (u < Ub - 1) gl = -__expf(a + pl[i] + be[(size_t)t * U1 + u + 1] - log_z);
      }
      if (d_blank) d_blank[off + i] = gb;
      if (d_label) d_label[off + i] = gl;
    }
  }
}

}  // namespace

RB_EXPORT int rb200_device_assert(const void* cond, long long n, int* status, int code, cudaStream_t stream) {
  if (n <= 0) return RB_OK;
  int grid = (int)((n + 255) / 256);
  if (grid > 1024) grid = 1024;
  assert_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)cond, n, status, code);
  return rb_check_launch("device_assert");
}

RB_EXPORT int rb200_edit_distance(const int* a, const int* a_len, int lda, const int* b, const int* b_len, int ldb, int* out, int batch, int max_b_len,
                                  cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  if (max_b_len > kEdMaxLen) {
    rb_set_error("edit_distance: second sequence length %d > %d", max_b_len, kEdMaxLen);
    return RB_ERR_UNSUPPORTED;
  }
  const int warps = 4;
  const size_t smem = (size_t)warps * 2 * (kEdMaxLen + 1) * sizeof(int);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(edit_distance_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr = true;
  }
  edit_distance_kernel<<<(batch + warps - 1) / warps, warps * 32, smem, stream>>>(a, a_len, lda, b, b_len, ldb, out, batch);
  return rb_check_launch("edit_distance");
}

// scratch: room for batch * beam * Kt candidates of 8 bytes, Kt = 8 / 16 / 32 for k <= 8 / 16 / 32 (rb200_beam_topk_scratch_bytes)
RB_EXPORT long long rb200_beam_topk_scratch_bytes(int batch, int beam, int k) {
  const int kt = k <= 8 ? 8 : (k <= 16 ? 16 : 32);
  return (long long)batch * beam * kt * (long long)sizeof(Cand);
}

RB_EXPORT int rb200_beam_topk(const void* logits, int is_bf16, int normalized, const float* prev_scores, const void* finished, int batch, int beam, int V,
                              int eos, int k, float* out_scores, int* out_backref, int* out_label, void* scratch, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  if (k < 1 || k > kTopkMaxK || beam < 1 || beam > 64 || (long long)beam * V > 0x7fffffffLL || !scratch) {
    rb_set_error("beam_topk: k=%d (<= %d), beam=%d (<= 64), scratch %p", k, kTopkMaxK, beam, scratch);
    return RB_ERR_UNSUPPORTED;
  }
  Cand* cands = reinterpret_cast<Cand*>(scratch);
  const int rows = batch * beam;
  const int kt = k <= 8 ? 8 : (k <= 16 ? 16 : 32);  // candidates kept per row (the scratch is sized for this)
  beam_topk_row_kernel<<<rows, kTopkThreads, 0, stream>>>(logits, is_bf16, normalized, prev_scores, (const uint8_t*)finished, beam, V, eos, kt, cands);
  int rc = rb_check_launch("beam_topk rows");
  if (rc != RB_OK) return rc;
  beam_topk_merge_kernel<<<batch, 32, 0, stream>>>(cands, beam, kt, V, out_scores, out_backref, out_label, k);
  return rb_check_launch("beam_topk merge");
}

RB_EXPORT int rb200_rnnt_loss(const float* lp_blank, const float* lp_label, const int* t_lens, const int* u_lens, int batch, int T, int U1, float* alpha,
                              float* beta, float* loss, float* d_blank, float* d_label, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  if ((size_t)4 * U1 * sizeof(float) > 48 * 1024) {
    rb_set_error("rnnt_loss: %d label positions exceed the shared-memory diagonals (at most 3071)", U1);
    return RB_ERR_UNSUPPORTED;
  }
  rnnt_kernel<<<batch, 256, (size_t)4 * U1 * sizeof(float), stream>>>(lp_blank, lp_label, t_lens, u_lens, T, U1, alpha, beta, loss, d_blank, d_label);
  return rb_check_launch("rnnt_loss");
}
