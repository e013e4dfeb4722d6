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

__device__ __forceinline__ void insert_topk(Cand* best, int k, float s, int idx) {
  if (s <= best[k - 1].s) return;
  int pos = k - 1;
  while (pos > 0 && best[pos - 1].s < s) {
    best[pos] = best[pos - 1];
    --pos;
  }
  best[pos].s = s;
  best[pos].idx = idx;
}

template <int K>
__global__ void __launch_bounds__(kTopkThreads)
beam_topk_kernel(const void* __restrict__ logits, int is_bf16, int normalized, const float* __restrict__ prev_scores,
                 const uint8_t* __restrict__ finished, int beam, int V, int eos, float* __restrict__ out_scores,
                 int* __restrict__ out_backref, int* __restrict__ out_label, int k_out) {
  __shared__ float sh_lse[64];
  __shared__ float sh_red[kTopkThreads / 32];
  __shared__ Cand sh_c[kTopkThreads / 32][K];
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = (size_t)b * beam * V;
  auto ld = [&](size_t i) -> float {
    return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[i]) : reinterpret_cast<const float*>(logits)[i];
  };
  // log-sum-exp per hypothesis
  for (int h = 0; h < beam; ++h) {
    float lse = 0.f;
    if (!normalized) {
      float mx = -INFINITY;
      for (int v = threadIdx.x; v < V; v += kTopkThreads) mx = fmaxf(mx, ld(base + (size_t)h * V + v));
      mx = warp_max(mx);
      if (lane == 0) sh_red[warp] = mx;
      __syncthreads();
      mx = sh_red[0];
      for (int w = 1; w < kTopkThreads / 32; ++w) mx = fmaxf(mx, sh_red[w]);
      __syncthreads();
      float sum = 0.f;
      for (int v = threadIdx.x; v < V; v += kTopkThreads) sum += __expf(ld(base + (size_t)h * V + v) - mx);
      sum = warp_sum(sum);
      if (lane == 0) sh_red[warp] = sum;
      __syncthreads();
      sum = 0.f;
      for (int w = 0; w < kTopkThreads / 32; ++w) sum += sh_red[w];
      __syncthreads();
      lse = mx + __logf(sum);
    }
    if (threadIdx.x == 0) sh_lse[h] = lse;
  }
  __syncthreads();
  Cand best[K];
#pragma unroll
  for (int i = 0; i < K; ++i) {
    best[i].s = -INFINITY;
    best[i].idx = -1;
  }
  const int total = beam * V;
  for (int i = threadIdx.x; i < total; i += kTopkThreads) {
    const int h = i / V, v = i - h * V;
    float s;
    if (finished && finished[(size_t)b * beam + h]) {
      s = v == eos ? prev_scores[(size_t)b * beam + h] : -INFINITY;
    } else {
      s = prev_scores[(size_t)b * beam + h] + ld(base + i) - sh_lse[h];
    }
    insert_topk(best, K, s, i);
  }
  // merge inside each warp: K rounds of "take the warp-wide best head"
  Cand merged[K];
  int head = 0;
#pragma unroll 1
  for (int r = 0; r < K; ++r) {
    float s = head < K ? best[head].s : -INFINITY;
    int idx = head < K ? best[head].idx : -1;
    float ms = s;
    int ml = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float os = __shfl_xor_sync(0xffffffffu, ms, o);
      const int ol = __shfl_xor_sync(0xffffffffu, ml, o);
      if (os > ms || (os == ms && ol < ml)) {
        ms = os;
        ml = ol;
      }
    }
    const int midx = __shfl_sync(0xffffffffu, idx, ml);
    if (lane == ml) ++head;
    merged[r].s = ms;
    merged[r].idx = midx;
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < K; ++r) sh_c[warp][r] = merged[r];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // final merge of the per-warp sorted lists
    int heads[kTopkThreads / 32];
    for (int w = 0; w < kTopkThreads / 32; ++w) heads[w] = 0;
    for (int r = 0; r < k_out; ++r) {
      int bw = -1;
      float bs = -INFINITY;
      for (int w = 0; w < kTopkThreads / 32; ++w) {
        if (heads[w] < K && sh_c[w][heads[w]].idx >= 0 && (bw < 0 || sh_c[w][heads[w]].s > bs)) {
          bs = sh_c[w][heads[w]].s;
          bw = w;
        }
      }
      int idx = -1;
      if (bw >= 0) {
        idx = sh_c[bw][heads[bw]].idx;
        ++heads[bw];
      }
      out_scores[(size_t)b * k_out + r] = bw >= 0 ? bs : -INFINITY;
      out_backref[(size_t)b * k_out + r] = idx >= 0 ? idx / V : 0;
      out_label[(size_t)b * k_out + r] = idx >= 0 ? idx % V : 0;
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
  // forward
  for (int d = 0; d < Tb + Ub - 1; ++d) {
    for (int u = threadIdx.x; u < Ub; u += blockDim.x) {
      const int t = d - u;
      if (t < 0 || t >= Tb) continue;
      float v;
      if (t == 0 && u == 0) v = 0.f;
      else {
        const float from_t = t > 0 ? al[(size_t)(t - 1) * U1 + u] + pb[(size_t)(t - 1) * U1 + u] : -INFINITY;
        const float from_u = u > 0 ? al[(size_t)t * U1 + u - 1] + pl[(size_t)t * U1 + u - 1] : -INFINITY;
        v = log_add(from_t, from_u);
      }
      al[(size_t)t * U1 + u] = v;
    }
    __syncthreads();
  }
  // backward
  for (int d = Tb + Ub - 2; d >= 0; --d) {
    for (int u = threadIdx.x; u < Ub; u += blockDim.x) {
      const int t = d - u;
      if (t < 0 || t >= Tb) continue;
      float v;
      if (t == Tb - 1 && u == Ub - 1) v = pb[(size_t)t * U1 + u];
      else {
        const float to_t = t < Tb - 1 ? be[(size_t)(t + 1) * U1 + u] + pb[(size_t)t * U1 + u] : -INFINITY;
        const float to_u = u < Ub - 1 ? be[(size_t)t * U1 + u + 1] + pl[(size_t)t * U1 + u] : -INFINITY;
        v = log_add(to_t, to_u);
      }
      be[(size_t)t * U1 + u] = v;
    }
    __syncthreads();
  }
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

RB_EXPORT int rb200_beam_topk(const void* logits, int is_bf16, int normalized, const float* prev_scores, const void* finished, int batch, int beam, int V,
                              int eos, int k, float* out_scores, int* out_backref, int* out_label, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  if (k < 1 || k > kTopkMaxK || beam < 1 || beam > 64 || (long long)beam * V > 0x7fffffffLL) {
    rb_set_error("beam_topk: k=%d (<= %d), beam=%d (<= 64)", k, kTopkMaxK, beam);
    return RB_ERR_UNSUPPORTED;
  }
  if (k <= 8) {
    beam_topk_kernel<8><<<batch, kTopkThreads, 0, stream>>>(logits, is_bf16, normalized, prev_scores, (const uint8_t*)finished, beam, V, eos, out_scores,
                                                           out_backref, out_label, k);
  } else if (k <= 16) {
    beam_topk_kernel<16><<<batch, kTopkThreads, 0, stream>>>(logits, is_bf16, normalized, prev_scores, (const uint8_t*)finished, beam, V, eos, out_scores,
                                                            out_backref, out_label, k);
  } else {
    beam_topk_kernel<32><<<batch, kTopkThreads, 0, stream>>>(logits, is_bf16, normalized, prev_scores, (const uint8_t*)finished, beam, V, eos, out_scores,
                                                            out_backref, out_label, k);
  }
  return rb_check_launch("beam_topk");
}

RB_EXPORT int rb200_rnnt_loss(const float* lp_blank, const float* lp_label, const int* t_lens, const int* u_lens, int batch, int T, int U1, float* alpha,
                              float* beta, float* loss, float* d_blank, float* d_label, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  rnnt_kernel<<<batch, 256, 0, stream>>>(lp_blank, lp_label, t_lens, u_lens, T, U1, alpha, beta, loss, d_blank, d_label);
  return rb_check_launch("rnnt_loss");
}
