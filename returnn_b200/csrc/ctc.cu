// CTC loss with fused log-softmax on packed logits [N, V] (bf16 or fp32), forward and gradient in three launches:
//
//   ctc_lse_gather   one warp per frame: log-sum-exp over the vocabulary (online softmax, one pass), then the
//                    log-probabilities of the 2S+1 extended states (blank, l1, blank, l2, ..., blank) of that frame
//   ctc_alpha_beta   one CTA per sequence: the alpha and the beta recursion run at the same time in the two halves of the CTA
//                    (shared memory, double buffered), and the log-likelihood
//   ctc_grad         CTAs over frames: softmax[t,:] streamed to the output, then the entries of the label classes corrected by
//                    their occupancies exp(alpha + beta - lp - logP) (several states share a class: all blanks, repeated labels)
//
// The [T, V] log-probabilities are never materialised. Scratch (global memory, given by the caller):
// lse [N], lp [N, SE], alpha [N, SE], beta [N, SE] floats with SE = 2 * max_target_len + 1, and logp [B].
// Infeasible alignments (fewer frames than needed) give loss 0 and zero gradient (zero_infinity semantics).
#include <algorithm>
#include "common.cuh"

namespace {

constexpr float kNegInf = -INFINITY;

__device__ __forceinline__ float ldf(const void* x, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]) : reinterpret_cast<const float*>(x)[i];
}
__device__ __forceinline__ float log_add(float a, float b) {
  if (a == kNegInf) return b;
  if (b == kNegInf) return a;
  const float m = fmaxf(a, b);
  return m + log1pf(__expf(-fabsf(a - b)));
}

// frame r belongs to sequence row_batch[r] at position row_pos[r]
__global__ void __launch_bounds__(256)
ctc_lse_gather_kernel(const void* __restrict__ logits, int is_bf16, const int* __restrict__ row_batch, const int* __restrict__ targets,
                      const int* __restrict__ tgt_lens, float* __restrict__ lse, float* __restrict__ lp, int n_rows, int V, int s_pitch,
                      int SE, int blank) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const size_t base = (size_t)r * V;
  float mx = kNegInf, sum = 0.f;
  // peel to a 16-byte boundary, vector body, scalar tail
  const int elem = is_bf16 ? 2 : 4;
  const int per16 = 16 / elem;
  int head = (int)((per16 - (base % per16)) % per16);
  if (head > V) head = V;
  for (int c = lane; c < head; c += 32) {
    const float a = ldf(logits, base + c, is_bf16);
    const float nm = fmaxf(mx, a);
    sum = (mx == kNegInf ? 0.f : sum * __expf(mx - nm)) + __expf(a - nm);
    mx = nm;
  }
  const int body8 = is_bf16 ? ((V - head) / 8) * 8 : 0;
  for (int c = head + lane * 8; c < head + body8; c += 256) {
    F8 a = load8(logits, base + c, 1);
    float lm = a.v[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, a.v[k]);
    const float nm = fmaxf(mx, lm);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += __expf(a.v[k] - nm);
    sum = (mx == kNegInf ? 0.f : sum * __expf(mx - nm)) + s;
    mx = nm;
  }
  for (int c = head + body8 + lane; c < V; c += 32) {
    const float a = ldf(logits, base + c, is_bf16);
    const float nm = fmaxf(mx, a);
    sum = (mx == kNegInf ? 0.f : sum * __expf(mx - nm)) + __expf(a - nm);
    mx = nm;
  }
  const float wm = warp_max(mx);
  const float ws = warp_sum(mx == kNegInf ? 0.f : sum * __expf(mx - wm));
  const float l = wm + logf(ws);
  if (lane == 0) lse[r] = l;
  const int b = row_batch[r];
  const int se = 2 * tgt_lens[b] + 1;
  for (int s = lane; s < se; s += 32) {
    const int cls = (s & 1) ? targets[(size_t)b * s_pitch + (s >> 1)] : blank;
    lp[(size_t)r * SE + s] = ldf(logits, base + cls, is_bf16) - l;
  }
}

// One CTA per sequence; dynamic shared memory: 4 * SE floats (double buffers of alpha and of beta) + SE ints (classes).
// The forward and the backward recursion do not depend on each other, so they run at the same time in the two halves of the CTA
// (threads [0, G) alpha, [G, 2G) beta, one lattice state per thread), each half with its own named barrier. A frame of a recursion
// is a short dependent chain (two shared-memory reads, two log-adds, a barrier); the log-probabilities it needs are fetched
// kCtcDepth frames ahead into registers, so that no global-memory latency sits on that chain. alpha goes to `al`, beta (including
// the frame's own log-probability) to `be`; the gradient kernel forms the occupancies exp(alpha + beta - lp - logP) from them.
constexpr int kCtcDepth = 8;

// log(e^a + e^b + e^c) without branches and with one logarithm: the dependent chain is max -> exp -> add -> log.
// Inputs may be -inf (e^-inf = 0); all three -inf gives log(0) = -inf.
__device__ __forceinline__ float log_add3(float a, float b, float c) {
  const float m = fmaxf(a, fmaxf(b, c));
  const float mm = (m == kNegInf) ? 0.f : m;
  return mm + __logf(__expf(a - mm) + __expf(b - mm) + __expf(c - mm));
}

__device__ __forceinline__ void bar_sync_named(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__global__ void __launch_bounds__(512)
ctc_alpha_beta_kernel(const float* __restrict__ lp, float* __restrict__ al, float* __restrict__ be, const int* __restrict__ cu,
                      const int* __restrict__ targets, const int* __restrict__ tgt_lens, float* __restrict__ logp_out, float* __restrict__ loss,
                      int s_pitch, int SE, int blank) {
  extern __shared__ float sm[];
  int* cls = reinterpret_cast<int*>(sm + 4 * SE);
  const int G = blockDim.x >> 1;
  const int b = blockIdx.x;
  const int r0 = cu[b];
  const int T = cu[b + 1] - r0;
  const int S = tgt_lens[b];
  const int se = 2 * S + 1;
  for (int s = threadIdx.x; s < se; s += blockDim.x) cls[s] = (s & 1) ? targets[(size_t)b * s_pitch + (s >> 1)] : blank;
  __syncthreads();
  if (T <= 0) {
    if (threadIdx.x == 0) {
      logp_out[b] = S == 0 ? 0.f : kNegInf;
      loss[b] = 0.f;
    }
    return;
  }
  if (se <= G) {
    const int dir = threadIdx.x >= G ? 1 : 0;
    const int s = threadIdx.x - dir * G;
    const int gb = (se + 31) & ~31;  // threads of this direction that take part (whole warps)
    if (s >= gb) return;
    const bool act = s < se;
    float* prev = sm + dir * 2 * SE;
    float* cur = prev + SE;
    const int bar = 1 + dir;
    float lq[kCtcDepth];
    if (dir == 0) {
      const bool skip = act && s >= 2 && (s & 1) && cls[s] != cls[s - 2];
      if (act) {
        const float a = (s < 2) ? lp[(size_t)r0 * SE + s] : kNegInf;
        prev[s] = a;
        al[(size_t)r0 * SE + s] = a;
      }
#pragma unroll
      for (int j = 0; j < kCtcDepth; ++j) lq[j] = (act && 1 + j < T) ? lp[(size_t)(r0 + 1 + j) * SE + s] : 0.f;
      bar_sync_named(bar, gb);
      for (int t0 = 1; t0 < T; t0 += kCtcDepth) {
        float nq[kCtcDepth];
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) nq[j] = (act && t0 + kCtcDepth + j < T) ? lp[(size_t)(r0 + t0 + kCtcDepth + j) * SE + s] : 0.f;
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) {
          const int t = t0 + j;
          if (t < T) {  // uniform over the CTA
            if (act) {
              float a = log_add3(prev[s], s >= 1 ? prev[s - 1] : kNegInf, skip ? prev[s - 2] : kNegInf);
              a = (a == kNegInf) ? kNegInf : a + lq[j];
              cur[s] = a;
              al[(size_t)(r0 + t) * SE + s] = a;
            }
            bar_sync_named(bar, gb);
            float* tmp = prev;
            prev = cur;
            cur = tmp;
          }
        }
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) lq[j] = nq[j];
      }
      if (s == 0) {
        float lpz = prev[se - 1];
        if (se >= 2) lpz = log_add(lpz, prev[se - 2]);
        logp_out[b] = lpz;
        loss[b] = (lpz == kNegInf) ? 0.f : -lpz;
      }
    } else {
      const bool skip = act && s + 2 < se && (s & 1) && cls[s] != cls[s + 2];
      if (act) {
        const size_t row = (size_t)(r0 + T - 1) * SE;
        const float bt = (s >= se - 2) ? lp[row + s] : kNegInf;
        prev[s] = bt;
        be[row + s] = bt;
      }
#pragma unroll
      for (int j = 0; j < kCtcDepth; ++j) lq[j] = (act && T - 2 - j >= 0) ? lp[(size_t)(r0 + T - 2 - j) * SE + s] : 0.f;
      bar_sync_named(bar, gb);
      for (int t0 = T - 2; t0 >= 0; t0 -= kCtcDepth) {
        float nq[kCtcDepth];
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) nq[j] = (act && t0 - kCtcDepth - j >= 0) ? lp[(size_t)(r0 + t0 - kCtcDepth - j) * SE + s] : 0.f;
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) {
          const int t = t0 - j;
          if (t >= 0) {
            if (act) {
              float bt = log_add3(prev[s], s + 1 < se ? prev[s + 1] : kNegInf, skip ? prev[s + 2] : kNegInf);
              bt = (bt == kNegInf) ? kNegInf : bt + lq[j];
              cur[s] = bt;
              be[(size_t)(r0 + t) * SE + s] = bt;
            }
            bar_sync_named(bar, gb);
            float* tmp = prev;
            prev = cur;
            cur = tmp;
          }
        }
#pragma unroll
        for (int j = 0; j < kCtcDepth; ++j) lq[j] = nq[j];
      }
    }
    return;
  }
  // ---- general case (more states than threads per direction): the whole CTA runs alpha, then beta
  float* prev = sm;
  float* cur = sm + SE;
  for (int s = threadIdx.x; s < se; s += blockDim.x) {
    const float a = (s < 2) ? lp[(size_t)r0 * SE + s] : kNegInf;
    prev[s] = a;
    al[(size_t)r0 * SE + s] = a;
  }
  __syncthreads();
  for (int t = 1; t < T; ++t) {
    const size_t row = (size_t)(r0 + t) * SE;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      float a = prev[s];
      if (s >= 1) a = log_add(a, prev[s - 1]);
      if (s >= 2 && (s & 1) && cls[s] != cls[s - 2]) a = log_add(a, prev[s - 2]);
      a = (a == kNegInf) ? kNegInf : a + lp[row + s];
      cur[s] = a;
      al[row + s] = a;
    }
    __syncthreads();
    float* tmp = prev;
    prev = cur;
    cur = tmp;
  }
  if (threadIdx.x == 0) {
    float lpz = prev[se - 1];
    if (se >= 2) lpz = log_add(lpz, prev[se - 2]);
    logp_out[b] = lpz;
    loss[b] = (lpz == kNegInf) ? 0.f : -lpz;
  }
  __syncthreads();
  {
    const size_t row = (size_t)(r0 + T - 1) * SE;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      const float bt = (s >= se - 2) ? lp[row + s] : kNegInf;
      prev[s] = bt;
      be[row + s] = bt;
    }
  }
  __syncthreads();
  for (int t = T - 2; t >= 0; --t) {
    const size_t row = (size_t)(r0 + t) * SE;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      float bt = prev[s];
      if (s + 1 < se) bt = log_add(bt, prev[s + 1]);
      if (s + 2 < se && (s & 1) && cls[s] != cls[s + 2]) bt = log_add(bt, prev[s + 2]);
      bt = (bt == kNegInf) ? kNegInf : bt + lp[row + s];
      cur[s] = bt;
      be[row + s] = bt;
    }
    __syncthreads();
    float* tmp = prev;
    prev = cur;
    cur = tmp;
  }
}

// Gradient w.r.t. the logits: softmax(logits) - (occupancy of each class). One CTA handles kGradFrames consecutive frames.
// Only the classes of the label sequence (at most 2S + 1 states, S + 1 distinct classes) have a non-zero occupancy, so the kernel
// first streams softmax(logits) for its frames straight to the output (no shared memory on that path), and then corrects the few
// label entries: state s "owns" its class if no earlier state has the same one; the owner sums the occupancies
// exp(alpha + beta - lp - logP) of all states with that class and rewrites the one output element.
// Dynamic shared memory: kGradFrames * SE floats (occupancies) + kGradFrames * SE ints (classes).
constexpr int kGradFrames = 8;

__global__ void __launch_bounds__(256)
ctc_grad_kernel(const void* __restrict__ logits, int is_bf16, const int* __restrict__ row_batch, const int* __restrict__ targets,
                const int* __restrict__ tgt_lens, const float* __restrict__ lse, const float* __restrict__ lp, const float* __restrict__ al,
                const float* __restrict__ be, const float* __restrict__ logp, void* __restrict__ grad, int n_rows, int V, int s_pitch, int SE,
                int blank) {
  extern __shared__ float gsm[];
  float* gam = gsm;                                                  // [kGradFrames][SE]
  int* gcls = reinterpret_cast<int*>(gsm + kGradFrames * SE);         // [kGradFrames][SE]
  const int r_begin = blockIdx.x * kGradFrames;
  const int r_end = min(n_rows, r_begin + kGradFrames);
  const int elem = is_bf16 ? 2 : 4;
  const int per16 = 16 / elem;
  // occupancies and classes of the frames' states (independent of the streaming pass below)
  for (int r = r_begin; r < r_end; ++r) {
    const int b = row_batch[r];
    const float lpz = logp[b];
    const int se = 2 * tgt_lens[b] + 1;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      const float a = al[(size_t)r * SE + s], bt = be[(size_t)r * SE + s];
      // beta already contains the frame's own log-probability
      gam[(r - r_begin) * SE + s] = (lpz == kNegInf || a == kNegInf || bt == kNegInf) ? 0.f : __expf(a + bt - lp[(size_t)r * SE + s] - lpz);
      gcls[(r - r_begin) * SE + s] = (s & 1) ? targets[(size_t)b * s_pitch + (s >> 1)] : blank;
    }
  }
  // softmax of every frame, streamed
  for (int r = r_begin; r < r_end; ++r) {
    const bool feasible = logp[row_batch[r]] != kNegInf;
    const size_t base = (size_t)r * V;
    const float l = lse[r];
    int head = (int)((per16 - (base % per16)) % per16);
    if (head > V) head = V;
    const int body8 = is_bf16 ? ((V - head) / 8) * 8 : 0;
    for (int c = threadIdx.x; c < V - body8; c += blockDim.x) {  // scalar head and tail around the 16-byte aligned vector body
      const int cc = c < head ? c : c + body8;
      const float g = feasible ? __expf(ldf(logits, base + cc, is_bf16) - l) : 0.f;
      if (is_bf16) reinterpret_cast<__nv_bfloat16*>(grad)[base + cc] = __float2bfloat16(g);
      else reinterpret_cast<float*>(grad)[base + cc] = g;
    }
    // four independent 16-byte loads per thread in flight (a row is about five vectors per thread): the pass is bound by
    // memory latency times bytes in flight, not by arithmetic
    constexpr int kU = 4;
    const int n_vec = body8 >> 3;
    for (int v0 = threadIdx.x; v0 < n_vec; v0 += blockDim.x * kU) {
      F8 a[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int v = v0 + u * blockDim.x;
        if (v < n_vec) a[u] = load8(logits, base + head + (size_t)v * 8, 1);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int v = v0 + u * blockDim.x;
        if (v < n_vec) {
#pragma unroll
          for (int k = 0; k < 8; ++k) a[u].v[k] = feasible ? __expf(a[u].v[k] - l) : 0.f;
          store8(grad, base + head + (size_t)v * 8, a[u], 1);
        }
      }
    }
  }
  __syncthreads();  // the streamed values are in place (and visible to this CTA) before single elements are rewritten
  for (int r = r_begin; r < r_end; ++r) {
    const int b = row_batch[r];
    if (logp[b] == kNegInf) continue;
    const int se = 2 * tgt_lens[b] + 1;
    const float* g_r = gam + (r - r_begin) * SE;
    const int* c_r = gcls + (r - r_begin) * SE;
    const size_t base = (size_t)r * V;
    const float l = lse[r];
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      const int c = c_r[s];
      bool first = true;
      float total = 0.f;
      for (int q = 0; q < se; ++q) {
        if (c_r[q] == c) {
          if (q < s) {
            first = false;
            break;
          }
          total += g_r[q];
        }
      }
      if (!first || total == 0.f) continue;
      const float g = __expf(ldf(logits, base + c, is_bf16) - l) - total;
      if (is_bf16) reinterpret_cast<__nv_bfloat16*>(grad)[base + c] = __float2bfloat16(g);
      else reinterpret_cast<float*>(grad)[base + c] = g;
    }
  }
}

}  // namespace

// scratch: at least n_rows * (1 + 3 * SE) + batch floats, SE = 2 * max_s + 1
RB_EXPORT int rb200_ctc_loss(const void* logits, int is_bf16, const int* cu, const int* row_batch, const int* targets, const int* tgt_lens,
                             float* loss, void* grad, float* scratch, int batch, int n_rows, int V, int s_pitch, int max_s, int blank,
                             long long scratch_floats, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  const int SE = 2 * max_s + 1;
  const long long need = (long long)n_rows * (1 + 3 * SE) + batch;
  if (scratch_floats < need) {
    rb_set_error("ctc_loss: scratch of %lld floats given, %lld needed", scratch_floats, need);
    return RB_ERR_ARG;
  }
  if (blank < 0 || blank >= V) {
    rb_set_error("ctc_loss: blank index %d outside [0, %d)", blank, V);
    return RB_ERR_ARG;
  }
  const size_t smem_ab = (size_t)(5 * SE) * sizeof(float);
  const size_t smem_grad = (size_t)kGradFrames * SE * 2 * sizeof(float);
  if (smem_ab > 200 * 1024 || smem_grad > 200 * 1024) {
    rb_set_error("ctc_loss: target length %d or vocabulary %d too large for the shared-memory buffers", max_s, V);
    return RB_ERR_UNSUPPORTED;
  }
  float* lse = scratch;
  float* lp = lse + n_rows;
  float* al = lp + (size_t)n_rows * SE;
  float* be = al + (size_t)n_rows * SE;
  float* logp = be + (size_t)n_rows * SE;
  if (n_rows > 0) {
    ctc_lse_gather_kernel<<<(n_rows + 7) / 8, 256, 0, stream>>>(logits, is_bf16, row_batch, targets, tgt_lens, lse, lp, n_rows, V, s_pitch, SE, blank);
    int st = rb_check_launch("ctc_lse_gather");
    if (st) return st;
  }
  if (smem_ab > 48 * 1024) cudaFuncSetAttribute(ctc_alpha_beta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_ab);
  const int per_dir = std::min(256, (SE + 31) / 32 * 32);  // threads per direction; longer label sequences take the sequential path
  ctc_alpha_beta_kernel<<<batch, 2 * per_dir, smem_ab, stream>>>(lp, al, be, cu, targets, tgt_lens, logp, loss, s_pitch, SE, blank);
  int st = rb_check_launch("ctc_alpha_beta");
  if (st) return st;
  if (n_rows > 0 && grad != nullptr) {
    if (smem_grad > 48 * 1024) cudaFuncSetAttribute(ctc_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_grad);
    ctc_grad_kernel<<<(n_rows + kGradFrames - 1) / kGradFrames, 256, smem_grad, stream>>>(
        logits, is_bf16, row_batch, targets, tgt_lens, lse, lp, al, be, logp, grad, n_rows, V, s_pitch, SE, blank);
    st = rb_check_launch("ctc_grad");
  }
  return st;
}

namespace {

// out[r, :] = grad[r, :] * dloss[row_batch[r]]: the backward of the loss function scales the gradient that the forward launches
// left behind (one pass instead of an fp32 copy, a multiply and a cast back)
__global__ void __launch_bounds__(256)
ctc_scale_rows_kernel(const void* __restrict__ grad, const int* __restrict__ row_batch, const float* __restrict__ dloss, void* __restrict__ out,
                      int V, int is_bf16) {
  const int r = blockIdx.x;
  const float sc = dloss[row_batch[r]];
  const size_t base = (size_t)r * V;
  const int vec = (is_bf16 && (base % 8) == 0) ? (V / 8) * 8 : 0;
  for (int c = threadIdx.x * 8; c < vec; c += blockDim.x * 8) {
    F8 a = load8(grad, base + c, 1);
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] *= sc;
    store8(out, base + c, a, 1);
  }
  for (int c = vec + threadIdx.x; c < V; c += blockDim.x) {
    const float g = ldf(grad, base + c, is_bf16) * sc;
    if (is_bf16) reinterpret_cast<__nv_bfloat16*>(out)[base + c] = __float2bfloat16(g);
    else reinterpret_cast<float*>(out)[base + c] = g;
  }
}

}  // namespace

// grad, out [n_rows, V] (bf16 or fp32, may be the same buffer), row_batch [n_rows], dloss [B] fp32
RB_EXPORT int rb200_ctc_scale_rows(const void* grad, const int* row_batch, const float* dloss, void* out, int n_rows, int V, int is_bf16,
                                   cudaStream_t stream) {
  if (n_rows <= 0 || V <= 0) return RB_OK;
  ctc_scale_rows_kernel<<<n_rows, 256, 0, stream>>>(grad, row_batch, dloss, out, V, is_bf16);
  return rb_check_launch("ctc_scale_rows");
}
