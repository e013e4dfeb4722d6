// CTC loss with fused log-softmax on packed logits [N, V] (bf16 or fp32), forward and gradient in three launches:
//
//   ctc_lse_gather   one warp per frame: log-sum-exp over the vocabulary (online softmax, one pass), then the
//                    log-probabilities of the 2S+1 extended states (blank, l1, blank, l2, ..., blank) of that frame
//   ctc_alpha_beta   one CTA per sequence: alpha and beta recursions over time in shared memory (double buffered),
//                    log-likelihood, and the state occupancies gamma[t,s] = exp(alpha + beta - lp - logP)
//   ctc_grad         CTAs over frames: occupancies scattered per class into a dense shared-memory row (several states
//                    share a class: all blanks, repeated labels), then grad[t,:] = softmax[t,:] - occupancy in one pass
//
// The [T, V] log-probabilities are never materialised. Scratch (global memory, given by the caller):
// lse [N], lp [N, SE], ab [N, SE] floats with SE = 2 * max_target_len + 1, and logp [B].
// Infeasible alignments (fewer frames than needed) give loss 0 and zero gradient (zero_infinity semantics).
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

// one CTA per sequence; dynamic shared memory: 2 * SE floats (alpha/beta double buffer) + SE ints (classes)
__global__ void __launch_bounds__(256)
ctc_alpha_beta_kernel(const float* __restrict__ lp, float* __restrict__ ab, const int* __restrict__ cu, const int* __restrict__ targets,
                      const int* __restrict__ tgt_lens, float* __restrict__ logp_out, float* __restrict__ loss, int s_pitch, int SE, int blank) {
  extern __shared__ float sm[];
  float* buf0 = sm;
  float* buf1 = sm + SE;
  int* cls = reinterpret_cast<int*>(sm + 2 * SE);
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
  if (se <= (int)blockDim.x) {
    // The usual case (at most 127 labels): one state per thread. A frame of the recursion is then a short dependent chain
    // (two shared-memory reads, two log-adds, a barrier); the log-probability of the next frame (and, in the beta pass, the
    // stored alpha) is fetched one frame ahead so that no global load sits on that chain.
    const int s = threadIdx.x;
    const bool act = s < se;
    const bool skip_a = act && s >= 2 && (s & 1) && cls[s] != cls[s - 2];
    const bool skip_b = act && s + 2 < se && (s & 1) && cls[s] != cls[s + 2];
    float* prev = buf0;
    float* cur = buf1;
    if (act) {
      const float a = (s < 2) ? lp[(size_t)r0 * SE + s] : kNegInf;
      prev[s] = a;
      ab[(size_t)r0 * SE + s] = a;
    }
    float l_next = (act && T > 1) ? lp[(size_t)(r0 + 1) * SE + s] : 0.f;
    __syncthreads();
    for (int t = 1; t < T; ++t) {
      const size_t row = (size_t)(r0 + t) * SE;
      const float l = l_next;
      if (act && t + 1 < T) l_next = lp[row + SE + s];
      if (act) {
        float a = prev[s];
        if (s >= 1) a = log_add(a, prev[s - 1]);
        if (skip_a) a = log_add(a, prev[s - 2]);
        a = (a == kNegInf) ? kNegInf : a + l;
        cur[s] = a;
        ab[row + s] = a;
      }
      __syncthreads();
      float* tmp = prev;
      prev = cur;
      cur = tmp;
    }
    __shared__ float logp_fast;
    if (threadIdx.x == 0) {
      float lpz = prev[se - 1];
      if (se >= 2) lpz = log_add(lpz, prev[se - 2]);
      logp_fast = lpz;
      logp_out[b] = lpz;
      loss[b] = (lpz == kNegInf) ? 0.f : -lpz;
    }
    __syncthreads();
    const float logp = logp_fast;
    if (logp == kNegInf) return;  // infeasible: the gradient kernel writes zeros
    {
      const size_t row = (size_t)(r0 + T - 1) * SE;
      if (act) {
        const float lt = lp[row + s];
        const float bt = (s >= se - 2) ? lt : kNegInf;
        prev[s] = bt;
        const float a = ab[row + s];  // written by this thread in the alpha pass
        ab[row + s] = (a == kNegInf || bt == kNegInf) ? 0.f : __expf(a + bt - lt - logp);
      }
    }
    float a_next = 0.f;
    l_next = 0.f;
    if (act && T > 1) {
      l_next = lp[(size_t)(r0 + T - 2) * SE + s];
      a_next = ab[(size_t)(r0 + T - 2) * SE + s];
    }
    __syncthreads();
    for (int t = T - 2; t >= 0; --t) {
      const size_t row = (size_t)(r0 + t) * SE;
      const float l = l_next, a = a_next;
      if (act && t > 0) {
        l_next = lp[row - SE + s];
        a_next = ab[row - SE + s];
      }
      if (act) {
        float bt = prev[s];
        if (s + 1 < se) bt = log_add(bt, prev[s + 1]);
        if (skip_b) bt = log_add(bt, prev[s + 2]);
        bt = (bt == kNegInf) ? kNegInf : bt + l;
        cur[s] = bt;
        ab[row + s] = (a == kNegInf || bt == kNegInf) ? 0.f : __expf(a + bt - l - logp);
      }
      __syncthreads();
      float* tmp = prev;
      prev = cur;
      cur = tmp;
    }
    return;
  }
  // ---- general case (more states than threads): alpha
  float* prev = buf0;
  float* cur = buf1;
  for (int s = threadIdx.x; s < se; s += blockDim.x) {
    const float a = (s < 2) ? lp[(size_t)r0 * SE + s] : kNegInf;
    prev[s] = a;
    ab[(size_t)r0 * SE + s] = a;
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
      ab[row + s] = a;
    }
    __syncthreads();
    float* tmp = prev;
    prev = cur;
    cur = tmp;
  }
  __shared__ float logp_sh;
  if (threadIdx.x == 0) {
    float lpz = prev[se - 1];
    if (se >= 2) lpz = log_add(lpz, prev[se - 2]);
    logp_sh = lpz;
    logp_out[b] = lpz;
    loss[b] = (lpz == kNegInf) ? 0.f : -lpz;
  }
  __syncthreads();
  const float logp = logp_sh;
  if (logp == kNegInf) return;  // infeasible: the gradient kernel writes zeros
  // ---- beta, and gamma = exp(alpha + beta - lp - logP) written over ab
  {
    const size_t row = (size_t)(r0 + T - 1) * SE;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      const float bt = (s >= se - 2) ? lp[row + s] : kNegInf;
      prev[s] = bt;
      const float a = ab[row + s];
      ab[row + s] = (a == kNegInf || bt == kNegInf) ? 0.f : __expf(a + bt - lp[row + s] - logp);
    }
  }
  __syncthreads();
  for (int t = T - 2; t >= 0; --t) {
    const size_t row = (size_t)(r0 + t) * SE;
    for (int s = threadIdx.x; s < se; s += blockDim.x) {
      float bt = prev[s];
      if (s + 1 < se) bt = log_add(bt, prev[s + 1]);
      if (s + 2 < se && (s & 1) && cls[s] != cls[s + 2]) bt = log_add(bt, prev[s + 2]);
      const float l = lp[row + s];
      bt = (bt == kNegInf) ? kNegInf : bt + l;
      cur[s] = bt;
      const float a = ab[row + s];
      ab[row + s] = (a == kNegInf || bt == kNegInf) ? 0.f : __expf(a + bt - l - logp);
    }
    __syncthreads();
    float* tmp = prev;
    prev = cur;
    cur = tmp;
  }
}

// one CTA handles `frames_per_cta` consecutive frames; dynamic shared memory: V floats (dense class occupancy)
__global__ void __launch_bounds__(256)
ctc_grad_kernel(const void* __restrict__ logits, int is_bf16, const int* __restrict__ row_batch, const int* __restrict__ targets,
                const int* __restrict__ tgt_lens, const float* __restrict__ lse, const float* __restrict__ gamma,
                const float* __restrict__ logp, void* __restrict__ grad, int n_rows, int V, int s_pitch, int SE, int blank,
                int frames_per_cta) {
  extern __shared__ float post[];
  for (int v = threadIdx.x; v < V; v += blockDim.x) post[v] = 0.f;
  __syncthreads();
  const int r_begin = blockIdx.x * frames_per_cta;
  const int r_end = min(n_rows, r_begin + frames_per_cta);
  const int elem = is_bf16 ? 2 : 4;
  const int per16 = 16 / elem;
  for (int r = r_begin; r < r_end; ++r) {
    const int b = row_batch[r];
    const bool feasible = logp[b] != kNegInf;
    const int se = 2 * tgt_lens[b] + 1;
    if (feasible) {
      for (int s = threadIdx.x; s < se; s += blockDim.x) {
        const float g = gamma[(size_t)r * SE + s];
        if (g != 0.f) {
          const int c = (s & 1) ? targets[(size_t)b * s_pitch + (s >> 1)] : blank;
          atomicAdd(&post[c], g);
        }
      }
    }
    __syncthreads();
    const size_t base = (size_t)r * V;
    const float l = lse[r];
    int head = (int)((per16 - (base % per16)) % per16);
    if (head > V) head = V;
    const int body8 = is_bf16 ? ((V - head) / 8) * 8 : 0;
    // scalar head and tail around the 16-byte aligned vector body
    for (int c = threadIdx.x; c < V - body8; c += blockDim.x) {
      const int cc = c < head ? c : c + body8;
      const float g = feasible ? __expf(ldf(logits, base + cc, is_bf16) - l) - post[cc] : 0.f;
      if (is_bf16) reinterpret_cast<__nv_bfloat16*>(grad)[base + cc] = __float2bfloat16(g);
      else reinterpret_cast<float*>(grad)[base + cc] = g;
    }
    for (int c = head + threadIdx.x * 8; c < head + body8; c += blockDim.x * 8) {
      F8 a = load8(logits, base + c, 1);
#pragma unroll
      for (int k = 0; k < 8; ++k) a.v[k] = feasible ? __expf(a.v[k] - l) - post[c + k] : 0.f;
      store8(grad, base + c, a, 1);
    }
    __syncthreads();
    // clear the touched classes for the next frame
    if (feasible) {
      for (int s = threadIdx.x; s < se; s += blockDim.x) {
        const int c = (s & 1) ? targets[(size_t)b * s_pitch + (s >> 1)] : blank;
        post[c] = 0.f;
      }
    }
    __syncthreads();
  }
}

}  // namespace

// scratch: at least n_rows * (1 + 2 * SE) + batch floats, SE = 2 * max_s + 1
RB_EXPORT int rb200_ctc_loss(const void* logits, int is_bf16, const int* cu, const int* row_batch, const int* targets, const int* tgt_lens,
                             float* loss, void* grad, float* scratch, int batch, int n_rows, int V, int s_pitch, int max_s, int blank,
                             long long scratch_floats, cudaStream_t stream) {
  if (batch <= 0) return RB_OK;
  const int SE = 2 * max_s + 1;
  const long long need = (long long)n_rows * (1 + 2 * SE) + batch;
  if (scratch_floats < need) {
    rb_set_error("ctc_loss: scratch of %lld floats given, %lld needed", scratch_floats, need);
    return RB_ERR_ARG;
  }
  if (blank < 0 || blank >= V) {
    rb_set_error("ctc_loss: blank index %d outside [0, %d)", blank, V);
    return RB_ERR_ARG;
  }
  const size_t smem_ab = (size_t)(3 * SE) * sizeof(float);
  const size_t smem_grad = (size_t)V * sizeof(float);
  if (smem_ab > 200 * 1024 || smem_grad > 200 * 1024) {
    rb_set_error("ctc_loss: target length %d or vocabulary %d too large for the shared-memory buffers", max_s, V);
    return RB_ERR_UNSUPPORTED;
  }
  float* lse = scratch;
  float* lp = lse + n_rows;
  float* ab = lp + (size_t)n_rows * SE;
  float* logp = ab + (size_t)n_rows * SE;
  if (n_rows > 0) {
    ctc_lse_gather_kernel<<<(n_rows + 7) / 8, 256, 0, stream>>>(logits, is_bf16, row_batch, targets, tgt_lens, lse, lp, n_rows, V, s_pitch, SE, blank);
    int st = rb_check_launch("ctc_lse_gather");
    if (st) return st;
  }
  if (smem_ab > 48 * 1024) cudaFuncSetAttribute(ctc_alpha_beta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_ab);
  ctc_alpha_beta_kernel<<<batch, 256, smem_ab, stream>>>(lp, ab, cu, targets, tgt_lens, logp, loss, s_pitch, SE, blank);
  int st = rb_check_launch("ctc_alpha_beta");
  if (st) return st;
  if (n_rows > 0 && grad != nullptr) {
    if (smem_grad > 48 * 1024) cudaFuncSetAttribute(ctc_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_grad);
    const int frames_per_cta = 8;
    ctc_grad_kernel<<<(n_rows + frames_per_cta - 1) / frames_per_cta, 256, smem_grad, stream>>>(
        logits, is_bf16, row_batch, targets, tgt_lens, lse, ab, logp, grad, n_rows, V, s_pitch, SE, blank, frames_per_cta);
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
