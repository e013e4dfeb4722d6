// Batched finite-state-acceptor kernels: forward-backward (full sum) and Viterbi (best path) over a batch of FSAs whose edges
// each consume one frame, plus the on-device construction of the CTC topology.
//
// One CTA per sequence runs the whole frame loop inside the kernel (no launch per frame): the edges of the sequence are spread
// over the threads, state scores live in global scratch [T+1][num_states] (all sequences share one state index space), and
// frames are separated by __syncthreads. Log-space accumulation into a target state uses a compare-and-swap loop on the float
// bits. Scores are log-probabilities internally; the interface uses negative logs like the reference ops
// (returnn/native_op.py:3259 FastBaumWelchOp, :4948 FastViterbiOp, :5320 GetCtcFsaFastBwOp).
#include "common.cuh"

namespace {

__device__ __forceinline__ float log_add2(float a, float b) {
  if (a == -INFINITY) return b;
  if (b == -INFINITY) return a;
  const float m = fmaxf(a, b);
  return m + __logf(__expf(a - m) + __expf(b - m));
}

__device__ __forceinline__ void atomic_log_add(float* addr, float v) {
  if (v == -INFINITY) return;
  int* ai = reinterpret_cast<int*>(addr);
  int old = *ai, assumed;
  do {
    assumed = old;
    const float nv = log_add2(__int_as_float(assumed), v);
    old = atomicCAS(ai, assumed, __float_as_int(nv));
  } while (old != assumed);
}

// packed (score, edge) maximum: score mapped to an order-preserving unsigned, edge index in the low word
__device__ __forceinline__ unsigned long long pack_max(float s, int e) {
  unsigned u = __float_as_uint(s);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned)e;
}
__device__ __forceinline__ float unpack_score(unsigned long long p) {
  unsigned u = (unsigned)(p >> 32);
  u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
  return __uint_as_float(u);
}

// edges: from, to, emission, each [E] sorted by sequence; edge_start [B+1]; weights [E] (-log); am [T, B, V] (-log);
// start/end/end2 [B] (end2 < 0: none); lens [B]. fwd, bwd: [T+1, S] pre-filled with -inf. out [T, B, V] pre-filled with -inf
// (log posterior sums, negated on return by the caller); obs [B] total log score.
__global__ void __launch_bounds__(256)
fbw_kernel(const int* __restrict__ e_from, const int* __restrict__ e_to, const int* __restrict__ e_em, const float* __restrict__ weights,
           const int* __restrict__ edge_start, const float* __restrict__ am, const int* __restrict__ start, const int* __restrict__ end,
           const int* __restrict__ end2, const int* __restrict__ lens, int T, int B, int V, int S, float* __restrict__ fwd,
           float* __restrict__ bwd, float* __restrict__ out, float* __restrict__ obs, const int* __restrict__ end_start,
           const int* __restrict__ end_state, const float* __restrict__ end_weight, const int* __restrict__ row_start) {
  const int b = blockIdx.x;
  // frame t of this sequence: row t * B + b of am / out [T, B, V], or row row_start[b] + t of the packed form [N, V]
  const size_t r_base = row_start ? (size_t)row_start[b] : (size_t)b;
  const size_t r_step = row_start ? 1 : (size_t)B;
  const int e0 = edge_start[b], e1 = edge_start[b + 1];
  const int Tb = lens[b];
  if (threadIdx.x == 0) {
    fwd[start[b]] = 0.f;
    if (end_start) {
      // any number of final states per sequence, each with its own weight (-log): entries end_start[b] .. end_start[b + 1]
      for (int i = end_start[b]; i < end_start[b + 1]; ++i) {
        float* slot = bwd + (size_t)Tb * S + end_state[i];
        *slot = log_add2(*slot, -end_weight[i]);
      }
    } else {
      bwd[(size_t)Tb * S + end[b]] = 0.f;
      if (end2 && end2[b] >= 0) bwd[(size_t)Tb * S + end2[b]] = 0.f;
    }
  }
  __syncthreads();
  for (int t = 0; t < Tb; ++t) {
    const float* cur = fwd + (size_t)t * S;
    float* nxt = fwd + (size_t)(t + 1) * S;
    const float* amt = am + (r_base + (size_t)t * r_step) * V;
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const float s = cur[e_from[e]];
      if (s > -INFINITY) atomic_log_add(nxt + e_to[e], s - weights[e] - amt[e_em[e]]);
    }
    __syncthreads();
  }
  for (int t = Tb - 1; t >= 0; --t) {
    const float* nxt = bwd + (size_t)(t + 1) * S;
    float* cur = bwd + (size_t)t * S;
    const float* amt = am + (r_base + (size_t)t * r_step) * V;
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const float s = nxt[e_to[e]];
      if (s > -INFINITY) atomic_log_add(cur + e_from[e], s - weights[e] - amt[e_em[e]]);
    }
    __syncthreads();
  }
  const float total = bwd[start[b]];
  if (threadIdx.x == 0) obs[b] = total;
  for (int t = 0; t < Tb; ++t) {
    const float* f = fwd + (size_t)t * S;
    const float* bw = bwd + (size_t)(t + 1) * S;
    const float* amt = am + (r_base + (size_t)t * r_step) * V;
    float* o = out + (r_base + (size_t)t * r_step) * V;
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const float a = f[e_from[e]], c = bw[e_to[e]];
      if (a > -INFINITY && c > -INFINITY) atomic_log_add(o + e_em[e], a - weights[e] - amt[e_em[e]] + c - total);
    }
  }
}

// Segmental forward-backward: an edge taken at frame t consumes a SEGMENT of l = 1 .. L frames and costs
//   weights[e] + am_scale * am[row_start[b] + t][l - 1][e_em[e]] + length_models[e_lenmod[e]][l - 1]          (all -log)
// am holds one row per (sequence, segment start frame): [N, L, V]; out has the same shape and receives the log posterior of
// (start frame, length, label). State scores fwd / bwd: [T_max + 1, S] pre-filled with -inf; out pre-filled with -inf.
// One CTA per sequence; the (edge, length) pairs of a frame are spread over the threads.
// (reference: returnn/native_op.py:4369 SegmentFastBaumWelchOp, kernels next_frame_fwd / next_frame_bwd)
__global__ void __launch_bounds__(256)
seg_fbw_kernel(const int* __restrict__ e_from, const int* __restrict__ e_to, const int* __restrict__ e_em, const int* __restrict__ e_lenmod,
               const float* __restrict__ weights, const int* __restrict__ edge_start, const float* __restrict__ am,
               const float* __restrict__ length_models, const int* __restrict__ row_start, const int* __restrict__ start,
               const int* __restrict__ end, const int* __restrict__ lens, int L, int V, int S, int T_max, float am_scale, float* __restrict__ fwd,
               float* __restrict__ bwd, float* __restrict__ out, float* __restrict__ obs) {
  const int b = blockIdx.x;
  const int e0 = edge_start[b], ne = edge_start[b + 1] - e0;
  const int Tb = lens[b];
  const size_t r0 = (size_t)row_start[b];
  if (threadIdx.x == 0) {
    fwd[start[b]] = 0.f;
    bwd[(size_t)Tb * S + end[b]] = 0.f;
  }
  __syncthreads();
  auto cost = [&](int e, int t, int l) -> float {  // l = segment length - 1
    return weights[e] + am_scale * am[((r0 + t) * L + l) * V + e_em[e]] + length_models[(size_t)e_lenmod[e] * L + l];
  };
  for (int t = 0; t < Tb; ++t) {
    const int lmax = min(L, Tb - t);
    const float* cur = fwd + (size_t)t * S;
    for (int i = threadIdx.x; i < ne * lmax; i += blockDim.x) {
      const int e = e0 + i / lmax, l = i % lmax;
      const float s = cur[e_from[e]];
      if (s > -INFINITY) atomic_log_add(fwd + (size_t)(t + l + 1) * S + e_to[e], s - cost(e, t, l));
    }
    __syncthreads();
  }
  for (int t = Tb - 1; t >= 0; --t) {
    const int lmax = min(L, Tb - t);
    float* cur = bwd + (size_t)t * S;
    for (int i = threadIdx.x; i < ne * lmax; i += blockDim.x) {
      const int e = e0 + i / lmax, l = i % lmax;
      const float s = bwd[(size_t)(t + l + 1) * S + e_to[e]];
      if (s > -INFINITY) atomic_log_add(cur + e_from[e], s - cost(e, t, l));
    }
    __syncthreads();
  }
  const float total = bwd[start[b]];
  if (threadIdx.x == 0) obs[b] = total;
  if (total == -INFINITY) return;
  for (int t = 0; t < Tb; ++t) {
    const int lmax = min(L, Tb - t);
    for (int i = threadIdx.x; i < ne * lmax; i += blockDim.x) {
      const int e = e0 + i / lmax, l = i % lmax;
      const float a = fwd[(size_t)t * S + e_from[e]], c = bwd[(size_t)(t + l + 1) * S + e_to[e]];
      if (a > -INFINITY && c > -INFINITY) atomic_log_add(out + ((r0 + t) * L + l) * V + e_em[e], a - cost(e, t, l) + c - total);
    }
  }
}

// best path: score [T+1, S] as packed (score, edge) words pre-filled with 0 (= "minus infinity": no edge); alignment [T, B]; best [B]
__global__ void __launch_bounds__(256)
viterbi_kernel(const int* __restrict__ e_from, const int* __restrict__ e_to, const int* __restrict__ e_em, const float* __restrict__ weights,
               const int* __restrict__ edge_start, const float* __restrict__ am, const int* __restrict__ start, const int* __restrict__ end,
               const int* __restrict__ end2, const int* __restrict__ lens, int T, int B, int V, int S, unsigned long long* __restrict__ score,
               int* __restrict__ alignment, float* __restrict__ best) {
  const int b = blockIdx.x;
  const int e0 = edge_start[b], e1 = edge_start[b + 1];
  const int Tb = lens[b];
  if (threadIdx.x == 0) score[start[b]] = pack_max(0.f, 0x7fffffff);
  __syncthreads();
  for (int t = 0; t < Tb; ++t) {
    const unsigned long long* cur = score + (size_t)t * S;
    unsigned long long* nxt = score + (size_t)(t + 1) * S;
    const float* amt = am + ((size_t)t * B + b) * V;
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const unsigned long long p = cur[e_from[e]];
      if (p != 0ull) atomicMax(nxt + e_to[e], pack_max(unpack_score(p) - weights[e] - amt[e_em[e]], e));
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int st = end[b];
    unsigned long long p = score[(size_t)Tb * S + st];
    if (end2 && end2[b] >= 0) {
      const unsigned long long p2 = score[(size_t)Tb * S + end2[b]];
      if (p2 > p) {
        p = p2;
        st = end2[b];
      }
    }
    best[b] = p != 0ull ? unpack_score(p) : -INFINITY;
    for (int t = Tb - 1; t >= 0; --t) {
      const unsigned long long q = score[(size_t)(t + 1) * S + st];
      if (q == 0ull) {
        alignment[(size_t)t * B + b] = 0;
        continue;
      }
      const int e = (int)(q & 0xffffffffu);
      alignment[(size_t)t * B + b] = e_em[e];
      st = e_from[e];
    }
    for (int t = Tb; t < T; ++t) alignment[(size_t)t * B + b] = 0;
  }
}

// CTC topology with label loops: states of sequence b are base_b + {0 .. 2*S_b}: even = blank, odd = labels. Edges per state:
// loop; to the next state; from a label to the next label when they differ. edge slots per sequence: 3 * (2*S_b + 1), unused
// slots are written as self-loops with weight +inf on the start state (they never contribute).
__global__ void ctc_fsa_kernel(const int* __restrict__ targets, int ldt, const int* __restrict__ tgt_lens, const int* __restrict__ state_base,
                               const int* __restrict__ edge_base, int blank, int label_loop, int* __restrict__ e_from, int* __restrict__ e_to,
                               int* __restrict__ e_em, float* __restrict__ weights, int* __restrict__ start, int* __restrict__ end,
                               int* __restrict__ end2) {
  const int b = blockIdx.x;
  const int Sb = tgt_lens[b];
  const int n_states = 2 * Sb + 1;
  const int sb = state_base[b], eb = edge_base[b];
  const int* tg = targets + (size_t)b * ldt;
  if (threadIdx.x == 0) {
    start[b] = sb;
    end[b] = sb + n_states - 1;
    end2[b] = Sb > 0 ? sb + n_states - 2 : -1;
  }
  for (int s = threadIdx.x; s < n_states; s += blockDim.x) {
    const bool is_label = s & 1;
    const int em = is_label ? tg[s / 2] : blank;
    // edges are labelled with the emission of their *target* state
    int k = eb + 3 * s;
    // loop
    const bool loop_ok = !is_label || label_loop;
    e_from[k] = sb + s; e_to[k] = sb + s; e_em[k] = em; weights[k] = loop_ok ? 0.f : INFINITY;
    ++k;
    // to next state
    if (s + 1 < n_states) {
      const int em1 = ((s + 1) & 1) ? tg[(s + 1) / 2] : blank;
      e_from[k] = sb + s; e_to[k] = sb + s + 1; e_em[k] = em1; weights[k] = 0.f;
    } else {
      e_from[k] = sb; e_to[k] = sb; e_em[k] = blank; weights[k] = INFINITY;
    }
    ++k;
    // label to next label (skip the blank) if different
    if (is_label && s + 2 < n_states && tg[s / 2] != tg[s / 2 + 1]) {
      e_from[k] = sb + s; e_to[k] = sb + s + 2; e_em[k] = tg[s / 2 + 1]; weights[k] = 0.f;
    } else {
      e_from[k] = sb; e_to[k] = sb; e_em[k] = blank; weights[k] = INFINITY;
    }
  }
}

}  // namespace

RB_EXPORT int rb200_fsa_fbw(const int* e_from, const int* e_to, const int* e_em, const float* weights, const int* edge_start, const float* am,
                            const int* start, const int* end, const int* end2, const int* lens, int T, int B, int V, int S, float* fwd, float* bwd,
                            float* out, float* obs, cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  fbw_kernel<<<B, 256, 0, stream>>>(e_from, e_to, e_em, weights, edge_start, am, start, end, end2, lens, T, B, V, S, fwd, bwd, out, obs, nullptr, nullptr,
                                    nullptr, nullptr);
  return rb_check_launch("fsa_fbw");
}

// as rb200_fsa_fbw, with a list of weighted final states per sequence: end_start [B+1] into end_state [N] / end_weight [N] (-log)
RB_EXPORT int rb200_fsa_fbw_multi_end(const int* e_from, const int* e_to, const int* e_em, const float* weights, const int* edge_start, const float* am,
                                      const int* start, const int* end_start, const int* end_state, const float* end_weight, const int* lens, int T,
                                      int B, int V, int S, float* fwd, float* bwd, float* out, float* obs, cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  fbw_kernel<<<B, 256, 0, stream>>>(e_from, e_to, e_em, weights, edge_start, am, start, nullptr, nullptr, lens, T, B, V, S, fwd, bwd, out, obs, end_start,
                                    end_state, end_weight, nullptr);
  return rb_check_launch("fsa_fbw_multi_end");
}

// as rb200_fsa_fbw on packed scores: am and out are [N, V], the frames of sequence b are rows row_start[b] .. row_start[b] + lens[b]
RB_EXPORT int rb200_fsa_fbw_packed(const int* e_from, const int* e_to, const int* e_em, const float* weights, const int* edge_start, const float* am,
                                   const int* start, const int* end, const int* end2, const int* lens, const int* row_start, int T_max, int B, int V,
                                   int S, float* fwd, float* bwd, float* out, float* obs, cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  fbw_kernel<<<B, 256, 0, stream>>>(e_from, e_to, e_em, weights, edge_start, am, start, end, end2, lens, T_max, B, V, S, fwd, bwd, out, obs, nullptr,
                                    nullptr, nullptr, row_start);
  return rb_check_launch("fsa_fbw_packed");
}

// segmental form: see seg_fbw_kernel
RB_EXPORT int rb200_fsa_seg_fbw(const int* e_from, const int* e_to, const int* e_em, const int* e_lenmod, const float* weights, const int* edge_start,
                                const float* am, const float* length_models, const int* row_start, const int* start, const int* end, const int* lens,
                                int B, int L, int V, int S, int T_max, float am_scale, float* fwd, float* bwd, float* out, float* obs,
                                cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  seg_fbw_kernel<<<B, 256, 0, stream>>>(e_from, e_to, e_em, e_lenmod, weights, edge_start, am, length_models, row_start, start, end, lens, L, V, S, T_max,
                                        am_scale, fwd, bwd, out, obs);
  return rb_check_launch("fsa_seg_fbw");
}

RB_EXPORT int rb200_fsa_viterbi(const int* e_from, const int* e_to, const int* e_em, const float* weights, const int* edge_start, const float* am,
                                const int* start, const int* end, const int* end2, const int* lens, int T, int B, int V, int S,
                                unsigned long long* score, int* alignment, float* best, cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  viterbi_kernel<<<B, 256, 0, stream>>>(e_from, e_to, e_em, weights, edge_start, am, start, end, end2, lens, T, B, V, S, score, alignment, best);
  return rb_check_launch("fsa_viterbi");
}

RB_EXPORT int rb200_ctc_fsa(const int* targets, int ldt, const int* tgt_lens, const int* state_base, const int* edge_base, int B, int blank,
                            int label_loop, int* e_from, int* e_to, int* e_em, float* weights, int* start, int* end, int* end2, cudaStream_t stream) {
  if (B <= 0) return RB_OK;
  ctc_fsa_kernel<<<B, 128, 0, stream>>>(targets, ldt, tgt_lens, state_base, edge_base, blank, label_loop, e_from, e_to, e_em, weights, start, end, end2);
  return rb_check_launch("ctc_fsa");
}
