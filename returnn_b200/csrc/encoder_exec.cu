// Native executor of the Conformer encoder stack on packed rows.
//
// One call runs the forward pass of all layers (or the backward pass of a range of layers) as a fixed sequence of kernel
// launches on one stream: LayerNorm, tcgen05 GEMMs with fused epilogues (bias, SiLU, dropout, residual, activation gradient),
// relative-position attention as batched GEMMs + softmax kernels, the GLU / depthwise conv / BatchNorm / SiLU kernels.
// The host side does no allocation: the caller passes one buffer for the saved activations and one scratch buffer, whose
// sizes rb200_enc_sizes reports. Parameter gradients are accumulated straight into the fp32 gradient arena (weight gradients
// by split-K GEMMs with atomics), so no per-parameter gradient tensors exist.
//
// Parameters come as a table [layers][P_COUNT][3] of addresses: fp32 master value, fp32 gradient, bf16 copy (GEMM weights only).
// The layer structure (reference: returnn/frontend/encoder/conformer.py, ConformerEncoderLayer.__call__):
//   x1 = x0 + 0.5 drop(FF1(LN(x0)));  x2 = x1 + drop(MHSA(LN(x1)));  x3 = x2 + drop(Conv(LN(x2)));
//   x4 = x3 + 0.5 drop(FF2(LN(x3)));  out = LN(x4)
#include "common.cuh"
#include "gemm.h"
#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <vector>

// entry points of the other translation units used here
extern "C" {
int rb200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows, int n,
                         float eps, int x_bf16, int w_bf16, int rms, cudaStream_t stream);
int rb200_layer_norm_bwd_ex(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx, float* part,
                            float* dgamma, float* dbeta, long long rows, int n, int n_part, int x_bf16, int w_bf16, int rms,
                            const void* dres, int accumulate, cudaStream_t stream);
int rb200_gemm_bf16_batched(const void* a, const void* b, void* c, const void* bias, long long a_rows, long long a_cols, long long b_rows,
                            long long b_cols, int lda, int ldb, int ldc, int m, int n, int k, int a_mn_major, int b_mn_major, int bias_bf16,
                            int act, int out_fp32, int accumulate, float alpha, int batch, int heads, const long long* offs, const int* lens,
                            int m_from_lens, int n_from_lens, int k_from_lens, int* status, cudaStream_t stream);
int rb200_att_prepare(const void* qkv, const float* u, const float* v, const int* row_batch, const int* row_pos, void* qu, void* qv, void* k,
                      void* vv, int n_rows, int heads, int dim, int lp, cudaStream_t stream);
int rb200_att_softmax_fwd_ex(const void* s_ac, const void* g, int scores_bf16, void* w, void* wd, const int* lens, int batch, int heads, int lp, int rp,
                             int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream);
int rb200_att_softmax_bwd_ex(const void* w, const void* dwd, int dwd_bf16, void* ds, void* dg, const int* lens, int batch, int heads, int lp, int rp,
                             int center, float p_drop, const long long* seed, const long long* offset, cudaStream_t stream);
int rb200_att_redrop(const void* w, void* wd, const int* lens, int batch, int heads, int lp, float p_drop, const long long* seed,
                     const long long* offset, cudaStream_t stream);
int rb200_att_pack_dqkv(const void* dqu, const void* dqv, const void* dk, const void* dv, const int* row_batch, const int* row_pos, void* dqkv,
                        int n_rows, int heads, int dim, int lp, cudaStream_t stream);
int rb200_att_rows_gather(const void* src, void* dst, const int* row_batch, const int* row_pos, int n_rows, int width, int lp, int to_padded,
                          cudaStream_t stream);
int rb200_glu_dwconv_fwd(const void* x, const float* filt, const float* bias, const int* row_batch, const int* row_pos, const int* lens,
                         void* y, float* part, int n_rows, int C, int K, cudaStream_t stream);
int rb200_bn_stats(const float* part, int n_tiles, int C, float count, float eps, float momentum, float* mean, float* rstd,
                   float* running_mean, float* running_var, cudaStream_t stream);
int rb200_bn_silu_fwd(const void* y, const float* mean, const float* rstd, const float* gamma, const float* beta, void* z, long long n_rows,
                      int C, cudaStream_t stream);
int rb200_bn_silu_bwd_ex(const void* y, const void* dz, const float* mean, const float* rstd, const float* gamma, const float* beta, void* ds,
                         float* part, int n_tiles, float* sum_ds, float* sum_ds_yh, long long n_rows, int C, int training, float* dgamma_acc,
                         float* dbeta_acc, cudaStream_t stream);
int rb200_glu_dwconv_bwd_ex(const void* x, const void* dy, const float* filt, const int* row_batch, const int* row_pos, const int* lens,
                            void* dx, float* part, float* dfilt, float* dbias, int n_rows, int C, int K, int accumulate, cudaStream_t stream);
}

// dimensions and hyper-parameters of one call (mirrored by a ctypes.Structure on the Python side)
struct RbEncDims {
  int n_rows, batch, D, F, H, Dh, conv_k, max_len, R, n_layers, training, n_launch;
  float ln_eps, p_res, p_ff, p_att, bn_eps, bn_momentum, att_scale, ff_res_scale;
};

enum {
  P_FF1_LN_G, P_FF1_LN_B, P_FF1_W1, P_FF1_B1, P_FF1_W2, P_FF1_B2,
  P_ATT_LN_G, P_ATT_LN_B, P_QKV_W, P_QKV_B, P_POS_W, P_POS_U, P_POS_V, P_PROJ_W, P_PROJ_B,
  P_CONV_LN_G, P_CONV_LN_B, P_PW1_W, P_PW1_B, P_DW_F, P_DW_B, P_BN_G, P_BN_B, P_PW2_W, P_PW2_B,
  P_FF2_LN_G, P_FF2_LN_B, P_FF2_W1, P_FF2_B1, P_FF2_W2, P_FF2_B2,
  P_FIN_LN_G, P_FIN_LN_B, P_BN_RM, P_BN_RV, P_COUNT
};

namespace {

// ---- small kernels ------------------------------------------------------------------------------------------------

// out[c] += sum_r y[r][c] with y = x, or y = dropout_mask * scale * x (then y is also written).
// A CTA owns 64 columns (8 threads x 8 columns: one 128-byte line per row) and a slice of the rows; 32 row lanes walk the
// slice with two independent 16-byte loads in flight each (three CTAs per SM). The 32 lane sums meet in shared memory and leave as ONE atomic per
// column and CTA (a CTA per full row made rows/8 atomics per column, which serialise in L2).
__global__ void __launch_bounds__(256, 3)
colsum_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ out, int rows, int C, int rows_per_cta,
              float scale, float p_drop, const long long* __restrict__ seed, const long long* __restrict__ offset, unsigned long long site) {
  rb_pdl_wait();  // may have been scheduled before the preceding kernel finished
  rb_pdl_launch();
  __shared__ float red[32][65];
  const int cg = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int col = blockIdx.y * 64 + cg * 8;
  const int r_begin = blockIdx.x * rows_per_cta;
  const int r_end = min(rows, r_begin + rows_per_cta);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool drop = p_drop > 0.f;
  const uint64_t sd = drop ? (uint64_t)seed[0] : 0, off = drop ? (uint64_t)offset[0] + site : 0;
  const uint32_t thresh = drop ? rb_dropout_thresh16(p_drop) : 0u;
  const float keep = drop ? scale / (1.f - p_drop) : scale;
  if (col < C) {
    const uint2 key = make_uint2((uint32_t)sd, (uint32_t)(sd >> 32));
    for (int rbase = r_begin + rl; rbase < r_end; rbase += 2 * 32) {
      F8 v[2];
      int64_t idx[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = rbase + u * 32;
        idx[u] = (int64_t)r * C + col;
        if (r < r_end) v[u] = load8(x, idx[u], 1);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = rbase + u * 32;
        if (r >= r_end) break;
        if (y) {
          if (drop) {
            rb_dropout_apply8(key, off + (uint64_t)idx[u], thresh, keep, v[u].v);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[u].v[i] *= keep;
          }
          store8(y, idx[u], v[u], 1);
          // sum what was stored (bf16-rounded), so that the bias gradient matches the GEMM operand
#pragma unroll
          for (int i = 0; i < 8; ++i) v[u].v[i] = __bfloat162float(__float2bfloat16(v[u].v[i]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[u].v[i];
      }
    }
  }
  if (!out) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][cg * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 64 && blockIdx.y * 64 + threadIdx.x < C) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) sum += red[k][threadIdx.x];
    atomicAdd(out + blockIdx.y * 64 + threadIdx.x, sum);
  }
}

int colsum(const void* x, void* y, float* out, int rows, int C, float scale, float p_drop, const long long* seed, const long long* offset,
           unsigned long long site, cudaStream_t s) {
  if (rows <= 0 || (!out && !y)) return RB_OK;
  if (C % 8) {
    rb_set_error("colsum: C=%d must be a multiple of 8", C);
    return RB_ERR_ARG;
  }
  const int chunks = (C + 63) / 64;
  // three resident CTAs per SM; at least 32 rows (one per lane) per CTA
  int splits = (3 * 148 + chunks - 1) / chunks;
  const int max_splits = (rows + 31) / 32;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  const int rows_per_cta = (rows + splits - 1) / splits;
  splits = (rows + rows_per_cta - 1) / rows_per_cta;
  rb_launch_pdl(colsum_kernel, dim3(splits, chunks), dim3(256), 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, out, rows, C, rows_per_cta, scale, p_drop, seed,
                                                     offset, site);
  return rb_check_launch("colsum");
}

// per-layer counter bases for the attention dropout: out[l] = offset[0] + first + l * stride
__global__ void offsets_kernel(const long long* __restrict__ offset, long long* __restrict__ out, int n, unsigned long long first,
                               unsigned long long stride) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = offset[0] + (long long)(first + (unsigned long long)i * stride);
}

// ---- buffer layout ------------------------------------------------------------------------------------------------

struct Bump {
  char* base;
  size_t off = 0;
  explicit Bump(void* b) : base(reinterpret_cast<char*>(b)) {}
  template <typename T>
  T* take(size_t count) {
    off = (off + 255) & ~(size_t)255;
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
};

typedef __nv_bfloat16 bf16;

struct Geometry {
  int n, B, D, F, H, Dh, HD, K, Lp, Rp, R, center, L;
  bool keep_wd;  // attention dropout active: dropout(w) is saved next to w
  size_t pad_rows;     // B * Lp
  size_t score_elems;  // B * H * Lp * Lp
  size_t band_elems;   // H * B * Lp * Rp
  unsigned long long site_ff_act, site_ff_out, site_att, site_att_out, site_conv_out, site_ff2_act, site_ff2_out, per_layer;
  explicit Geometry(const RbEncDims& d) {
    keep_wd = d.training && d.p_att > 0.f;
    n = d.n_rows; B = d.batch; D = d.D; F = d.F; H = d.H; Dh = d.Dh; HD = H * Dh; K = d.conv_k; L = d.n_layers;
    Lp = (d.max_len + 63) / 64 * 64;
    Rp = 2 * Lp;
    R = d.R;
    center = (R - 1) / 2;
    pad_rows = (size_t)B * Lp;
    score_elems = (size_t)B * H * Lp * Lp;
    band_elems = (size_t)H * B * Lp * Rp;
    auto r8 = [](unsigned long long v) { return (v + 7ull) & ~7ull; };
    unsigned long long o = 0;
    site_ff_act = o; o += r8((unsigned long long)n * F);
    site_ff_out = o; o += r8((unsigned long long)n * D);
    site_att = o; o += r8(score_elems);
    site_att_out = o; o += r8((unsigned long long)n * D);
    site_conv_out = o; o += r8((unsigned long long)n * D);
    site_ff2_act = o; o += r8((unsigned long long)n * F);
    site_ff2_out = o; o += r8((unsigned long long)n * D);
    per_layer = o;
  }
};

// activations kept from forward to backward, per layer
struct Saved {
  bf16 *ln1, *z1, *a1, *x1, *ln2, *qu, *qv, *kk, *vv, *w, *wd, *posp, *att, *x2, *ln3, *g, *y, *zc, *x3, *ln4, *z2, *a2, *x4, *out;
  float *st1, *st2, *st3, *st4, *st5, *bn_ms;
};

struct SavedLayout {
  long long* att_off = nullptr;  // [L]
  size_t total = 0;
  Bump bump;
  const Geometry& g;
  SavedLayout(void* base, const Geometry& geo) : bump(base), g(geo) { att_off = bump.take<long long>(geo.L); }
  Saved layer() {
    Saved s;
    const size_t n = g.n, D = g.D, F = g.F, HD = g.HD;
    s.ln1 = bump.take<bf16>(n * D); s.st1 = bump.take<float>(2 * n);
    s.z1 = bump.take<bf16>(n * F); s.a1 = bump.take<bf16>(n * F); s.x1 = bump.take<bf16>(n * D);
    s.ln2 = bump.take<bf16>(n * D); s.st2 = bump.take<float>(2 * n);
    s.qu = bump.take<bf16>(4 * g.pad_rows * HD);  // qu, qv, kk, vv back to back: one memset
    s.qv = s.qu ? s.qu + g.pad_rows * HD : nullptr;
    s.kk = s.qu ? s.qu + 2 * g.pad_rows * HD : nullptr;
    s.vv = s.qu ? s.qu + 3 * g.pad_rows * HD : nullptr;
    s.w = bump.take<bf16>(g.score_elems);
    // the dropped probabilities are kept too (recomputing them in the backward pass costs a full pass over the scores)
    s.wd = g.keep_wd ? bump.take<bf16>(g.score_elems) : s.w;
    s.posp = bump.take<bf16>((size_t)g.R * HD);
    s.att = bump.take<bf16>(n * HD); s.x2 = bump.take<bf16>(n * D);
    s.ln3 = bump.take<bf16>(n * D); s.st3 = bump.take<float>(2 * n);
    s.g = bump.take<bf16>(n * 2 * D); s.y = bump.take<bf16>(n * D); s.bn_ms = bump.take<float>(2 * D);
    s.zc = bump.take<bf16>(n * D); s.x3 = bump.take<bf16>(n * D);
    s.ln4 = bump.take<bf16>(n * D); s.st4 = bump.take<float>(2 * n);
    s.z2 = bump.take<bf16>(n * F); s.a2 = bump.take<bf16>(n * F); s.x4 = bump.take<bf16>(n * D);
    s.st5 = bump.take<float>(2 * n);
    s.out = bump.take<bf16>(n * D);
    return s;
  }
};

inline int ln_parts(int n) {
  int p = (n + 15) / 16;
  if (p > 592) p = 592;
  if (p < 1) p = 1;
  return p;
}
inline int bn_tiles_a(int n) {  // 16 rows per CTA: a few hundred CTAs for the batches of a training step
  int t = (n + 15) / 16;
  if (t > 592) t = 592;
  if (t < 1) t = 1;
  return t;
}

// ---- per-op timing (off by default) ---------------------------------------------------------------------------------
// When enabled, every op of a forward/backward call is followed by an event on the stream; at the end of the call the stream
// is synchronised and the time between consecutive events is added to a table keyed by the op's tag. The numbers are
// in-pipeline times (warm L2, no gaps between launches), which is what a step is made of; a profiler that serialises and
// flushes caches reports other numbers.
struct OpProfile {
  std::mutex mu;
  bool enabled = false;
  std::map<std::string, std::pair<long long, double>> table;  // tag -> (count, ms)
  std::map<std::string, double> host_ms;                       // tag -> host time spent issuing the op
  std::vector<cudaEvent_t> pool;
  cudaEvent_t get() {
    if (!pool.empty()) {
      cudaEvent_t e = pool.back();
      pool.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};
OpProfile& op_profile() {
  static OpProfile p;
  return p;
}

struct Exec {
  const RbEncDims& d;
  Geometry g;
  const long long* tab;
  const int *lens, *row_batch, *row_pos;
  const long long *seed, *offset;
  int* status;
  cudaStream_t s;
  int st = RB_OK;
  int launches = 0;
  bool prof = false;
  std::vector<std::pair<std::string, cudaEvent_t>> marks;
  std::vector<double> mark_host_ms;
  std::chrono::steady_clock::time_point last_host;

  Exec(const RbEncDims& dims, const long long* t, const int* l, const int* rb, const int* rp, const long long* sd, const long long* of,
       int* stat, cudaStream_t stream)
      : d(dims), g(dims), tab(t), lens(l), row_batch(rb), row_pos(rp), seed(sd), offset(of), status(stat), s(stream) {
    OpProfile& p = op_profile();
    {
      std::lock_guard<std::mutex> lk(p.mu);
      prof = p.enabled;
    }
    if (prof) mark("(start)");  // takes the lock itself
  }
  void mark(const char* tag) {
    // caller holds no lock; the pool is only touched under the lock
    OpProfile& p = op_profile();
    cudaEvent_t ev;
    {
      std::lock_guard<std::mutex> lk(p.mu);
      ev = p.get();
    }
    const auto now = std::chrono::steady_clock::now();
    mark_host_ms.push_back(marks.empty() ? 0.0 : std::chrono::duration<double, std::milli>(now - last_host).count());
    cudaEventRecord(ev, s);
    last_host = std::chrono::steady_clock::now();  // the event record itself is not the op's cost
    std::string t(tag ? tag : "?");
    const size_t par = t.find('(', 1);
    if (par != std::string::npos) t.resize(par);
    marks.emplace_back(t, ev);
  }
  // end of a call: with timing on, wait for the stream and book the intervals
  void finish() {
    if (!prof || marks.size() < 2) return;
    cudaStreamSynchronize(s);
    OpProfile& p = op_profile();
    std::lock_guard<std::mutex> lk(p.mu);
    for (size_t i = 1; i < marks.size(); ++i) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, marks[i - 1].second, marks[i].second) == cudaSuccess) {
        auto& slot = p.table[marks[i].first];
        slot.first += 1;
        slot.second += ms;
      }
      p.host_ms[marks[i].first] += mark_host_ms[i];
    }
    for (auto& m : marks) p.pool.push_back(m.second);
    marks.clear();
    mark_host_ms.clear();
  }

  const float* p32(int l, int i) const { return reinterpret_cast<const float*>(tab[((size_t)l * P_COUNT + i) * 3 + 0]); }
  float* g32(int l, int i) const { return reinterpret_cast<float*>(tab[((size_t)l * P_COUNT + i) * 3 + 1]); }
  const bf16* p16(int l, int i) const { return reinterpret_cast<const bf16*>(tab[((size_t)l * P_COUNT + i) * 3 + 2]); }
  unsigned long long site(int l, unsigned long long s_) const { return (unsigned long long)l * g.per_layer + s_; }
  float pdrop(float p) const { return d.training ? p : 0.f; }

  void run(int code, const char* tag = nullptr) {
    ++launches;
    if (st == RB_OK && code != RB_OK) st = code;
    if (prof) mark(tag);
  }
  void run_tagged(const char* tag, int code) { run(code, tag); }
  bool ok() const { return st == RB_OK; }

  // y = [resid + res_scale *] drop(act(x·W + b)); z (optional) receives the pre-activation
  void linear_fwd(const void* x, int l, int wi, int bi, int m, int in, int out, void* y, void* z, int act, float p_drop,
                  unsigned long long site_, const void* resid, float res_scale) {
    if (!ok()) return;
    RbGemm q;
    q.a = x; q.b = p16(l, wi); q.m = m; q.n = out; q.k = in; q.lda = in; q.ldb = out; q.ldc = out;
    q.a_mn_major = 0; q.b_mn_major = 1;
    q.bias = bi >= 0 ? p32(l, bi) : nullptr;
    q.act = act;
    if (z) { q.c = z; q.c2 = y; } else { q.c = y; }
    q.drop_p = p_drop; q.seed = seed; q.offset = offset; q.drop_site = site_;
    q.resid = resid; q.res_scale = res_scale; q.status = status;
    run(rb_gemm(q, s), "gemm_fwd");
  }
  // dx = (dy·W^T) [* act'(z)] [* dropout mask]
  void linear_dgrad(const void* dy, int l, int wi, int m, int in, int out, void* dx, const void* z, int act, float p_drop,
                    unsigned long long site_) {
    if (!ok()) return;
    RbGemm q;
    q.a = dy; q.b = p16(l, wi); q.c = dx; q.m = m; q.n = in; q.k = out; q.lda = out; q.ldb = out; q.ldc = in;
    q.a_mn_major = 0; q.b_mn_major = 0;
    q.dact_z = z; q.act = z ? act : 0;
    q.drop_p = p_drop; q.seed = seed; q.offset = offset; q.drop_site = site_; q.status = status;
    run(rb_gemm(q, s), "gemm_dgrad");
  }
  // dW += x^T·dy (fp32, atomics, contraction split over CTAs); db += column sums of dy
  void linear_wgrad(const void* x, const void* dy, int l, int wi, int bi, int m, int in, int out, bool bias_sum) {
    if (!ok()) return;
    if (g32(l, wi)) {
      RbGemm q;
      q.a = x; q.b = dy; q.c = g32(l, wi); q.m = in; q.n = out; q.k = m; q.lda = in; q.ldb = out; q.ldc = out;
      q.a_mn_major = 1; q.b_mn_major = 1; q.out_fp32 = 1; q.accumulate = 2; q.status = status;
      run(rb_gemm(q, s), "gemm_wgrad");
    }
    if (bias_sum && bi >= 0 && g32(l, bi)) run(colsum(dy, nullptr, g32(l, bi), m, out, 1.f, 0.f, nullptr, nullptr, 0, s), "colsum_bias");
  }
  void layer_norm(const void* x, int l, int gi, void* y, float* stats) {
    if (!ok()) return;
    run(rb200_layer_norm_fwd(x, p32(l, gi), p32(l, gi + 1), y, stats, stats + g.n, g.n, g.D, d.ln_eps, 1, 0, 0, s), "layer_norm_fwd");
  }
  void layer_norm_bwd(const void* x, const void* dy, int l, int gi, const float* stats, void* dx, const void* dres, float* part) {
    if (!ok()) return;
    run(rb200_layer_norm_bwd_ex(x, dy, p32(l, gi), stats, stats + g.n, dx, part, g32(l, gi), g32(l, gi + 1), g.n, g.D, ln_parts(g.n), 1, 0, 0,
                                dres, 1, s), "layer_norm_bwd");
    ++launches;
  }
  void bgemm(const void* a, const void* b, void* c, int m, int n, int k, int a_mn, int b_mn, int lda, int ldb, int ldc, long long a_rows,
             long long a_cols, long long b_rows, long long b_cols, const long long (&offs)[10], int batch, int heads, const int* lens_, int m_l,
             int n_l, int k_l, float alpha, int out_fp32) {
    if (!ok()) return;
    run(rb200_gemm_bf16_batched(a, b, c, nullptr, a_rows, a_cols, b_rows, b_cols, lda, ldb, ldc, m, n, k, a_mn, b_mn, 0, 0, out_fp32, 0, alpha,
                                batch, heads, offs, lens_, m_l, n_l, k_l, status, s), "gemm_batched");
  }
  void memset0(void* p, size_t bytes) {
    if (!ok()) return;
    cudaError_t e = cudaMemsetAsync(p, 0, bytes, s);
    ++launches;
    if (e != cudaSuccess) {
      rb_set_error("encoder: cudaMemsetAsync: %s", cudaGetErrorString(e));
      st = RB_ERR_LAUNCH;
    }
  }
};

// scratch of the forward pass
struct TmpFwd {
  bf16 *qkv, *o_pad;
  float *s_ac, *band, *conv_part;
  TmpFwd(void* base, const Geometry& g, size_t* total) {
    Bump b(base);
    qkv = b.take<bf16>((size_t)g.n * 3 * g.HD);
    s_ac = b.take<float>(g.score_elems);
    band = b.take<float>(g.band_elems);
    o_pad = b.take<bf16>(g.pad_rows * g.HD);
    conv_part = b.take<float>((size_t)((g.n + 31) / 32) * 2 * g.D);
    if (total) *total = b.off + 256;
  }
};

// scratch of the backward pass
struct TmpBwd {
  bf16 *dA, *dB, *tD, *tD2, *tD3, *tW, *datt, *do_pad, *ds, *dband, *dqu, *dqv, *dk, *dv, *dpos;
  float *dwd, *ln_part, *bn_part, *conv_part, *sum_ds, *sum_ds_yh;
  TmpBwd(void* base, const Geometry& g, size_t* total) {
    Bump b(base);
    const size_t n = g.n, D = g.D, HD = g.HD;
    size_t wide = g.F;
    if ((size_t)3 * HD > wide) wide = 3 * HD;
    if ((size_t)2 * D > wide) wide = 2 * D;
    dA = b.take<bf16>(n * D); dB = b.take<bf16>(n * D);
    tD = b.take<bf16>(n * D); tD2 = b.take<bf16>(n * D); tD3 = b.take<bf16>(n * D);
    tW = b.take<bf16>(n * wide);
    datt = b.take<bf16>(n * HD);
    do_pad = b.take<bf16>(g.pad_rows * HD);
    ds = b.take<bf16>(g.score_elems);
    dband = b.take<bf16>(g.band_elems);
    dqu = b.take<bf16>(4 * g.pad_rows * HD);
    dqv = dqu ? dqu + g.pad_rows * HD : nullptr;
    dk = dqu ? dqu + 2 * g.pad_rows * HD : nullptr;
    dv = dqu ? dqu + 3 * g.pad_rows * HD : nullptr;
    dpos = b.take<bf16>((size_t)g.R * HD);
    dwd = b.take<float>(g.score_elems);
    ln_part = b.take<float>((size_t)ln_parts(g.n) * 2 * D);
    bn_part = b.take<float>((size_t)bn_tiles_a(g.n) * 2 * D);
    conv_part = b.take<float>((size_t)((g.n + 31) / 32) * D * (g.K + 1));
    sum_ds = b.take<float>(D); sum_ds_yh = b.take<float>(D);
    if (total) *total = b.off + 256;
  }
};

int check_dims(const RbEncDims& d) {
  const Geometry g(d);
  if (d.n_rows <= 0 || d.batch <= 0 || d.n_layers <= 0) {
    rb_set_error("encoder: empty batch");
    return RB_ERR_ARG;
  }
  if (g.D % 64 || g.F % 8 || g.Dh % 64 || g.HD != g.D || g.Lp > 512 || g.K < 1 || g.K > 64 || g.R > g.Rp || g.center < d.max_len - 1) {
    rb_set_error("encoder: unsupported geometry D=%d F=%d H=%d Dh=%d max_len=%d K=%d R=%d", g.D, g.F, g.H, g.Dh, d.max_len, g.K, g.R);
    return RB_ERR_UNSUPPORTED;
  }
  return RB_OK;
}

}  // namespace

// bytes of the three caller-provided buffers, where the stack output [n_rows, D] bf16 lies inside `saved`, and how many
// dropout counters one forward pass consumes (the caller advances its offset by that much after the call)
RB_EXPORT int rb200_enc_sizes(const RbEncDims* d, long long* saved_bytes, long long* tmp_fwd_bytes, long long* tmp_bwd_bytes,
                              long long* out_offset, long long* rng_count) {
  int st = check_dims(*d);
  if (st) return st;
  const Geometry g(*d);
  SavedLayout lay(nullptr, g);
  Saved last;
  for (int l = 0; l < g.L; ++l) last = lay.layer();
  (void)last;
  size_t out_off;
  {
    // the output of the last layer is the last n*D bf16 block taken
    out_off = lay.bump.off - (size_t)g.n * g.D * sizeof(bf16);
  }
  size_t tf = 0, tb = 0;
  TmpFwd f(nullptr, g, &tf);
  TmpBwd b(nullptr, g, &tb);
  *saved_bytes = (long long)(lay.bump.off + 256);
  *tmp_fwd_bytes = (long long)tf;
  *tmp_bwd_bytes = (long long)tb;
  *out_offset = (long long)out_off;
  *rng_count = (long long)(g.per_layer * (unsigned long long)g.L);
  return RB_OK;
}

// Forward pass of all layers. x_in [n_rows, D] bf16; sinus [R, D] bf16 (relative positions -(L-1) .. L-1, L >= max_len);
// saved / tmp: 256-byte aligned buffers of the sizes reported by rb200_enc_sizes. Returns the number of launches in *n_launch.
RB_EXPORT int rb200_enc_forward(const RbEncDims* dims, const long long* tab, const void* x_in, const void* sinus, const int* lens,
                                const int* row_batch, const int* row_pos, void* saved, void* tmp, const long long* seed, const long long* offset,
                                int* status, int* n_launch, cudaStream_t stream) {
  int st = check_dims(*dims);
  if (st) return st;
  Exec e(*dims, tab, lens, row_batch, row_pos, seed, offset, status, stream);
  const Geometry& g = e.g;
  const RbEncDims& d = *dims;
  SavedLayout lay(saved, g);
  TmpFwd t(tmp, g, nullptr);
  const float p_res = e.pdrop(d.p_res), p_ff = e.pdrop(d.p_ff), p_att = e.pdrop(d.p_att);
  if (p_att > 0.f) {
    offsets_kernel<<<1, 64, 0, stream>>>(offset, lay.att_off, g.L, g.site_att, g.per_layer);
    e.run_tagged("rb_check_launch", rb_check_launch("enc_offsets"));
  }
  const void* x0 = x_in;
  const int n = g.n, D = g.D, F = g.F, HD = g.HD, Lp = g.Lp, Rp = g.Rp, B = g.B, H = g.H, Dh = g.Dh;
  for (int l = 0; l < g.L && e.ok(); ++l) {
    Saved sv = lay.layer();
    // ---- feed-forward 1
    e.layer_norm(x0, l, P_FF1_LN_G, sv.ln1, sv.st1);
    e.linear_fwd(sv.ln1, l, P_FF1_W1, P_FF1_B1, n, D, F, sv.a1, sv.z1, 2, p_ff, e.site(l, g.site_ff_act), nullptr, 1.f);
    e.linear_fwd(sv.a1, l, P_FF1_W2, P_FF1_B2, n, F, D, sv.x1, nullptr, 0, p_res, e.site(l, g.site_ff_out), x0, d.ff_res_scale);
    // ---- self-attention
    e.layer_norm(sv.x1, l, P_ATT_LN_G, sv.ln2, sv.st2);
    e.linear_fwd(sv.ln2, l, P_QKV_W, P_QKV_B, n, D, 3 * HD, t.qkv, nullptr, 0, 0.f, 0, nullptr, 1.f);
    e.linear_fwd(sinus, l, P_POS_W, -1, g.R, D, HD, sv.posp, nullptr, 0, 0.f, 0, nullptr, 1.f);
    e.memset0(sv.qu, 4 * g.pad_rows * HD * sizeof(bf16));
    if (e.ok()) e.run_tagged("att_prepare", rb200_att_prepare(t.qkv, e.p32(l, P_POS_U), e.p32(l, P_POS_V), row_batch, row_pos, sv.qu, sv.qv, sv.kk, sv.vv, n, H, Dh, Lp, stream));
    {
      const long long o1[10] = {Lp, 0, 0, Dh, Lp, 0, 0, Dh, (long long)H * Lp * Lp, (long long)Lp * Lp};
      // scores and bias band in bf16, like the matmul outputs of the reference under autocast: halves the traffic of this stage
      e.bgemm(sv.qu, sv.kk, t.s_ac, Lp, Lp, Dh, 0, 0, HD, HD, Lp, (long long)B * Lp, HD, (long long)B * Lp, HD, o1, B * H, H, lens, 1, 1, 0,
              d.att_scale, 0);
      const long long o2[10] = {Lp, 0, 0, Dh, 0, 0, 0, Dh, (long long)Lp * Rp, (long long)B * Lp * Rp};
      e.bgemm(sv.qv, sv.posp, t.band, Lp, g.R, Dh, 0, 0, HD, HD, Rp, (long long)B * Lp, HD, g.R, HD, o2, B * H, H, lens, 1, 0, 0, d.att_scale, 0);
    }
    // w and wd need no memset: the softmax kernel zeroes the margin that the GEMMs read beyond each sequence's length
    bf16* wd = p_att > 0.f ? sv.wd : sv.w;
    if (e.ok()) e.run_tagged("att_softmax_fwd_ex", rb200_att_softmax_fwd_ex(t.s_ac, t.band, 1, sv.w, wd, lens, B, H, Lp, Rp, g.center, p_att, seed, lay.att_off + l, stream));
    {
      const long long o3[10] = {(long long)H * Lp, Lp, 0, 0, Lp, 0, 0, Dh, (long long)Lp * HD, Dh};
      e.bgemm(wd, sv.vv, t.o_pad, Lp, Dh, Lp, 0, 1, Lp, HD, HD, (long long)B * H * Lp, Lp, (long long)B * Lp, HD, o3, B * H, H, lens, 1, 0, 1, 1.f, 0);
    }
    if (e.ok()) e.run_tagged("att_rows_gather", rb200_att_rows_gather(t.o_pad, sv.att, row_batch, row_pos, n, HD, Lp, 0, stream));
    e.linear_fwd(sv.att, l, P_PROJ_W, P_PROJ_B, n, HD, D, sv.x2, nullptr, 0, p_res, e.site(l, g.site_att_out), sv.x1, 1.f);
    // ---- convolution module
    e.layer_norm(sv.x2, l, P_CONV_LN_G, sv.ln3, sv.st3);
    e.linear_fwd(sv.ln3, l, P_PW1_W, P_PW1_B, n, D, 2 * D, sv.g, nullptr, 0, 0.f, 0, nullptr, 1.f);
    if (e.ok()) e.run_tagged("glu_dwconv_fwd", rb200_glu_dwconv_fwd(sv.g, e.p32(l, P_DW_F), e.p32(l, P_DW_B), row_batch, row_pos, lens, sv.y, t.conv_part, n, D, g.K, stream));
    if (e.ok()) {
      const bool upd = d.training != 0;
      if (d.training) {
        e.run_tagged("bn_stats", rb200_bn_stats(t.conv_part, (n + 31) / 32, D, (float)n, d.bn_eps, d.bn_momentum, sv.bn_ms, sv.bn_ms + D,
                             upd ? const_cast<float*>(e.p32(l, P_BN_RM)) : nullptr, upd ? const_cast<float*>(e.p32(l, P_BN_RV)) : nullptr, stream));
      } else {
        rb_set_error("encoder: the native executor runs the training graph only");
        e.st = RB_ERR_UNSUPPORTED;
      }
    }
    if (e.ok()) e.run_tagged("bn_silu_fwd", rb200_bn_silu_fwd(sv.y, sv.bn_ms, sv.bn_ms + D, e.p32(l, P_BN_G), e.p32(l, P_BN_B), sv.zc, n, D, stream));
    e.linear_fwd(sv.zc, l, P_PW2_W, P_PW2_B, n, D, D, sv.x3, nullptr, 0, p_res, e.site(l, g.site_conv_out), sv.x2, 1.f);
    // ---- feed-forward 2
    e.layer_norm(sv.x3, l, P_FF2_LN_G, sv.ln4, sv.st4);
    e.linear_fwd(sv.ln4, l, P_FF2_W1, P_FF2_B1, n, D, F, sv.a2, sv.z2, 2, p_ff, e.site(l, g.site_ff2_act), nullptr, 1.f);
    e.linear_fwd(sv.a2, l, P_FF2_W2, P_FF2_B2, n, F, D, sv.x4, nullptr, 0, p_res, e.site(l, g.site_ff2_out), sv.x3, d.ff_res_scale);
    // ---- final LayerNorm
    e.layer_norm(sv.x4, l, P_FIN_LN_G, sv.out, sv.st5);
    x0 = sv.out;
  }
  e.finish();
  if (n_launch) *n_launch = e.launches;
  return e.st;
}

// Backward pass of layers [layer_lo, layer_hi). dx [n_rows, D] bf16 holds the gradient w.r.t. the output of layer
// layer_hi-1 on entry and w.r.t. the input of layer layer_lo on return. x_in is the input of layer 0 (as in forward).
RB_EXPORT int rb200_enc_backward(const RbEncDims* dims, const long long* tab, const void* x_in, const void* sinus, const int* lens,
                                 const int* row_batch, const int* row_pos, void* saved, void* tmp, void* dx, int layer_lo, int layer_hi,
                                 const long long* seed, const long long* offset, int* status, int* n_launch, cudaStream_t stream) {
  int st = check_dims(*dims);
  if (st) return st;
  Exec e(*dims, tab, lens, row_batch, row_pos, seed, offset, status, stream);
  const Geometry& g = e.g;
  const RbEncDims& d = *dims;
  if (layer_lo < 0 || layer_hi > g.L || layer_lo >= layer_hi) {
    rb_set_error("encoder backward: layer range [%d, %d) of %d", layer_lo, layer_hi, g.L);
    return RB_ERR_ARG;
  }
  SavedLayout lay(saved, g);
  std::vector<Saved> sv_all(g.L);
  for (int l = 0; l < g.L; ++l) sv_all[l] = lay.layer();
  TmpBwd t(tmp, g, nullptr);
  const float p_res = e.pdrop(d.p_res), p_ff = e.pdrop(d.p_ff), p_att = e.pdrop(d.p_att);
  const int n = g.n, D = g.D, F = g.F, HD = g.HD, Lp = g.Lp, Rp = g.Rp, B = g.B, H = g.H, Dh = g.Dh;

  // dropout(residual-branch) backward + bias gradient:  dy = mask * scale * dx_total;  db += colsum(dy)
  auto branch_in = [&](const void* dxt, void* dy, int l, int bi, float scale, float p, unsigned long long site_) {
    if (!e.ok()) return;
    e.run_tagged("colsum_dropout", colsum(dxt, dy, bi >= 0 ? e.g32(l, bi) : nullptr, n, D, scale, p, seed, offset, site_, stream));
  };

  for (int l = layer_hi - 1; l >= layer_lo && e.ok(); --l) {
    const Saved& sv = sv_all[l];
    const void* x0 = l == 0 ? x_in : (const void*)sv_all[l - 1].out;
    // ---- final LayerNorm: dx (d out) -> dA (d x4)
    e.layer_norm_bwd(sv.x4, dx, l, P_FIN_LN_G, sv.st5, t.dA, nullptr, t.ln_part);
    // ---- feed-forward 2: dA -> dB (d x3)
    branch_in(t.dA, t.tD, l, P_FF2_B2, d.ff_res_scale, p_res, e.site(l, g.site_ff2_out));
    e.linear_wgrad(sv.a2, t.tD, l, P_FF2_W2, P_FF2_B2, n, F, D, false);
    e.linear_dgrad(t.tD, l, P_FF2_W2, n, F, D, t.tW, sv.z2, 2, p_ff, e.site(l, g.site_ff2_act));
    e.linear_wgrad(sv.ln4, t.tW, l, P_FF2_W1, P_FF2_B1, n, D, F, true);
    e.linear_dgrad(t.tW, l, P_FF2_W1, n, D, F, t.tD2, nullptr, 0, 0.f, 0);
    e.layer_norm_bwd(sv.x3, t.tD2, l, P_FF2_LN_G, sv.st4, t.dB, t.dA, t.ln_part);
    // ---- convolution module: dB -> dA (d x2)
    branch_in(t.dB, t.tD, l, P_PW2_B, 1.f, p_res, e.site(l, g.site_conv_out));
    e.linear_wgrad(sv.zc, t.tD, l, P_PW2_W, P_PW2_B, n, D, D, false);
    e.linear_dgrad(t.tD, l, P_PW2_W, n, D, D, t.tD2, nullptr, 0, 0.f, 0);
    if (e.ok()) {
      e.run_tagged("bn_silu_bwd_ex", rb200_bn_silu_bwd_ex(sv.y, t.tD2, sv.bn_ms, sv.bn_ms + D, e.p32(l, P_BN_G), e.p32(l, P_BN_B), t.tD3, t.bn_part, bn_tiles_a(n), t.sum_ds,
                                 t.sum_ds_yh, n, D, 1, e.g32(l, P_BN_G), e.g32(l, P_BN_B), stream));
      e.launches += 2;
    }
    if (e.ok()) {
      e.run_tagged("glu_dwconv_bwd_ex", rb200_glu_dwconv_bwd_ex(sv.g, t.tD3, e.p32(l, P_DW_F), row_batch, row_pos, lens, t.tW, t.conv_part, e.g32(l, P_DW_F), e.g32(l, P_DW_B), n, D,
                                    g.K, 1, stream));
      e.launches += 1;
    }
    e.linear_wgrad(sv.ln3, t.tW, l, P_PW1_W, P_PW1_B, n, D, 2 * D, true);
    e.linear_dgrad(t.tW, l, P_PW1_W, n, D, 2 * D, t.tD2, nullptr, 0, 0.f, 0);
    e.layer_norm_bwd(sv.x2, t.tD2, l, P_CONV_LN_G, sv.st3, t.dA, t.dB, t.ln_part);
    // ---- self-attention: dA -> dB (d x1)
    branch_in(t.dA, t.tD, l, P_PROJ_B, 1.f, p_res, e.site(l, g.site_att_out));
    e.linear_wgrad(sv.att, t.tD, l, P_PROJ_W, P_PROJ_B, n, HD, D, false);
    e.linear_dgrad(t.tD, l, P_PROJ_W, n, HD, D, t.datt, nullptr, 0, 0.f, 0);
    e.memset0(t.do_pad, g.pad_rows * HD * sizeof(bf16));
    if (e.ok()) e.run_tagged("att_rows_gather", rb200_att_rows_gather(t.datt, t.do_pad, row_batch, row_pos, n, HD, Lp, 1, stream));
    const bf16* wd = p_att > 0.f ? sv.wd : sv.w;
    {
      const long long o4[10] = {Lp, 0, 0, Dh, Lp, 0, 0, Dh, (long long)H * Lp * Lp, (long long)Lp * Lp};
      e.bgemm(t.do_pad, sv.vv, t.dwd, Lp, Lp, Dh, 0, 0, HD, HD, Lp, (long long)B * Lp, HD, (long long)B * Lp, HD, o4, B * H, H, lens, 1, 1, 0, 1.f, 0);
      const long long o5[10] = {(long long)H * Lp, Lp, 0, 0, Lp, 0, 0, Dh, (long long)Lp * HD, Dh};
      e.bgemm(wd, t.do_pad, t.dv, Lp, Dh, Lp, 1, 1, Lp, HD, HD, (long long)B * H * Lp, Lp, (long long)B * Lp, HD, o5, B * H, H, lens, 1, 0, 1, 1.f, 0);
    }
    e.memset0(t.dband, g.band_elems * sizeof(bf16));
    if (e.ok()) e.run_tagged("att_softmax_bwd_ex", rb200_att_softmax_bwd_ex(sv.w, t.dwd, 1, t.ds, t.dband, lens, B, H, Lp, Rp, g.center, p_att, seed, lay.att_off + l, stream));
    e.memset0(t.dqu, 2 * g.pad_rows * HD * sizeof(bf16));  // dqu, dqv: their column sums run over all padded rows
    {
      const long long o6[10] = {(long long)H * Lp, Lp, 0, 0, Lp, 0, 0, Dh, (long long)Lp * HD, Dh};
      e.bgemm(t.ds, sv.kk, t.dqu, Lp, Dh, Lp, 0, 1, Lp, HD, HD, (long long)B * H * Lp, Lp, (long long)B * Lp, HD, o6, B * H, H, lens, 1, 0, 1, d.att_scale, 0);
      e.bgemm(t.ds, sv.qu, t.dk, Lp, Dh, Lp, 1, 1, Lp, HD, HD, (long long)B * H * Lp, Lp, (long long)B * Lp, HD, o6, B * H, H, lens, 1, 0, 1, d.att_scale, 0);
      const long long o8[10] = {Lp, (long long)B * Lp, 0, 0, 0, 0, 0, Dh, (long long)Lp * HD, Dh};
      e.bgemm(t.dband, sv.posp, t.dqv, Lp, Dh, g.R, 0, 1, Rp, HD, HD, (long long)H * B * Lp, Rp, g.R, HD, o8, B * H, H, lens, 1, 0, 0, d.att_scale, 0);
      const long long o9[10] = {0, (long long)B * Lp, 0, 0, 0, 0, 0, Dh, 0, Dh};
      e.bgemm(t.dband, sv.qv, t.dpos, g.R, Dh, B * Lp, 1, 1, Rp, HD, HD, (long long)H * B * Lp, Rp, (long long)B * Lp, HD, o9, H, H, nullptr, 0, 0, 0,
              d.att_scale, 0);
    }
    if (e.ok()) e.run_tagged("att_pack_dqkv", rb200_att_pack_dqkv(t.dqu, t.dqv, t.dk, t.dv, row_batch, row_pos, t.tW, n, H, Dh, Lp, stream));
    if (e.ok() && e.g32(l, P_POS_U)) e.run_tagged("colsum", colsum(t.dqu, nullptr, e.g32(l, P_POS_U), (int)g.pad_rows, HD, 1.f, 0.f, nullptr, nullptr, 0, stream));
    if (e.ok() && e.g32(l, P_POS_V)) e.run_tagged("colsum", colsum(t.dqv, nullptr, e.g32(l, P_POS_V), (int)g.pad_rows, HD, 1.f, 0.f, nullptr, nullptr, 0, stream));
    e.linear_wgrad(sinus, t.dpos, l, P_POS_W, -1, g.R, D, HD, false);
    e.linear_wgrad(sv.ln2, t.tW, l, P_QKV_W, P_QKV_B, n, D, 3 * HD, true);
    e.linear_dgrad(t.tW, l, P_QKV_W, n, D, 3 * HD, t.tD2, nullptr, 0, 0.f, 0);
    e.layer_norm_bwd(sv.x1, t.tD2, l, P_ATT_LN_G, sv.st2, t.dB, t.dA, t.ln_part);
    // ---- feed-forward 1: dB -> dx (d x0)
    branch_in(t.dB, t.tD, l, P_FF1_B2, d.ff_res_scale, p_res, e.site(l, g.site_ff_out));
    e.linear_wgrad(sv.a1, t.tD, l, P_FF1_W2, P_FF1_B2, n, F, D, false);
    e.linear_dgrad(t.tD, l, P_FF1_W2, n, F, D, t.tW, sv.z1, 2, p_ff, e.site(l, g.site_ff_act));
    e.linear_wgrad(sv.ln1, t.tW, l, P_FF1_W1, P_FF1_B1, n, D, F, true);
    e.linear_dgrad(t.tW, l, P_FF1_W1, n, D, F, t.tD2, nullptr, 0, 0.f, 0);
    e.layer_norm_bwd(x0, t.tD2, l, P_FF1_LN_G, sv.st1, dx, t.dB, t.ln_part);
  }
  e.finish();
  if (n_launch) *n_launch = e.launches;
  return e.st;
}

// out[c] += sum over rows of x[r][c] (bf16 [rows, C] contiguous, fp32 out, atomics): bias gradient of a linear layer
RB_EXPORT int rb200_colsum_bf16(const void* x, float* out, int rows, int C, cudaStream_t stream) {
  return colsum(x, nullptr, out, rows, C, 1.f, 0.f, nullptr, nullptr, 0, stream);
}

// per-op timing of the executor calls: enable/disable (clears the table), and a text report "tag count device_ms host_ms" per line
RB_EXPORT int rb200_enc_profile_enable(int on) {
  OpProfile& p = op_profile();
  std::lock_guard<std::mutex> lk(p.mu);
  p.enabled = on != 0;
  p.table.clear();
  p.host_ms.clear();
  return RB_OK;
}

RB_EXPORT int rb200_enc_profile_report(char* buf, int len) {
  OpProfile& p = op_profile();
  std::lock_guard<std::mutex> lk(p.mu);
  std::string out;
  for (const auto& kv : p.table) {
    char line[256];
    const auto h = p.host_ms.find(kv.first);
    snprintf(line, sizeof(line), "%s %lld %.6f %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second, h == p.host_ms.end() ? 0.0 : h->second);
    out += line;
  }
  if (buf && len > 0) {
    const size_t n = out.size() < (size_t)len - 1 ? out.size() : (size_t)len - 1;
    memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return (int)out.size() + 1;
}
