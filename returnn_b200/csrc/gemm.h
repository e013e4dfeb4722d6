// Internal C++ interface of the persistent tcgen05 GEMM (gemm_persist.cu), used by the C entry points and by the native
// encoder executor. D[m,n] = epilogue(alpha * op(A)·op(B)).
#pragma once
#include <cuda_runtime.h>

struct RbGemm {
  const void* a = nullptr;   // bf16; stored [m][k] (a_mn_major = 0) or [k][m] (1), row pitch lda elements
  const void* b = nullptr;   // bf16; stored [n][k] (b_mn_major = 0) or [k][n] (1), row pitch ldb elements
  void* c = nullptr;         // bf16 or fp32 [m][ldc]
  void* c2 = nullptr;        // optional bf16 [m][ldc]: receives the final value while c receives the pre-activation
  const void* bias = nullptr;
  int bias_bf16 = 0;
  int m = 0, n = 0, k = 0, lda = 0, ldb = 0, ldc = 0;
  int a_mn_major = 0, b_mn_major = 0;
  int ab_fp16 = 0;           // A and B hold IEEE fp16 instead of bf16 (same size, so the copies and layouts are the same; only the MMA reads them differently)
  int act = 0;               // 0 none, 1 relu, 2 silu, 3 gelu(erf)
  int out_fp32 = 0;
  int accumulate = 0;        // fp32 output only: 0 store, 1 c += value, 2 atomic c += value (needed with split_k > 1)
  float alpha = 1.f;
  // epilogue, applied in this order to v = alpha * acc + bias:
  const void* dact_z = nullptr;  // bf16 [m][ldc]: v *= act'(z)  (act names the function; the value itself is not activated then)
  float drop_p = 0.f;            // dropout on the (activated) value; mask of element (r, c) = philox(seed, offset + drop_site + r*ldc + c)
  const long long* seed = nullptr;
  const long long* offset = nullptr;
  unsigned long long drop_site = 0;
  const void* resid = nullptr;   // bf16 [m][ldc]: final = resid + res_scale * v
  float res_scale = 1.f;
  int split_k = 0;               // 0: chosen by the launcher (> 1 only with accumulate == 2)
  // batched form (batch > 0): problem z = b * heads + h reads A from the stored origin (b*a_rb + h*a_rh, b*a_cb + h*a_ch),
  // B likewise, and writes at element offset b*c_sb + h*c_sh. m / n / k are fixed or lens[b] where the *_from_lens flag is set;
  // a problem with an empty extent is skipped. a_rows .. b_cols are the extents of the stored matrices.
  int batch = 0, heads = 1;
  long long a_rb = 0, a_rh = 0, a_cb = 0, a_ch = 0, b_rb = 0, b_rh = 0, b_cb = 0, b_ch = 0, c_sb = 0, c_sh = 0;
  long long a_rows = 0, a_cols = 0, b_rows = 0, b_cols = 0;
  const int* lens = nullptr;
  int m_from_lens = 0, n_from_lens = 0, k_from_lens = 0;
  int* status = nullptr;         // device word: 0 fine, else (role << 24 | detail) of the wait that gave up
};

// returns an RB_* status code; the launch is asynchronous on `stream`
int rb_gemm(const RbGemm& g, cudaStream_t stream);

// CTA-pair kernel (gemm_2cta.cu): rb_gemm routes to it when rb_gemm_pair_wanted says so
bool rb_gemm_pair_wanted(const RbGemm& g);
int rb_gemm_pair(const RbGemm& g, cudaStream_t stream);
