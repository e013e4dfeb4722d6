// LSTM recurrence executor: the time loop runs on the host side of this library as a fixed launch sequence per step
// (recurrent projection on the tcgen05 GEMM + one fused cell kernel), forward and backward, so Python makes one call per
// sequence batch and direction. Gate order i, f, g, o; weights W_rec [4H, H]; frames t >= lens[b] leave the state untouched
// and produce zero output (with reverse = 1 every sequence therefore starts at its own last frame).
// Math of rf.LSTM / NativeLstm2 (returnn/frontend/rec.py, returnn/native_op.py:1029-1464), masking as in the reference's
// packed-sequence path (returnn/torch/frontend/_backend.py:2796-2810).
//
// Saved for backward: gates [T,B,4H] (activations, bf16), cell states [T,B,H] (fp32), previous hidden state per frame
// [T,B,H] (bf16). Backward per step: cell kernel (dz_t, dc carry, dh pass-through of masked rows) then dh_{t-1} += dz_t·W_rec
// on the GEMM with accumulation; after the loop one split-K GEMM gives dW_rec = dz^T·h_prev over all frames.
#include "common.cuh"
#include "gemm.h"

// lstm_persist.cu: the whole recurrence in one cooperative kernel, for the shapes it supports
bool rb_lstm_persist_supported(int T, int B, int H);
int rb_lstm_persist_fwd(const void* z_in, const void* w_rec, const int* lens, const float* h0, const float* c0, int T, int B, int H, int reverse,
                        void* y, float* c_all, void* gates, void* hprev_all, float* h_final, float* c_final, void* hbuf, int* status,
                        cudaStream_t stream);
int rb_lstm_persist_bwd(const void* dy, const float* dh_final, const float* dc_final, const void* w_rec, const int* lens, const void* gates,
                        const float* c_all, const float* c0, int T, int B, int H, int reverse, void* dz, float* dh0, float* dc0, int* status,
                        cudaStream_t stream);

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

// z_rec [B,4H] fp32 (h_prev·W_rec^T), z_in [B,4H] bf16 (x·W_ff^T + b) -> gates, c, h
__global__ void __launch_bounds__(256)
lstm_cell_fwd_kernel(const float* __restrict__ z_rec, const bf16* __restrict__ z_in, const int* __restrict__ lens, int t, int B, int H,
                     float* __restrict__ c_state, bf16* __restrict__ h_state, bf16* __restrict__ y_t, float* __restrict__ c_t,
                     bf16* __restrict__ gates_t, bf16* __restrict__ hprev_t) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  const size_t zo = (size_t)b * 4 * H + j;
  const bool valid = !lens || t < lens[b];
  const bf16 hp = h_state[idx];
  hprev_t[idx] = hp;
  const float cp = c_state[idx];
  if (!valid) {
    y_t[idx] = __float2bfloat16(0.f);
    c_t[idx] = cp;
    gates_t[zo] = gates_t[zo + H] = gates_t[zo + 2 * H] = gates_t[zo + 3 * H] = __float2bfloat16(0.f);
    return;
  }
  const float i = sigm(z_rec[zo] + __bfloat162float(z_in[zo]));
  const float f = sigm(z_rec[zo + H] + __bfloat162float(z_in[zo + H]));
  const float g = tanhf(z_rec[zo + 2 * H] + __bfloat162float(z_in[zo + 2 * H]));
  const float o = sigm(z_rec[zo + 3 * H] + __bfloat162float(z_in[zo + 3 * H]));
  const float c = f * cp + i * g;
  const float h = o * tanhf(c);
  c_state[idx] = c;
  c_t[idx] = c;
  const bf16 hb = __float2bfloat16(h);
  h_state[idx] = hb;
  y_t[idx] = hb;
  gates_t[zo] = __float2bfloat16(i);
  gates_t[zo + H] = __float2bfloat16(f);
  gates_t[zo + 2 * H] = __float2bfloat16(g);
  gates_t[zo + 3 * H] = __float2bfloat16(o);
}

// dh_in [B,H] fp32: gradient arriving at h_t from later steps; on return it holds the pass-through part of dh_{t-1}
// (the masked rows), to which the GEMM then adds dz_t·W_rec.
__global__ void __launch_bounds__(256)
lstm_cell_bwd_kernel(const bf16* __restrict__ dy_t, float* __restrict__ dh_io, float* __restrict__ dc_state, const bf16* __restrict__ gates_t,
                     const float* __restrict__ c_t, const float* __restrict__ c_prev, const int* __restrict__ lens, int t, int B, int H,
                     bf16* __restrict__ dz_t) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  const size_t zo = (size_t)b * 4 * H + j;
  const bool valid = !lens || t < lens[b];
  if (!valid) {
    // state was copied: gradients pass through, the output (zero) has no gradient
    dz_t[zo] = dz_t[zo + H] = dz_t[zo + 2 * H] = dz_t[zo + 3 * H] = __float2bfloat16(0.f);
    return;
  }
  const float dh = dh_io[idx] + (dy_t ? __bfloat162float(dy_t[idx]) : 0.f);
  const float i = __bfloat162float(gates_t[zo]), f = __bfloat162float(gates_t[zo + H]);
  const float g = __bfloat162float(gates_t[zo + 2 * H]), o = __bfloat162float(gates_t[zo + 3 * H]);
  const float tc = tanhf(c_t[idx]);
  const float dc = dc_state[idx] + dh * o * (1.f - tc * tc);
  dz_t[zo] = __float2bfloat16(dc * g * i * (1.f - i));
  dz_t[zo + H] = __float2bfloat16(dc * c_prev[idx] * f * (1.f - f));
  dz_t[zo + 2 * H] = __float2bfloat16(dc * i * (1.f - g * g));
  dz_t[zo + 3 * H] = __float2bfloat16(dh * tc * o * (1.f - o));
  dc_state[idx] = dc * f;
  dh_io[idx] = 0.f;
}

__global__ void bf16_to_f32_kernel(const bf16* __restrict__ x, float* __restrict__ y, long long n) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __bfloat162float(x[i]);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, bf16* __restrict__ y, long long n) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16(x[i]);
}

}  // namespace

// z_in [T,B,4H] bf16; w_rec [4H,H] bf16; lens [B] or null; h0, c0 [B,H] fp32.
// Outputs: y [T,B,H] bf16, c_all [T,B,H] fp32, gates [T,B,4H] bf16, hprev_all [T,B,H] bf16, h_final / c_final [B,H] fp32 (c_final is also
// the running cell state), scratch: z_rec [B,4H] fp32, h_state [B,H] bf16.
RB_EXPORT int rb200_lstm_fwd(const void* z_in, const void* w_rec, const int* lens, const float* h0, const float* c0, int T, int B, int H, int reverse,
                             void* y, float* c_all, void* gates, void* hprev_all, float* h_final, float* c_final, float* z_rec, void* h_state,
                             int* status, int* n_launch, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return RB_OK;
  if (H % 8) {
    rb_set_error("lstm: hidden size %d must be a multiple of 8", H);
    return RB_ERR_UNSUPPORTED;
  }
  if (rb_lstm_persist_supported(T, B, H)) {
    // z_rec (B*4H floats) is large enough for the two bf16 copies of the hidden state that the CTAs exchange
    if (n_launch) *n_launch = 2;
    return rb_lstm_persist_fwd(z_in, w_rec, lens, h0, c0, T, B, H, reverse, y, c_all, gates, hprev_all, h_final, c_final, z_rec, status, stream);
  }
  const long long bh = (long long)B * H;
  const int grid = (int)((bh + 255) / 256);
  cudaMemcpyAsync(c_final, c0, bh * sizeof(float), cudaMemcpyDeviceToDevice, stream);
  f32_to_bf16_kernel<<<grid, 256, 0, stream>>>(h0, (bf16*)h_state, bh);
  int launches = 2;
  for (int s = 0; s < T; ++s) {
    const int t = reverse ? T - 1 - s : s;
    RbGemm g;
    g.a = h_state; g.b = w_rec; g.c = z_rec; g.m = B; g.n = 4 * H; g.k = H; g.lda = H; g.ldb = H; g.ldc = 4 * H;
    g.a_mn_major = 0; g.b_mn_major = 0; g.out_fp32 = 1; g.status = status;
    int st = rb_gemm(g, stream);
    if (st) return st;
    lstm_cell_fwd_kernel<<<grid, 256, 0, stream>>>(z_rec, (const bf16*)z_in + (size_t)t * B * 4 * H, lens, t, B, H, c_final, (bf16*)h_state,
                                                   (bf16*)y + (size_t)t * bh, c_all + (size_t)t * bh, (bf16*)gates + (size_t)t * B * 4 * H,
                                                   (bf16*)hprev_all + (size_t)t * bh);
    launches += 2;
  }
  int st = rb_check_launch("lstm_fwd");
  if (st) return st;
  // final hidden state in fp32
  bf16_to_f32_kernel<<<grid, 256, 0, stream>>>((const bf16*)h_state, h_final, bh);
  ++launches;
  if (n_launch) *n_launch = launches;
  return rb_check_launch("lstm_fwd_final");
}

// dy [T,B,H] bf16 (may be null), dh_final / dc_final [B,H] fp32 (may be null): incoming gradients. Outputs: dz [T,B,4H] bf16 (gradient of
// z_in and operand of the weight-gradient GEMMs), dw_rec [4H,H] fp32 (accumulated into), dh0 / dc0 [B,H] fp32 (dh0 doubles as the running
// dh buffer, dc0 as the running dc buffer).
RB_EXPORT int rb200_lstm_bwd(const void* dy, const float* dh_final, const float* dc_final, const void* w_rec, const int* lens, const void* gates,
                             const float* c_all, const float* c0, const void* hprev_all, int T, int B, int H, int reverse, void* dz, float* dw_rec,
                             float* dh0, float* dc0, int* status, int* n_launch, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return RB_OK;
  if (rb_lstm_persist_supported(T, B, H)) {
    int st = rb_lstm_persist_bwd(dy, dh_final, dc_final, w_rec, lens, gates, c_all, c0, T, B, H, reverse, dz, dh0, dc0, status, stream);
    if (st) return st;
    int launches = 2;
    if (dw_rec) {
      RbGemm g;
      g.a = dz; g.b = hprev_all; g.c = dw_rec; g.m = 4 * H; g.n = H; g.k = T * B; g.lda = 4 * H; g.ldb = H; g.ldc = H;
      g.a_mn_major = 1; g.b_mn_major = 1; g.out_fp32 = 1; g.accumulate = 2; g.status = status;
      st = rb_gemm(g, stream);
      if (st) return st;
      ++launches;
    }
    if (n_launch) *n_launch = launches;
    return rb_check_launch("lstm_bwd_persist");
  }
  const long long bh = (long long)B * H;
  const int grid = (int)((bh + 255) / 256);
  if (dh_final) cudaMemcpyAsync(dh0, dh_final, bh * sizeof(float), cudaMemcpyDeviceToDevice, stream);
  else cudaMemsetAsync(dh0, 0, bh * sizeof(float), stream);
  if (dc_final) cudaMemcpyAsync(dc0, dc_final, bh * sizeof(float), cudaMemcpyDeviceToDevice, stream);
  else cudaMemsetAsync(dc0, 0, bh * sizeof(float), stream);
  int launches = 2;
  for (int s = T - 1; s >= 0; --s) {
    const int t = reverse ? T - 1 - s : s;           // frame processed at forward step s
    const int t_prev = reverse ? t + 1 : t - 1;      // frame of forward step s - 1
    const float* c_prev = s > 0 ? c_all + (size_t)t_prev * bh : c0;
    lstm_cell_bwd_kernel<<<grid, 256, 0, stream>>>(dy ? (const bf16*)dy + (size_t)t * bh : nullptr, dh0, dc0, (const bf16*)gates + (size_t)t * B * 4 * H,
                                                   c_all + (size_t)t * bh, c_prev, lens, t, B, H, (bf16*)dz + (size_t)t * B * 4 * H);
    // dh_{s-1} = pass-through + dz_t · W_rec   ([B,4H] x [4H,H])
    RbGemm g;
    g.a = (const bf16*)dz + (size_t)t * B * 4 * H; g.b = w_rec; g.c = dh0; g.m = B; g.n = H; g.k = 4 * H; g.lda = 4 * H; g.ldb = H; g.ldc = H;
    g.a_mn_major = 0; g.b_mn_major = 1; g.out_fp32 = 1; g.accumulate = 1; g.status = status;
    int st = rb_gemm(g, stream);
    if (st) return st;
    launches += 2;
  }
  if (dw_rec) {
    // dW_rec[4H,H] += dz^T [4H, T*B] · h_prev [T*B, H]
    RbGemm g;
    g.a = dz; g.b = hprev_all; g.c = dw_rec; g.m = 4 * H; g.n = H; g.k = T * B; g.lda = 4 * H; g.ldb = H; g.ldc = H;
    g.a_mn_major = 1; g.b_mn_major = 1; g.out_fp32 = 1; g.accumulate = 2; g.status = status;
    int st = rb_gemm(g, stream);
    if (st) return st;
    ++launches;
  }
  if (n_launch) *n_launch = launches;
  return rb_check_launch("lstm_bwd");
}
