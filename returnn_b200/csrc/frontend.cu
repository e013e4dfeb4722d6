// Conv2d subsampling frontend of the Conformer (3x3 convolutions over (time, feature) with ReLU, max-pool (1,2) after the first,
// time strides on the later ones; reference: ConformerConvSubsample, returnn/frontend/encoder/conformer.py:89-183) as
// implicit GEMMs on the tcgen05 GEMM: gather kernels build the patch matrices in NHWC order, the GEMM epilogue applies bias + ReLU
// (forward) or the ReLU gradient (backward). Sequence lengths are honoured inside the gathers: frames at or beyond a sequence's
// length read as zero, and the last layer is produced directly in packed-row form (valid frames only).
//
//   conv1 (C_in = 1): direct kernel, fused ReLU + max-pool over feature pairs + time mask        -> [B, T, F/2, C1]
//   conv k >= 2: im2col  [rows, 9*C_in]  x  W [C_out, 9*C_in]^T  (+bias, ReLU)                    -> [rows, C_out]
//   backward data: transposed gather of dY [rows_in, 9*C_out]  x  W' [9*C_out, C_in], epilogue * relu'(saved output)
//   backward weights: patch matrix^T x dY on the split-K GEMM; conv1: direct reduction kernel (recomputes its activations)
#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

// ---- conv1: x [B, T, F] bf16 (one input channel), w [C, 9] fp32 (kt major, kf minor), bias [C] -> y [B, T, F/2, C] bf16
__global__ void __launch_bounds__(256)
conv1_relu_pool_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, const int* __restrict__ lens,
                           int B, int T, int F, int C, bf16* __restrict__ y) {
  extern __shared__ float sw[];  // [C][9] + [C]
  for (int i = threadIdx.x; i < C * 9; i += blockDim.x) sw[i] = w[i];
  for (int i = threadIdx.x; i < C; i += blockDim.x) sw[C * 9 + i] = bias ? bias[i] : 0.f;
  __syncthreads();
  const int Fp = F / 2, G = C / 8;
  const long long total = (long long)B * T * Fp * G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    long long r = i / G;
    const int fp = (int)(r % Fp);
    r /= Fp;
    const int t = (int)(r % T), b = (int)(r / T);
    F8 o;
    const int len = lens[b];
    if (t >= len) {
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = 0.f;
    } else {
      // 3 x 4 input neighbourhood of the feature pair (2fp, 2fp+1)
      float in[3][4];
#pragma unroll
      for (int dt = 0; dt < 3; ++dt) {
        const int tt = t - 1 + dt;
#pragma unroll
        for (int df = 0; df < 4; ++df) {
          const int ff = 2 * fp - 1 + df;
          in[dt][df] = (tt >= 0 && tt < len && ff >= 0 && ff < F) ? __bfloat162float(x[((size_t)b * T + tt) * F + ff]) : 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int c = g * 8 + k;
        float a0 = sw[C * 9 + c], a1 = a0;
#pragma unroll
        for (int dt = 0; dt < 3; ++dt)
#pragma unroll
          for (int df = 0; df < 3; ++df) {
            const float wv = sw[c * 9 + dt * 3 + df];
            a0 += wv * in[dt][df];
            a1 += wv * in[dt][df + 1];
          }
        o.v[k] = fmaxf(fmaxf(a0, a1), 0.f);
      }
    }
    store8(y, i * 8, o, 1);
  }
}

// gradient of conv1's filter and bias: recompute the two pre-pool activations, route dy to the larger one if positive
__global__ void __launch_bounds__(256)
conv1_relu_pool_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, const int* __restrict__ lens,
                           const bf16* __restrict__ dy, int B, int T, int F, int C, float* __restrict__ dw, float* __restrict__ dbias) {
  extern __shared__ float sw[];  // [C][9] + [C] weights, then [C][9] + [C] accumulators
  float* acc = sw + C * 10;
  for (int i = threadIdx.x; i < C * 9; i += blockDim.x) sw[i] = w[i];
  for (int i = threadIdx.x; i < C; i += blockDim.x) sw[C * 9 + i] = bias ? bias[i] : 0.f;
  for (int i = threadIdx.x; i < C * 10; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int Fp = F / 2, G = C / 8;
  // a thread keeps its channel group for all its positions, so its sums stay in registers
  const int g = threadIdx.x % G;
  const long long positions = (long long)B * T * Fp;
  const long long stride = (long long)gridDim.x * (blockDim.x / G);
  float gw[8][9], gb[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    gb[k] = 0.f;
#pragma unroll
    for (int j = 0; j < 9; ++j) gw[k][j] = 0.f;
  }
  for (long long p = (long long)blockIdx.x * (blockDim.x / G) + threadIdx.x / G; p < positions; p += stride) {
    const int fp = (int)(p % Fp);
    const long long r = p / Fp;
    const int t = (int)(r % T), b = (int)(r / T);
    const int len = lens[b];
    if (t >= len) continue;
    float in[3][4];
#pragma unroll
    for (int dt = 0; dt < 3; ++dt) {
      const int tt = t - 1 + dt;
#pragma unroll
      for (int df = 0; df < 4; ++df) {
        const int ff = 2 * fp - 1 + df;
        in[dt][df] = (tt >= 0 && tt < len && ff >= 0 && ff < F) ? __bfloat162float(x[((size_t)b * T + tt) * F + ff]) : 0.f;
      }
    }
    F8 d = load8(dy, (p * G + g) * 8, 1);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = g * 8 + k;
      float a0 = sw[C * 9 + c], a1 = a0;
#pragma unroll
      for (int dt = 0; dt < 3; ++dt)
#pragma unroll
        for (int df = 0; df < 3; ++df) {
          const float wv = sw[c * 9 + dt * 3 + df];
          a0 += wv * in[dt][df];
          a1 += wv * in[dt][df + 1];
        }
      const bool first = a0 >= a1;
      const float m = first ? a0 : a1;
      if (m > 0.f) {
        const float gv = d.v[k];
        gb[k] += gv;
        const int sh = first ? 0 : 1;
#pragma unroll
        for (int dt = 0; dt < 3; ++dt)
#pragma unroll
          for (int df = 0; df < 3; ++df) gw[k][dt * 3 + df] += gv * in[dt][df + sh];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = g * 8 + k;
    atomicAdd(&acc[C * 9 + c], gb[k]);
#pragma unroll
    for (int j = 0; j < 9; ++j) atomicAdd(&acc[c * 9 + j], gw[k][j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < C * 9; i += blockDim.x) atomicAdd(dw + i, acc[i]);
  if (dbias)
    for (int i = threadIdx.x; i < C; i += blockDim.x) atomicAdd(dbias + i, acc[C * 9 + i]);
}

// ---- patch gather (forward): x [B, T, F, C] -> col [rows, 9 * C], K order (kt, kf, c).
// rows = all (b, to, f) of the padded output (row_batch == null, To given), or the valid output frames only (row_batch / row_pos
// [n_frames], rows = n_frames * F). Input frames >= lens_in[b] read as zero.
__global__ void __launch_bounds__(256)
im2col_kernel(const bf16* __restrict__ x, const int* __restrict__ lens_in, int T, int F, int C, int stride_t, int pad_t, int To,
              const int* __restrict__ row_batch, const int* __restrict__ row_pos, long long n_out_frames, bf16* __restrict__ col) {
  const int G = C / 8;
  const long long total = n_out_frames * F * 9 * G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    long long r = i / G;
    const int j = (int)(r % 9);
    r /= 9;
    const int f = (int)(r % F);
    const long long fr = r / F;
    int b, to;
    if (row_batch) {
      b = row_batch[fr];
      to = row_pos[fr];
    } else {
      b = (int)(fr / To);
      to = (int)(fr % To);
    }
    const int tt = to * stride_t - pad_t + j / 3;
    const int ff = f - 1 + j % 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tt >= 0 && tt < lens_in[b] && tt < T && ff >= 0 && ff < F) v = *reinterpret_cast<const uint4*>(x + (((size_t)b * T + tt) * F + ff) * C + g * 8);
    *reinterpret_cast<uint4*>(col + (r * 9 + j) * C + g * 8) = v;
  }
}

// ---- transposed patch gather (backward data): dy [out frames, F, Co] -> colT [B * T * F, 9 * Co], K order (kt, kf, co):
// colT[(b, t, f), (kt, kf, :)] = dy[(b, to, f + 1 - kf), :] with to = (t + pad_t - kt) / stride_t when that division is exact and
// to < lens_out[b]; rows with t >= lens_in[b] are zero. dy is a padded batch [B, To, F, Co] (cu == null) or packed frames (frame index = cu[b] + to).
__global__ void __launch_bounds__(256)
im2col_transposed_kernel(const bf16* __restrict__ dy, const int* __restrict__ lens_out, const int* __restrict__ lens_in, const int* __restrict__ cu,
                         int B, int T, int F, int Co, int stride_t, int pad_t, int To, bf16* __restrict__ col) {
  const int G = Co / 8;
  const long long total = (long long)B * T * F * 9 * G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    long long r = i / G;
    const int j = (int)(r % 9);
    r /= 9;
    const int f = (int)(r % F);
    const long long bt = r / F;
    const int b = (int)(bt / T), t = (int)(bt % T);
    const int num = t + pad_t - j / 3;
    const int fo = f + 1 - j % 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    // input frames at or beyond the sequence's length were read as zero in the forward pass: they get no gradient
    if (t < lens_in[b] && num >= 0 && num % stride_t == 0 && fo >= 0 && fo < F) {
      const int to = num / stride_t;
      if (to < lens_out[b] && to < To) {
        const long long frame = cu ? (long long)cu[b] + to : (long long)b * To + to;
        v = *reinterpret_cast<const uint4*>(dy + (frame * F + fo) * Co + g * 8);
      }
    }
    *reinterpret_cast<uint4*>(col + (r * 9 + j) * Co + g * 8) = v;
  }
}

// ---- patch-gradient gather (backward data, output side): dcol [out frames * F, 9 * Ci] = dy . W holds, for every output position,
// the gradient of its 3x3xCi input patch; the input gradient is the sum over the (at most ceil(3/stride) x 3) patches that contain
// the input position:  dx[(b, t, f), :] = sum_{kt, kf} dcol[(b, to, f + 1 - kf), (kt, kf, :)]  with to = (t + pad_t - kt) / stride_t
// where exact and to < lens_out[b]; zero for t >= lens_in[b]; optionally times relu'(z). A gather: no atomics, and the matrix
// product has out-frames rows (the transposed-patch form above has stride_t times more, most of them zeros).
__global__ void __launch_bounds__(256)
col2im_kernel(const bf16* __restrict__ dcol, const int* __restrict__ lens_out, const int* __restrict__ lens_in, const int* __restrict__ cu, int B,
              int T, int F, int Ci, int stride_t, int pad_t, int To, const bf16* __restrict__ relu_z, bf16* __restrict__ dx) {
  const int G = Ci / 8;
  const long long total = (long long)B * T * F * G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    long long r = i / G;  // (b, t, f)
    const int f = (int)(r % F);
    const long long bt = r / F;
    const int b = (int)(bt / T), t = (int)(bt % T);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (t < lens_in[b]) {
      const int lo = lens_out[b];
#pragma unroll
      for (int kt = 0; kt < 3; ++kt) {
        const int num = t + pad_t - kt;
        if (num < 0 || num % stride_t) continue;
        const int to = num / stride_t;
        if (to >= lo || to >= To) continue;
        const long long frame = cu ? (long long)cu[b] + to : (long long)b * To + to;
#pragma unroll
        for (int kf = 0; kf < 3; ++kf) {
          const int fo = f + 1 - kf;
          if (fo < 0 || fo >= F) continue;
          const uint4 v = *reinterpret_cast<const uint4*>(dcol + ((frame * F + fo) * 9 + kt * 3 + kf) * Ci + g * 8);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 p2 = __bfloat1622float2(h[q]);
            acc[2 * q] += p2.x;
            acc[2 * q + 1] += p2.y;
          }
        }
      }
      if (relu_z) {
        const uint4 z = *reinterpret_cast<const uint4*>(relu_z + r * Ci + g * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&z);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 p2 = __bfloat1622float2(h[q]);
          if (!(p2.x > 0.f)) acc[2 * q] = 0.f;
          if (!(p2.y > 0.f)) acc[2 * q + 1] = 0.f;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<uint4*>(dx + r * Ci + g * 8) = o;
  }
}

int grid_for(long long total) {
  long long g = (total + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

RB_EXPORT int rb200_conv1_relu_pool_fwd(const void* x, const float* w, const float* bias, const int* lens, int B, int T, int F, int C, void* y,
                                        cudaStream_t stream) {
  if (B <= 0 || T <= 0) return RB_OK;
  if (C % 8 || F % 2 || C > 256) {
    rb_set_error("conv1: C=%d must be a multiple of 8 (<= 256) and F=%d even", C, F);
    return RB_ERR_UNSUPPORTED;
  }
  const long long total = (long long)B * T * (F / 2) * (C / 8);
  conv1_relu_pool_fwd_kernel<<<grid_for(total), 256, (size_t)C * 10 * sizeof(float), stream>>>((const bf16*)x, w, bias, lens, B, T, F, C, (bf16*)y);
  return rb_check_launch("conv1_relu_pool_fwd");
}

RB_EXPORT int rb200_conv1_relu_pool_bwd(const void* x, const float* w, const float* bias, const int* lens, const void* dy, int B, int T, int F, int C,
                                        float* dw, float* dbias, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return RB_OK;
  if (C % 8 || F % 2 || C > 256 || 256 % (C / 8)) return RB_ERR_UNSUPPORTED;
  conv1_relu_pool_bwd_kernel<<<148 * 4, 256, (size_t)C * 20 * sizeof(float), stream>>>((const bf16*)x, w, bias, lens, (const bf16*)dy, B, T, F, C, dw,
                                                                                      dbias);
  return rb_check_launch("conv1_relu_pool_bwd");
}

RB_EXPORT int rb200_im2col_3x3(const void* x, const int* lens_in, int T, int F, int C, int stride_t, int pad_t, int To, const int* row_batch,
                               const int* row_pos, long long n_out_frames, void* col, cudaStream_t stream) {
  if (n_out_frames <= 0) return RB_OK;
  if (C % 8) return RB_ERR_UNSUPPORTED;
  im2col_kernel<<<grid_for(n_out_frames * F * 9 * (C / 8)), 256, 0, stream>>>((const bf16*)x, lens_in, T, F, C, stride_t, pad_t, To, row_batch, row_pos,
                                                                               n_out_frames, (bf16*)col);
  return rb_check_launch("im2col_3x3");
}

RB_EXPORT int rb200_im2col_3x3_transposed(const void* dy, const int* lens_out, const int* lens_in, const int* cu, int B, int T, int F, int Co, int stride_t, int pad_t,
                                          int To, void* col, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return RB_OK;
  if (Co % 8) return RB_ERR_UNSUPPORTED;
  im2col_transposed_kernel<<<grid_for((long long)B * T * F * 9 * (Co / 8)), 256, 0, stream>>>((const bf16*)dy, lens_out, lens_in, cu, B, T, F, Co,
                                                                                              stride_t, pad_t, To, (bf16*)col);
  return rb_check_launch("im2col_3x3_transposed");
}

// dx [B, T, F, Ci] from the patch gradients dcol [out frames * F, 9 * Ci] (see col2im_kernel); relu_z (optional) [B, T, F, Ci]
RB_EXPORT int rb200_col2im_3x3(const void* dcol, const int* lens_out, const int* lens_in, const int* cu, int B, int T, int F, int Ci, int stride_t,
                               int pad_t, int To, const void* relu_z, void* dx, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return RB_OK;
  if (Ci % 8) return RB_ERR_UNSUPPORTED;
  col2im_kernel<<<grid_for((long long)B * T * F * (Ci / 8)), 256, 0, stream>>>((const bf16*)dcol, lens_out, lens_in, cu, B, T, F, Ci, stride_t, pad_t,
                                                                                To, (const bf16*)relu_z, (bf16*)dx);
  return rb_check_launch("col2im_3x3");
}
