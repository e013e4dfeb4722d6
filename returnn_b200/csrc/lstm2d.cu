// Cell kernels of the two-dimensional LSTM (one direction, scanning from the top-left corner). All cells of an anti-diagonal
// t + s = d are independent, so one launch handles the R = (cells on the diagonal) x (batch) rows of a diagonal.
//   i, f, l, o = sigmoid(z[0..3]);  g = tanh(z[4]);  c = (i g + f l c_up + f (1 - l) c_left) m;  h = o tanh(c) m
// "up" is the cell at (t - 1, s), "left" the one at (t, s - 1); l ("lambda") mixes the two predecessor states; m is 1 inside the
// (height x width) extent of the batch entry and 0 outside. fp32 throughout.
// (cell math of returnn/native_op.py:1735-1790, the forward kernel of its TwoDLSTM op, and :1890-1990, its backward kernel)
#include <algorithm>
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

// z [R, 5n]: pre-activations in, activated gates (i, f, l, o, g) out
__global__ void __launch_bounds__(256)
lstm2d_cell_fwd_kernel(float* __restrict__ z, const float* __restrict__ c_up, const float* __restrict__ c_left, const float* __restrict__ mask,
                       float* __restrict__ c, float* __restrict__ h, long long total, int n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / n;
    const int j = (int)(i - r * n);
    float* zr = z + r * 5 * n;
    const float ig = sigm(zr[j]), fg = sigm(zr[n + j]), lg = sigm(zr[2 * n + j]), og = sigm(zr[3 * n + j]), g = tanhf(zr[4 * n + j]);
    const float m = mask[r];
    const float cc = (ig * g + fg * lg * c_up[i] + fg * (1.f - lg) * c_left[i]) * m;
    zr[j] = ig;
    zr[n + j] = fg;
    zr[2 * n + j] = lg;
    zr[3 * n + j] = og;
    zr[4 * n + j] = g;
    c[i] = cc;
    h[i] = og * tanhf(cc) * m;
  }
}

// gates [R, 5n] (activated); dh, dc_in [R, n]: gradient w.r.t. h and the part of dc that arrives from the two successor cells;
// dz [R, 5n] gradient w.r.t. the pre-activations; dc_up, dc_left [R, n] what flows on into the predecessor cell states
__global__ void __launch_bounds__(256)
lstm2d_cell_bwd_kernel(const float* __restrict__ gates, const float* __restrict__ c, const float* __restrict__ c_up, const float* __restrict__ c_left,
                       const float* __restrict__ mask, const float* __restrict__ dh, const float* __restrict__ dc_in, float* __restrict__ dz,
                       float* __restrict__ dc_up, float* __restrict__ dc_left, long long total, int n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / n;
    const int j = (int)(i - r * n);
    const float* gr = gates + r * 5 * n;
    float* dzr = dz + r * 5 * n;
    const float ig = gr[j], fg = gr[n + j], lg = gr[2 * n + j], og = gr[3 * n + j], g = gr[4 * n + j];
    const float m = mask[r];
    const float tc = tanhf(c[i]);
    const float dhv = dh[i] * m;
    const float dc = (dhv * og * (1.f - tc * tc) + dc_in[i]) * m;
    const float cu = c_up[i], cl = c_left[i];
    dzr[j] = dc * g * ig * (1.f - ig);
    dzr[n + j] = dc * (lg * cu + (1.f - lg) * cl) * fg * (1.f - fg);
    dzr[2 * n + j] = dc * fg * (cu - cl) * lg * (1.f - lg);
    dzr[3 * n + j] = dhv * tc * og * (1.f - og);
    dzr[4 * n + j] = dc * ig * (1.f - g * g);
    dc_up[i] = dc * fg * lg;
    dc_left[i] = dc * fg * (1.f - lg);
  }
}

}  // namespace

RB_EXPORT int rb200_lstm2d_cell_fwd(float* z, const float* c_up, const float* c_left, const float* mask, float* c, float* h, long long rows, int n,
                                    cudaStream_t stream) {
  const long long total = rows * n;
  if (total <= 0) return RB_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  lstm2d_cell_fwd_kernel<<<blocks, 256, 0, stream>>>(z, c_up, c_left, mask, c, h, total, n);
  return rb_check_launch("lstm2d_cell_fwd");
}

RB_EXPORT int rb200_lstm2d_cell_bwd(const float* gates, const float* c, const float* c_up, const float* c_left, const float* mask, const float* dh,
                                    const float* dc_in, float* dz, float* dc_up, float* dc_left, long long rows, int n, cudaStream_t stream) {
  const long long total = rows * n;
  if (total <= 0) return RB_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  lstm2d_cell_bwd_kernel<<<blocks, 256, 0, stream>>>(gates, c, c_up, c_left, mask, dh, dc_in, dz, dc_up, dc_left, total, n);
  return rb_check_launch("lstm2d_cell_bwd");
}
