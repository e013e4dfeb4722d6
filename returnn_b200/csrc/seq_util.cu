// Small sequence utilities, each one pass over its output:
//   chunk / unchunk          [T, B, D] <-> [chunk_size, B * n_chunks, D] windows of the time axis (chunk c of sequence b is column
//                            b * n_chunks + c); unchunk averages the frames that overlapping windows share
//   select_by_index          y[t, b] = x[t, b, idx[t, b]] and its gradient
//   sparse_to_dense          W[s0[i, b], b, s1[i, b]] += weight[i, b] from COO entries (i, b)
//   max_argmax_sparse        per (t, b): max and argmax over the COO entries of that frame
//   sparse_ce_softmax_grad   CE[t, b] = - sum_i y[t, b, i] log softmax(z[t, b])[i] with y in COO form, and d/dz = softmax - y
// (reference ops: returnn/native_op.py:2321 Chunking, :2478 UnChunking, :2655 SubtensorBatchedIndex, :2799 SparseToDense,
//  :2880 MaxAndArgmaxSparse, :2988 CrossEntropySoftmaxAndGradientZSparse)
#include <algorithm>
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
chunk_kernel(const float* __restrict__ x, const int* __restrict__ lens, int T, int B, int D, int chunk_size, int chunk_step, int n_chunks,
             float* __restrict__ y, float* __restrict__ y_mask) {
  const long long total = (long long)chunk_size * B * n_chunks * D;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const long long r = i / D;
    const int col = (int)(r % ((long long)B * n_chunks));
    const int ot = (int)(r / ((long long)B * n_chunks));
    const int b = col / n_chunks, c = col % n_chunks;
    const int t = c * chunk_step + ot;
    const bool ok = t < T && t < lens[b];
    y[i] = ok ? x[((size_t)t * B + b) * D + d] : 0.f;
    if (d == 0) y_mask[r] = ok ? 1.f : 0.f;
  }
}

__global__ void __launch_bounds__(256)
unchunk_kernel(const float* __restrict__ y, const float* __restrict__ y_mask, int T, int B, int D, int chunk_size, int chunk_step, int n_chunks,
               float* __restrict__ x, float* __restrict__ x_mask, float* __restrict__ factors) {
  const long long total = (long long)T * B * D;
  const int cols = B * n_chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const long long r = i / D;
    const int b = (int)(r % B), t = (int)(r / B);
    // windows c with c * step <= t < c * step + size
    const int c_hi = min(n_chunks - 1, t / chunk_step);
    const int c_lo = max(0, (t - chunk_size) / chunk_step + ((t - chunk_size) >= 0 ? 1 : 0));
    float acc = 0.f;
    int cnt = 0;
    for (int c = c_lo; c <= c_hi; ++c) {
      const int ot = t - c * chunk_step;
      if (ot < 0 || ot >= chunk_size) continue;
      const size_t rr = (size_t)ot * cols + (size_t)b * n_chunks + c;
      if (y_mask[rr] > 0.1f) {
        acc += y[rr * D + d];
        ++cnt;
      }
    }
    x[i] = cnt ? acc / cnt : 0.f;
    if (d == 0) {
      x_mask[r] = cnt ? 1.f : 0.f;
      factors[r] = cnt ? 1.f / cnt : 1.f;
    }
  }
}

__global__ void __launch_bounds__(256)
select_kernel(const float* __restrict__ x, const int* __restrict__ idx, long long rows, int D, float* __restrict__ y) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
    const int j = idx[r];
    y[r] = (j >= 0 && j < D) ? x[r * D + j] : 0.f;
  }
}

__global__ void __launch_bounds__(256)
select_bwd_kernel(const float* __restrict__ dy, const int* __restrict__ idx, long long rows, int D, float* __restrict__ dx) {
  const long long total = rows * D;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / D;
    dx[i] = ((int)(i - r * D) == idx[r]) ? dy[r] : 0.f;
  }
}

// entries (i, b), i < n_entries: frame s0[i, b], class s1[i, b], value w[i, b], used when mask[i, b] > 0.1
__global__ void __launch_bounds__(256)
sparse_to_dense_kernel(const int* __restrict__ s0, const int* __restrict__ s1, const float* __restrict__ w, const float* __restrict__ mask,
                       int n_entries, int T, int B, int D, float* __restrict__ out) {
  const long long total = (long long)n_entries * B;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    if (mask[i] < 0.1f) continue;
    const int b = (int)(i % B);
    const int t = s0[i], c = s1[i];
    if (t < 0 || t >= T || c < 0 || c >= D) continue;
    atomicAdd(out + ((size_t)t * B + b) * D + c, w[i]);
  }
}

__device__ __forceinline__ unsigned long long pack_val_idx(float s, int e) {  // order-preserving: larger score wins, then smaller index
  unsigned u = __float_as_uint(s);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned)(0x7fffffff - e);
}

__global__ void __launch_bounds__(256)
max_argmax_sparse_kernel(const int* __restrict__ s0, const int* __restrict__ s1, const float* __restrict__ w, const float* __restrict__ mask,
                         int n_entries, int T, int B, unsigned long long* __restrict__ best) {
  const long long total = (long long)n_entries * B;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    if (mask[i] < 0.1f) continue;
    const int b = (int)(i % B);
    const int t = s0[i];
    if (t < 0 || t >= T) continue;
    atomicMax(best + (size_t)t * B + b, pack_val_idx(w[i], s1[i]));
  }
}

__global__ void __launch_bounds__(256)
unpack_max_kernel(const unsigned long long* __restrict__ best, long long n, float* __restrict__ out_max, int* __restrict__ out_arg) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long p = best[i];
    if (p == 0ull) continue;  // no entry for this frame: the caller's initial values stay
    unsigned u = (unsigned)(p >> 32);
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    out_max[i] = __uint_as_float(u);
    out_arg[i] = 0x7fffffff - (int)(p & 0xffffffffu);
  }
}

// one warp per frame (t, b): log-sum-exp of z, softmax into grad; ce and the COO targets are applied by the second kernel
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const float* __restrict__ z, const float* __restrict__ z_mask, long long rows, int D, float* __restrict__ grad,
                    float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const float* zr = z + r * D;
  float* gr = grad + r * D;
  if (z_mask[r] < 0.1f) {
    for (int c = lane; c < D; c += 32) gr[c] = 0.f;
    if (lane == 0) lse[r] = 0.f;
    return;
  }
  float mx = -INFINITY;
  for (int c = lane; c < D; c += 32) mx = fmaxf(mx, zr[c]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int c = lane; c < D; c += 32) sum += __expf(zr[c] - mx);
  sum = warp_sum(sum);
  const float l = mx + __logf(sum);
  for (int c = lane; c < D; c += 32) gr[c] = __expf(zr[c] - l);
  if (lane == 0) lse[r] = l;
}

__global__ void __launch_bounds__(256)
sparse_ce_apply_kernel(const float* __restrict__ z, const float* __restrict__ z_mask, const int* __restrict__ yt, const int* __restrict__ yi,
                       const float* __restrict__ yw, const float* __restrict__ ymask, int n_entries, int T, int B, int D,
                       const float* __restrict__ lse, float* __restrict__ ce, float* __restrict__ grad) {
  const long long total = (long long)n_entries * B;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    if (ymask[i] < 0.1f) continue;
    const int b = (int)(i % B);
    const int t = yt[i], c = yi[i];
    if (t < 0 || t >= T || c < 0 || c >= D) continue;
    const size_t r = (size_t)t * B + b;
    if (z_mask[r] < 0.1f) continue;
    atomicAdd(ce + r, -yw[i] * (z[r * D + c] - lse[r]));
    atomicAdd(grad + r * D + c, -yw[i]);
  }
}

inline int grid_for(long long total) { return (int)std::min<long long>(std::max<long long>((total + 255) / 256, 1), 148LL * 8); }

}  // namespace

RB_EXPORT int rb200_chunk(const float* x, const int* lens, int T, int B, int D, int chunk_size, int chunk_step, int n_chunks, float* y, float* y_mask,
                          cudaStream_t stream) {
  const long long total = (long long)chunk_size * B * n_chunks * D;
  if (total <= 0) return RB_OK;
  chunk_kernel<<<grid_for(total), 256, 0, stream>>>(x, lens, T, B, D, chunk_size, chunk_step, n_chunks, y, y_mask);
  return rb_check_launch("chunk");
}

RB_EXPORT int rb200_unchunk(const float* y, const float* y_mask, int T, int B, int D, int chunk_size, int chunk_step, int n_chunks, float* x,
                            float* x_mask, float* factors, cudaStream_t stream) {
  const long long total = (long long)T * B * D;
  if (total <= 0) return RB_OK;
  unchunk_kernel<<<grid_for(total), 256, 0, stream>>>(y, y_mask, T, B, D, chunk_size, chunk_step, n_chunks, x, x_mask, factors);
  return rb_check_launch("unchunk");
}

RB_EXPORT int rb200_select_by_index(const float* x, const int* idx, long long rows, int D, float* y, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  select_kernel<<<grid_for(rows), 256, 0, stream>>>(x, idx, rows, D, y);
  return rb_check_launch("select_by_index");
}

RB_EXPORT int rb200_select_by_index_bwd(const float* dy, const int* idx, long long rows, int D, float* dx, cudaStream_t stream) {
  if (rows <= 0) return RB_OK;
  select_bwd_kernel<<<grid_for(rows * D), 256, 0, stream>>>(dy, idx, rows, D, dx);
  return rb_check_launch("select_by_index_bwd");
}

RB_EXPORT int rb200_sparse_to_dense(const int* s0, const int* s1, const float* w, const float* mask, int n_entries, int T, int B, int D, float* out,
                                    cudaStream_t stream) {
  if ((long long)n_entries * B <= 0) return RB_OK;
  sparse_to_dense_kernel<<<grid_for((long long)n_entries * B), 256, 0, stream>>>(s0, s1, w, mask, n_entries, T, B, D, out);
  return rb_check_launch("sparse_to_dense");
}

// best: scratch [T * B] of 8 bytes, zero-filled by the caller
RB_EXPORT int rb200_max_argmax_sparse(const int* s0, const int* s1, const float* w, const float* mask, int n_entries, int T, int B,
                                      unsigned long long* best, float* out_max, int* out_arg, cudaStream_t stream) {
  if ((long long)n_entries * B > 0) {
    max_argmax_sparse_kernel<<<grid_for((long long)n_entries * B), 256, 0, stream>>>(s0, s1, w, mask, n_entries, T, B, best);
    int st = rb_check_launch("max_argmax_sparse");
    if (st) return st;
  }
  if ((long long)T * B > 0) unpack_max_kernel<<<grid_for((long long)T * B), 256, 0, stream>>>(best, (long long)T * B, out_max, out_arg);
  return rb_check_launch("max_argmax_sparse (unpack)");
}

// ce [T * B] zero-filled by the caller; lse: scratch [T * B]
RB_EXPORT int rb200_sparse_ce_softmax_grad(const float* z, const float* z_mask, const int* yt, const int* yi, const float* yw, const float* ymask,
                                           int n_entries, int T, int B, int D, float* lse, float* ce, float* grad, cudaStream_t stream) {
  const long long rows = (long long)T * B;
  if (rows <= 0) return RB_OK;
  softmax_rows_kernel<<<(int)((rows + 7) / 8), 256, 0, stream>>>(z, z_mask, rows, D, grad, lse);
  int st = rb_check_launch("sparse_ce softmax");
  if (st) return st;
  if ((long long)n_entries * B > 0)
    sparse_ce_apply_kernel<<<grid_for((long long)n_entries * B), 256, 0, stream>>>(z, z_mask, yt, yi, yw, ymask, n_entries, T, B, D, lse, ce, grad);
  return rb_check_launch("sparse_ce apply");
}
