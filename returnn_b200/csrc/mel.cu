// Log-mel filterbank features from raw audio in one kernel: framing, Hann window, DFT (zero-padded to n_fft), power spectrum,
// mel filterbank, log. fp32 throughout (the reference upcasts bf16 audio to fp32 for the STFT, returnn/torch/frontend/_backend.py:2695-2711;
// math of returnn/frontend/audio/mel.py:163-208). One CTA computes kFrames consecutive frames of one recording: the windowed
// frames and a cos / sin table live in shared memory, every thread owns one frequency bin for all frames, then the mel
// projection runs from the power spectrum in shared memory.
#include <algorithm>
#include <cuda_fp16.h>
#include "common.cuh"

namespace {

constexpr int kFrames = 8;
constexpr int kMaxFft = 1024;
constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
log_mel_kernel(const float* __restrict__ audio, const int* __restrict__ lens, long long row_pitch, int n_frames_max, int window, int step, int n_fft,
               const float* __restrict__ win, const float* __restrict__ fbank, int n_mel, float log_scale, float eps, float* __restrict__ out) {
  extern __shared__ float sh[];
  float* sx = sh;                          // [kFrames][window]
  float* scos = sx + kFrames * window;     // [n_fft]
  float* ssin = scos + n_fft;              // [n_fft]
  float* spow = ssin + n_fft;              // [kFrames][n_bins]
  const int n_bins = n_fft / 2 + 1;
  const int row = blockIdx.y;
  const int f0 = blockIdx.x * kFrames;
  const int len = lens ? lens[row] : (int)row_pitch;
  const int n_frames = len >= window ? (len - window) / step + 1 : 0;
  if (f0 >= n_frames_max) return;
  const float* a = audio + (size_t)row * row_pitch;
  for (int i = threadIdx.x; i < kFrames * window; i += kThreads) {
    const int f = i / window, n = i - f * window;
    const int fr = f0 + f;
    sx[i] = fr < n_frames ? a[(size_t)fr * step + n] * win[n] : 0.f;
  }
  for (int i = threadIdx.x; i < n_fft; i += kThreads) {
    float s, c;
    sincospif(2.0f * (float)i / (float)n_fft, &s, &c);
    scos[i] = c;
    ssin[i] = s;
  }
  __syncthreads();
  const int mask = n_fft - 1;
  for (int k = threadIdx.x; k < n_bins; k += kThreads) {
    float re[kFrames], im[kFrames];
#pragma unroll
    for (int f = 0; f < kFrames; ++f) re[f] = im[f] = 0.f;
    int idx = 0;
    for (int n = 0; n < window; ++n) {
      const float c = scos[idx], s = ssin[idx];
#pragma unroll
      for (int f = 0; f < kFrames; ++f) {
        const float x = sx[f * window + n];
        re[f] += x * c;
        im[f] -= x * s;
      }
      idx = (idx + k) & mask;
    }
#pragma unroll
    for (int f = 0; f < kFrames; ++f) spow[f * n_bins + k] = re[f] * re[f] + im[f] * im[f];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kFrames * n_mel; i += kThreads) {
    const int f = i / n_mel, m = i - f * n_mel;
    const int fr = f0 + f;
    if (fr >= n_frames_max) continue;
    float acc = 0.f;
    const float* p = spow + f * n_bins;
    for (int k = 0; k < n_bins; ++k) acc += p[k] * fbank[(size_t)k * n_mel + m];
    const float v = fr < n_frames ? __logf(fmaxf(acc, eps)) * log_scale : 0.f;
    out[((size_t)row * n_frames_max + fr) * n_mel + m] = v;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The tensor-core form: the DFT of all frames is ONE matrix product, frames [rows * slots, window] x table [window, n_fft], on the
// tcgen05 GEMM. The frames are never materialised: the A operand is a strided view of the audio (row pitch = step samples, so
// consecutive rows overlap by window - step samples), which a TMA tensor map expresses directly. fp32 audio and table are split into
// fp16 high and low parts and three products (hi*hi + hi*lo + lo*hi) accumulate in fp32, which keeps 22 mantissa bits per factor
// (bf16 parts would keep 16: an error floor 96 dB under a frame's strongest component, audible in the weakest mel bands).
// Audio is expected within fp16's range (|x| < 65504; samples scaled to [-1, 1] or raw 16-bit PCM values both are).
// The two kernels here are the ends of that pipeline: the split of the audio, and power spectrum -> mel -> log.

// audio [rows, T] fp32 -> hi, lo [rows * Tp + tail] fp16 with audio[r][c] at r * Tp + c, zeros elsewhere (Tp = slots * step)
__global__ void __launch_bounds__(256)
split_hi_lo_kernel(const float* __restrict__ audio, int rows, long long T, long long Tp, long long total, __half* __restrict__ hi,
                   __half* __restrict__ lo) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / Tp, c = i - r * Tp;
    float x = 0.f;
    if (r < rows && c < T) x = audio[r * T + c];
    const __half h = __float2half_rn(x);
    hi[i] = h;
    lo[i] = __float2half_rn(x - __half2float(h));
  }
}

// spec [rows * slots, ld] fp32: column 2j = Re X_j, 2j + 1 = Im X_j for 0 < j < n_fft / 2; column 0 = X_0 and column 1 = X_{n_fft/2}
// (both real). One warp per frame: power spectrum into shared memory, then every lane sums the bins of its mel filters, which are
// contiguous ranges [fb_start[m], fb_start[m] + fb_len[m]) of the filterbank matrix fbank [n_bins, n_mel].
constexpr int kMelWarps = 8;

__global__ void __launch_bounds__(kMelWarps * 32)
mel_from_spectrum_kernel(const float* __restrict__ spec, int ld, int slots, int n_frames_max, const int* __restrict__ lens, long long T, int window,
                         int step, int n_fft, const float* __restrict__ fbank, const int* __restrict__ fb_start, const int* __restrict__ fb_len,
                         int n_mel, float log_scale, float eps, float* __restrict__ out) {
  extern __shared__ float spow[];  // [kMelWarps][n_bins]
  const int n_bins = n_fft / 2 + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int fr = blockIdx.x * kMelWarps + warp;
  if (fr >= n_frames_max) return;
  const long long len = lens ? (long long)lens[row] : T;
  const int n_frames = len >= window ? (int)((len - window) / step + 1) : 0;
  float* o = out + ((size_t)row * n_frames_max + fr) * n_mel;
  if (fr >= n_frames) {
    for (int m = lane; m < n_mel; m += 32) o[m] = 0.f;
    return;
  }
  const float2* sp = reinterpret_cast<const float2*>(spec + ((size_t)row * slots + fr) * ld);
  float* pw = spow + warp * n_bins;
  for (int j = lane; j < n_fft / 2; j += 32) {
    const float2 v = sp[j];
    if (j == 0) {
      pw[0] = v.x * v.x;
      pw[n_fft / 2] = v.y * v.y;
    } else {
      pw[j] = v.x * v.x + v.y * v.y;
    }
  }
  __syncwarp();
  for (int m = lane; m < n_mel; m += 32) {
    const int k0 = fb_start[m], n = fb_len[m];
    float acc = 0.f;
    for (int k = k0; k < k0 + n; ++k) acc += pw[k] * fbank[(size_t)k * n_mel + m];
    o[m] = __logf(fmaxf(acc, eps)) * log_scale;
  }
}

}  // namespace

RB_EXPORT int rb200_split_hi_lo_fp16(const float* audio, int rows, long long T, long long Tp, long long total, void* hi, void* lo, cudaStream_t stream) {
  if (total <= 0) return RB_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 16);
  split_hi_lo_kernel<<<blocks, 256, 0, stream>>>(audio, rows, T, Tp, total, reinterpret_cast<__half*>(hi), reinterpret_cast<__half*>(lo));
  return rb_check_launch("split_hi_lo");
}

RB_EXPORT int rb200_mel_from_spectrum(const float* spec, int ld, int rows, int slots, int n_frames_max, const int* lens, long long T, int window, int step,
                                      int n_fft, const float* fbank, const int* fb_start, const int* fb_len, int n_mel, float log_scale, float eps,
                                      float* out, cudaStream_t stream) {
  if (rows <= 0 || n_frames_max <= 0) return RB_OK;
  if ((ld % 2) || n_fft < 2 || (reinterpret_cast<uintptr_t>(spec) & 7)) {
    rb_set_error("mel_from_spectrum: ld=%d must be even and the spectrum 8-byte aligned", ld);
    return RB_ERR_ARG;
  }
  const size_t smem = (size_t)kMelWarps * (n_fft / 2 + 1) * sizeof(float);
  if (smem > 48 * 1024) {
    rb_set_error("mel_from_spectrum: n_fft=%d too large", n_fft);
    return RB_ERR_UNSUPPORTED;
  }
  dim3 grid((n_frames_max + kMelWarps - 1) / kMelWarps, rows);
  mel_from_spectrum_kernel<<<grid, kMelWarps * 32, smem, stream>>>(spec, ld, slots, n_frames_max, lens, T, window, step, n_fft, fbank, fb_start, fb_len,
                                                                 n_mel, log_scale, eps, out);
  return rb_check_launch("mel_from_spectrum");
}

// audio [rows, row_pitch] fp32; lens [rows] (samples; null: all rows full); win [window] window function; fbank [n_fft/2+1, n_mel];
// out [rows, n_frames_max, n_mel] with n_frames_max = (row_pitch - window) / step + 1; frames past a row's length are written as 0.
// n_fft must be a power of two <= 1024.
RB_EXPORT int rb200_log_mel(const float* audio, const int* lens, int rows, long long row_pitch, int window, int step, int n_fft, const float* win,
                            const float* fbank, int n_mel, float log_scale, float eps, float* out, cudaStream_t stream) {
  if (rows <= 0 || row_pitch < window) return RB_OK;
  if (n_fft > kMaxFft || (n_fft & (n_fft - 1)) || window > n_fft || n_mel < 1) {
    rb_set_error("log_mel: n_fft=%d must be a power of two <= %d and >= window=%d", n_fft, kMaxFft, window);
    return RB_ERR_UNSUPPORTED;
  }
  const int n_frames_max = (int)((row_pitch - window) / step + 1);
  const size_t smem = ((size_t)kFrames * window + 2 * n_fft + (size_t)kFrames * (n_fft / 2 + 1)) * sizeof(float);
  static size_t attr = 0;
  if (smem > 48 * 1024 && smem > attr) {
    cudaFuncSetAttribute(log_mel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr = smem;
  }
  dim3 grid((n_frames_max + kFrames - 1) / kFrames, rows);
  log_mel_kernel<<<grid, kThreads, smem, stream>>>(audio, lens, row_pitch, n_frames_max, window, step, n_fft, win, fbank, n_mel, log_scale, eps, out);
  return rb_check_launch("log_mel");
}
