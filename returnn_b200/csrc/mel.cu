// Log-mel filterbank features from raw audio in one kernel: framing, Hann window, DFT (zero-padded to n_fft), power spectrum,
// mel filterbank, log. fp32 throughout (the reference upcasts bf16 audio to fp32 for the STFT, returnn/torch/frontend/_backend.py:2695-2711;
// math of returnn/frontend/audio/mel.py:163-208). One CTA computes kFrames consecutive frames of one recording: the windowed
// frames and a cos / sin table live in shared memory, every thread owns one frequency bin for all frames, then the mel
// projection runs from the power spectrum in shared memory.
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

}  // namespace

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
