/*
 * Allocation-free entry point of librb200.so. This has no counterpart in the reference framework.
 *
 * rb200_layer_norm_bwd_noalloc computes the LayerNorm / RMSNorm backward pass (dx, dgamma, dbeta) like
 * rb200_layer_norm_bwd, but takes no scratch buffer from the caller: the per-CTA partial sums of dgamma and dbeta go
 * into a fixed array inside the library (2.3 MiB of device memory per GPU that uses the library, held until the process
 * exits). It is meant for callers that cannot allocate device memory when they call: programs without an allocator of
 * their own, processes whose memory pool already owns the whole device so that cudaMalloc fails, and loops that cannot
 * afford the device-wide synchronisation which cudaMalloc and cudaFree imply. The function itself calls no cudaMalloc,
 * no cudaFree and no library routine that allocates.
 *
 * Limits: n (the normalised row length) must be a positive multiple of 8 and at most
 * rb200_layer_norm_bwd_noalloc_max_n() = 2048; other values are rejected with status 1 and a message in
 * rb200_last_error(). rows >= 1.
 *
 * The first call on a device looks up the device address of the built-in array (cudaGetSymbolAddress); make that first
 * call outside of any stream capture. All calls on one device share the array and it keeps the previous call's
 * contents; nothing in it needs to be cleared between calls. Calls that overlap on the same GPU race on it: issue them
 * on one stream or otherwise serialise them.
 *
 * Inputs and outputs are device pointers owned by the caller:
 *   x, dy   [rows, n]  bf16 (x_bf16 = 1) or fp32 (0)         gamma [n] bf16 (w_bf16 = 1) or fp32
 *   mean, rstd [rows] fp32 as saved by rb200_layer_norm_fwd  dx [rows, n] like x     dgamma, dbeta [n] fp32
 *   rms = 1 for RMSNorm (mean is ignored).
 * Returns 0 on success.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int rb200_layer_norm_bwd_noalloc(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                                 float* dgamma, float* dbeta, long long rows, int n, int x_bf16, int w_bf16, int rms, cudaStream_t stream);
int rb200_layer_norm_bwd_noalloc_max_n(void);
int rb200_layer_norm_bwd_noalloc_parts(void);

#ifdef __cplusplus
}
#endif
