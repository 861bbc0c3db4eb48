// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference framework; it exists for hosts that drive
// this library under a fixed device-memory budget.
//
// Who needs it: the regular backward (msrl_rmsnorm_bwd) expects the caller to bring a scratch
// buffer for the partial weight-gradient sums, which in practice means "allocate one".  Some
// callers cannot:
//   * a co-located RL worker after it has handed all remaining HBM to the rollout KV cache --
//     an allocation at that point fails or forces the cache to shrink;
//   * a plain C/C++ host that links this library without a tensor framework and owns only the
//     input and output buffers it was given;
//   * latency-critical sections where a device allocation (which may synchronise the device)
//     is not acceptable.
// For them the scratch lives inside the library: a file-scope device array of
// MSRL_RMSNORM_NOALLOC_SCRATCH_BYTES (4 MiB) that every GPU which loads the library keeps
// reserved until the process exits.
//
// Limits: hidden size H must be a multiple of 8 and at most MSRL_RMSNORM_NOALLOC_MAX_H; any
// number of rows.  Larger H is rejected with cudaErrorInvalidValue and a message on stderr;
// nothing is launched in that case.
//
// Set-up: the first call on each device looks up the address of the library's scratch array for
// that device (with that device current).  Make this first call during initialisation, before
// any stream capture is started on the device.
//
// Sharing: all calls on one device use the same scratch array and it keeps whatever the last
// call left in it.  Every call overwrites the part it reads before reading it, so nothing has to
// be cleared between calls -- but two calls whose kernels overlap in time on one GPU (different
// streams, different host threads) race on the scratch and corrupt each other's weight gradient.
// Serialise them on one stream or with events.
//
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define MSRL_RMSNORM_NOALLOC_MAX_H 8192
#define MSRL_RMSNORM_NOALLOC_BLOCKS 128
#define MSRL_RMSNORM_NOALLOC_SCRATCH_BYTES (MSRL_RMSNORM_NOALLOC_BLOCKS * MSRL_RMSNORM_NOALLOC_MAX_H * 4)

#ifdef __cplusplus
extern "C" {
#endif

// dx[rows, H] = d loss / d x of y = x * rsqrt(mean(x^2) + eps) * w   (+ dres when dres != NULL)
// dw (+)= sum over rows of dy * x * rstd, written to dw_f32 and/or dw_bf16 (either may be NULL);
// accumulate != 0 adds to the existing contents.  All matrices are contiguous bf16 [rows, H];
// rstd is the fp32 [rows] vector produced by the forward.  dy, x, w, dx (and dres when given) must
// be 16-byte aligned; a NULL or misaligned one is refused with cudaErrorInvalidValue before
// anything is launched.  With both dw outputs NULL only dx is computed.  Returns a cudaError_t as int.
int msrl_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                             const void* dres, void* dx, float* dw_f32, void* dw_bf16, int accumulate,
                             long long rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
