// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (its RMSNorm backward is
// autograd over PyTorch ops, which allocates freely); it exists for this
// library's own C-ABI users.
//
// Who cannot allocate, and why: (1) native host code that drives these kernels
// without PyTorch loaded has no caching allocator to ask, and a raw cudaMalloc /
// cudaFree on the hot path synchronises the whole device, which would stall the
// rollout and weight-push streams that run beside training; (2) a process that has
// handed nearly all of HBM to the KV cache and the flat parameter buffers may find
// that an allocation of a few MB fails at exactly the wrong moment. The regular
// entry point, b200_rmsnorm_bwd, leaves the scratch to its caller; this one brings
// its own.
//
// Same arithmetic, same launch shapes and the same results as b200_rmsnorm_bwd;
// the per-block partial sums of dw live in a fixed array in device global memory
// (static storage of the kernel library, 304 x 8192 floats = 9.5 MiB per device)
// instead of a caller-provided buffer.
//
//  * Limits: H a multiple of 8 and H <= B200_RMSNORM_STATIC_MAX_H (8192); the
//    launch needs at most B200_RMSNORM_STATIC_MAX_BLOCKS (304) blocks, which holds
//    for any T on devices with up to 152 SMs. Beyond either limit the call launches
//    nothing, prints one line to stderr and returns B200_ERR_STATIC_SCRATCH_TOO_SMALL.
//  * Set-up: the first call on each device looks up the device address of the array
//    (with that device current) and keeps it; make that first call before any
//    stream capture begins.
//  * Nothing has to be zeroed: every block overwrites its whole row of partial sums
//    before the column sum reads it. dw is overwritten, or added to when
//    dw_accumulate != 0.
//  * The array is shared by all calls on a device: two calls that overlap in time
//    (different streams or threads, same device) race on it. Order them on one
//    stream or with events.
//  * The call itself performs no cudaMalloc / cudaFree and calls no allocating
//    library routine.
#pragma once
#include <cuda_runtime.h>

#define B200_RMSNORM_STATIC_MAX_H 8192
#define B200_RMSNORM_STATIC_MAX_BLOCKS 304
#define B200_ERR_STATIC_SCRATCH_TOO_SMALL (-120)

#ifdef __cplusplus
extern "C" {
#endif

// dy, x, dx: bf16 [T, H]; w: bf16 [H]; rstd: fp32 [T]; dres: bf16 [T, H] or null; dw: fp32 [H].
// Returns 0, B200_ERR_STATIC_SCRATCH_TOO_SMALL, -100 (H not a multiple of 8) or a negative CUDA error.
int b200_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, float* dw, int dw_accumulate, int T, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
