// Column sum without any allocation. This entry point has no counterpart in the
// reference; it exists for callers that are not allowed to allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a region that
// a framework's caching allocator does not own (a plugin callback that must not touch
// the allocator, a hook invoked while another allocator holds its lock), or a process
// whose memory budget was fixed at start-up. cocclkColSum (train_api.h) asks such a
// caller for a scratch buffer; this variant keeps its scratch in a fixed array that is
// part of the library image, so the caller passes only its input and output.
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns the built-in scratch can serve (any number of rows).
#define COCCLK_NOALLOC_MAX_COLS 16384
// Device indices the per-device address cache covers.
#define COCCLK_NOALLOC_MAX_DEVICES 64

// out[n] (+)= sum over m of x[m][n], x is a row-major bf16 matrix [M, N], out is fp32 [N].
//
//  * Allocates nothing: no cudaMalloc/cudaFree, no allocating library call. Scratch is a
//    4 MiB __device__ array (64 partial rows x COCCLK_NOALLOC_MAX_COLS floats) that every
//    GPU which loads this library holds until the process exits.
//  * N must be a multiple of 8 and at most COCCLK_NOALLOC_MAX_COLS; larger N is refused
//    with COCCLK_NOALLOC_TOO_LARGE and a message retrievable by cocclkNoAllocLastError().
//  * The first call on each device looks up the device address of the scratch array
//    (cudaGetSymbolAddress, with that device current) and caches it. Make that first
//    call before starting any stream capture on that device. The cache has one slot per
//    device index 0..COCCLK_NOALLOC_MAX_DEVICES-1; a call with a higher index current is
//    refused with COCCLK_NOALLOC_BAD_SHAPE and a message (nothing is launched).
//  * All calls on a device share the one scratch array, which keeps whatever the last
//    call left in it. Nothing in it needs to start at zero (every partial sum that is
//    read is written first by the same call), but two calls that overlap on the GPU
//    (different streams, no ordering between them) race on it: serialise them.
//
// Returns 0, a cudaError_t, or one of the negative codes below.
#define COCCLK_NOALLOC_BAD_SHAPE (-1)
#define COCCLK_NOALLOC_TOO_LARGE (-2)
int cocclkColSumNoAlloc(const void* x, float* out, int accumulate, int M, int N, cudaStream_t stream);

// Message of the last failure of cocclkColSumNoAlloc on the calling thread ("" if none).
const char* cocclkNoAllocLastError(void);

#ifdef __cplusplus
}
#endif
