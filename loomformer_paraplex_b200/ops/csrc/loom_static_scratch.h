// Entry points that never allocate.  This header has no counterpart in the reference project.
//
// loom_grad_norm_static computes exactly what loom_grad_norm (loom_c_api.h) computes -- the global L2 norm of a
// flat fp32 gradient buffer, the clip coefficient for `max_norm`, and a finite flag -- but takes no scratch
// pointer from the caller.  Its per-block partial sums live in a fixed array compiled into the library's device
// image, so the call performs no cudaMalloc / cudaFree and calls into no allocating library (not the torch
// caching allocator either).
//
// Who needs this: a host program that links this library without torch and owns no device allocator; a
// recovery path that runs after an out-of-memory error, when asking the driver for more memory would fail
// again; a serving process that has handed every free byte to its KV pool up front; and any path that must
// not stall on the device-wide synchronisation that cudaMalloc and cudaFree imply.
//
// Limits and rules:
//   * nparts (number of partial sums == thread blocks of the first kernel) must be in [1, LOOM_STATIC_PARTS_MAX];
//     n must be a multiple of 4 and `grads` 16-byte aligned (the kernel reads float4).  Anything else is refused
//     with a negative code; loom_static_strerror() turns a code into text.
//   * The first call on each device looks up the address of the built-in array (cudaGetSymbolAddress) with that
//     device current.  Make that first call during start-up, before any stream capture begins.
//   * Every call on a device shares the one array.  Nothing in it has to start at zero: each call overwrites
//     the nparts entries it later reads.  For the same reason two calls that overlap in time on one device
//     (different streams, or different host threads) race on the array and give wrong norms -- keep calls on
//     one device ordered on a single stream.
//   * stats must point to at least 3 floats of device memory: [0] norm, [1] clip coefficient, [2] finite (1/0).
//     atom_out may be null; when given, its first 3 floats are cleared as loom_grad_norm does.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LOOM_STATIC_PARTS_MAX 1024        // 4 KB of device memory per loaded library image

#define LOOM_STATIC_OK 0
#define LOOM_STATIC_E_PARTS (-101)        // nparts outside [1, LOOM_STATIC_PARTS_MAX]
#define LOOM_STATIC_E_SHAPE (-102)        // n not a positive multiple of 4, or grads not 16-byte aligned
#define LOOM_STATIC_E_NULL (-103)         // grads or stats is null
#define LOOM_STATIC_E_SYMBOL (-104)       // the built-in array's address could not be obtained on this device
#define LOOM_STATIC_E_DEVICE (-105)       // device ordinal beyond the table of cached addresses (64)

int loom_grad_norm_static(const float* grads, long long n, float max_norm, int nparts, float* stats,
                          float* atom_out, cudaStream_t stream);
const char* loom_static_strerror(int code);

#ifdef __cplusplus
}
#endif
