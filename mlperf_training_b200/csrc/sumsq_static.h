// Sum of squares of a flat gradient buffer through an entry point that never allocates.
//
// This entry point has no counterpart in the reference; it exists for callers of this library
// that must not allocate device memory while they run:
//   * a C or C++ host (a health monitor, a logging thread) that links this library without torch
//     and so has no caching allocator to ask for a scratch tensor;
//   * a training loop that runs close to the memory limit and wants the gradient-norm reduction to
//     be independent of allocator state (no growth, no fragmentation, no implicit synchronisation
//     from a cudaMalloc on a cache miss).
//
// b200_sumsq (the regular entry point) takes its partial-sum scratch from the caller, which in the
// Python package is a fresh torch tensor per call.  b200_sumsq_static keeps the scratch in a
// file-scope __device__ array of B200_SUMSQ_STATIC_SLOTS floats (4 KB per device, part of the
// module image, present on every device that loads the library).
//
// Set-up: the first call on a device (made with that device current) looks the array's address up
// with cudaGetSymbolAddress, checks the return code and caches the pointer for that device; later
// calls only launch.  Make that first call once per device during initialisation, before any
// stream capture begins on that device, because symbol look-up may load the module.
//
// Shared state: every call on a device uses the same array.  Nothing in it has to be zero - each
// slot that the final pass reads was written by the first pass of the same call - but two calls
// that overlap in time on different streams of one device race on it.  Issue all calls for a
// device on one stream, or order the streams with events.
//
// Limit: n <= B200_SUMSQ_STATIC_MAX_ELEMS.  The first pass runs min(4 x SM count,
// B200_SUMSQ_STATIC_SLOTS) CTAs (592 on a 148-SM part) and each slot accumulates ceil(n / CTAs)
// squares in fp32 - at most about 2^22.9 at the largest n - before the fixed-order final reduction,
// which bounds the rounding error; a larger n is rejected with a non-zero return code and a message
// in b200_last_error().
//
// The stream must belong to the device that is current at the call: the scratch pointer is the
// current device's, and a stream of another device is not detected here.
#pragma once

#define B200_SUMSQ_STATIC_SLOTS 1024
#define B200_SUMSQ_STATIC_MAX_ELEMS (1ll << 32)

#ifdef __cplusplus
extern "C" {
#endif

// out[0] = sum(g[i]^2) (accumulate == 0) or out[0] += sum(g[i]^2) (accumulate != 0), fp32, fixed
// reduction order.  g: n elements, bf16 if g_is_bf16 else fp32, on the current device.  out: one
// fp32 on the same device.  stream: a cudaStream_t (0 = default stream).  Returns 0 on success.
__attribute__((visibility("default")))
int b200_sumsq_static(const void* g, long long n, int g_is_bf16, float* out, int accumulate, void* stream);

// Largest n accepted (B200_SUMSQ_STATIC_MAX_ELEMS), for callers that bind by symbol only.
__attribute__((visibility("default")))
long long b200_sumsq_static_max_elems(void);

#ifdef __cplusplus
}
#endif
