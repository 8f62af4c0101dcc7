// Allocation-free sampling entry point.
//
// This entry point has no counterpart in the reference.  It exists for callers that are not
// allowed to allocate device memory at the moment they need to sample: code running where a
// cudaMalloc is unacceptable (a serving loop with a fixed memory plan, a host thread that must not
// take the allocator lock, a foreign runtime that embeds this library and owns all device memory
// itself, so it cannot hand the library a scratch buffer it does not have).  The regular sampler,
// b200_sample_topk, needs a caller-provided scratch buffer of T * V floats; this variant keeps that
// scratch inside the library instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest T * V the built-in scratch holds: 2,097,152 floats = 8 MiB.  Every GPU that loads this
// library carries those 8 MiB from load until the process exits, whether or not this is called.
#define B200_SAMPLE_NOALLOC_MAX_ELEMS (1u << 21)

// Return codes besides 0 (success) and positive cudaError_t values.
#define B200_NOALLOC_ERR_TOO_LARGE (-1)   // T * V exceeds B200_SAMPLE_NOALLOC_MAX_ELEMS
#define B200_NOALLOC_ERR_BAD_ARG (-2)     // T < 1, V < 1, top_k outside 1..64, or top_k > V

// Temperature / top-k / top-p sampling of one token per row of `logits` ([T][V] fp32, device
// memory), exactly as b200_sample_topk does, but with the T * V floats of working space taken from
// an array compiled into the library.  The caller still owns and passes every input and output:
// `u` ([T] uniform random numbers in [0,1)) and `out_id` ([T] int32) are device pointers.
//
// * A row without a single finite logit (all NaN or -inf) yields token id 0; fewer than top_k finite
//   entries means the candidates are the finite ones only.
// * Calls no cudaMalloc, cudaFree or any other allocating routine.
// * T * V larger than B200_SAMPLE_NOALLOC_MAX_ELEMS is refused with B200_NOALLOC_ERR_TOO_LARGE
//   (and one line on stderr); nothing is launched.
// * The first call on each device looks up the device address of the built-in array (with that
//   device current).  Make that first call outside any CUDA stream capture.
// * All calls on a device share the one array.  It keeps whatever the previous call left in it;
//   the kernel overwrites the part it uses before reading it, so nothing needs clearing between
//   calls.  Two calls whose kernels overlap on the GPU (different streams, no ordering between
//   them) race on the array and may both return wrong tokens: order them.
int b200_sample_topk_noalloc(const float* logits, int T, int V, float temperature, int top_k, float top_p,
                             const float* u, int* out_id, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
