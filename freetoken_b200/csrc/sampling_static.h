// ft_sample_static: the sampler for callers that must not allocate.
//
// This entry point has no counterpart in the reference.  It exists for hosts
// that embed the sampling kernel where device memory cannot be obtained at call
// time: code running inside a fixed memory budget handed out at start-up, code
// called from a context in which cudaMalloc is forbidden (for instance while
// another component owns the allocator, or inside a latency-critical loop that
// must never take the allocator's lock), and plain C callers that have no
// PyTorch caching allocator to lean on.  ft_sample() needs the caller to bring
// a scratch buffer of rows * vocab floats for the un-normalised probabilities;
// ft_sample_static() brings its own: a fixed array inside the library.
//
// What to know before using it:
//  * The scratch is FT_SAMPLE_STATIC_FLOATS floats (4 MiB).  Every GPU on which
//    the library is loaded keeps that much memory until the process exits.
//  * rows * vocab must not exceed FT_SAMPLE_STATIC_FLOATS; a larger request is
//    refused with FT_ERR_STATIC_TOO_LARGE (-103) and nothing is launched.
//  * The first call on each device looks up the array's device address (with
//    that device current).  Make that first call outside of any stream capture.
//  * All calls share the one array and it keeps whatever the last call left.
//    Nothing in it has to start at zero: the kernel writes every value it later
//    reads.  Two calls whose kernels overlap on the GPU (different streams, no
//    ordering between them) would overwrite each other's probabilities: order
//    them on one stream or with events.
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
//
// Arguments are those of ft_sample() without the scratch pointer: float32
// logits [rows, vocab]; per-row temperature (<= 0: argmax), top_k (<= 0 or
// >= vocab: off), top_p (>= 1: off) and uniform number in [0,1); any of
// temperature / top_k / top_p may be null (all rows greedy / filter off);
// out receives int32 [rows].  Returns 0, a negative FT_ERR_* code, or a
// positive cudaError_t.
#pragma once

#include <cuda_runtime.h>

#define FT_SAMPLE_STATIC_FLOATS (1 << 20)
#define FT_ERR_STATIC_TOO_LARGE -103

#ifdef __cplusplus
extern "C" {
#endif

int ft_sample_static(const float* logits, const float* temperature, const int* top_k,
                     const float* top_p, const float* uniform, int* out, int rows, int vocab,
                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
