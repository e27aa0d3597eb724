/* pkv_sample_static_scratch: token sampling for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for users of this
 * library only.
 *
 * Who it is for. pkv_sample (sampling.cu) needs a work area of n_rows * vocab floats in device
 * memory and leaves it to the caller to provide one. Some callers cannot: a plugin that runs
 * inside another program's stream callback or under an allocator it does not own, a host
 * process whose memory pool is frozen once serving starts, a bare C program that links this
 * library without a CUDA allocator of its own. For them this function does the same sampling
 * with a work area that is part of the library image: a file-scope device array of
 * PKV_SAMPLE_STATIC_FLOATS floats (4 MiB). Every GPU that loads the library holds those 4 MiB
 * until the process exits, whether or not this function is ever called.
 *
 * What it does. Exactly what pkv_sample does (greedy below `greedy_below`, else temperature and
 * nucleus sampling with one uniform number per row; see sampling.cu), on the caller's inputs
 * and into the caller's output. It calls no cudaMalloc, no cudaFree and no allocating library
 * routine.
 *
 * Limits and rules.
 *  - n_rows * vocab must not exceed PKV_SAMPLE_STATIC_FLOATS; a larger request is refused with
 *    PKV_SAMPLE_STATIC_TOO_LARGE (-5) and nothing is launched.
 *  - The addresses are kept for device indices 0 to 63; on a device with a higher index the
 *    call is refused with PKV_SAMPLE_STATIC_DEVICE_INDEX (-6).
 *  - The first call on each device looks up the device address of the work area
 *    (cudaGetSymbolAddress, with that device current) and keeps it. Make that first call
 *    outside of any stream capture.
 *  - All calls share the one work area and it keeps what the last call left there. Nothing in
 *    it has to start at zero: every value a call reads was written by that call first. Two calls
 *    that overlap on the GPU (different streams, no ordering between them) race on it; order
 *    them, or use pkv_sample with work areas of your own.
 *
 * Returns 0 on success, a negative code for a refused argument, a positive cudaError_t for a
 * failed set-up or launch. All pointers are device pointers; `stream` is a cudaStream_t.
 */
#ifndef PKV_SAMPLING_NOALLOC_H
#define PKV_SAMPLING_NOALLOC_H

#include <stdint.h>

#define PKV_SAMPLE_STATIC_FLOATS (1 << 20)
#define PKV_SAMPLE_STATIC_TOO_LARGE (-5)
#define PKV_SAMPLE_STATIC_DEVICE_INDEX (-6)

#ifdef __cplusplus
extern "C" {
#endif

int pkv_sample_static_scratch(const float* logits, long long row_stride, const float* temperature,
                              const float* top_p, const double* uniform, int32_t* out, int n_rows, int vocab,
                              float greedy_below, void* stream);

#ifdef __cplusplus
}
#endif

#endif
