/* Entry point for callers that must not allocate device memory.
 *
 * This has no counterpart in the reference project; it exists for embedders of this
 * library that are not allowed to call cudaMalloc (or any allocating routine, PyTorch's
 * caching allocator included) at the point where they need an RMSNorm backward: code that
 * runs inside a fixed memory budget handed out up front, plugins living in a host process
 * that owns all device memory, and real-time loops where an allocation could block.
 *
 * ceo_rmsnorm_bwd (ceo_kernels.h) needs a caller-provided fp32 scratch buffer for the
 * per-CTA partial sums of the weight gradient.  ceo_rmsnorm_bwd_noalloc computes exactly
 * the same thing, but keeps that scratch in a file-scope device array inside the library:
 *
 *   - Limit: D <= CEO_NOALLOC_MAX_D (2048) and D % 8 == 0; any number of rows.  A larger D
 *     returns CEO_ERR_NOALLOC_TOO_LARGE (-6) and prints one line to stderr; nothing is
 *     launched.  The array is CEO_NORM_BWD_MAX_BLOCKS x CEO_NOALLOC_MAX_D floats
 *     (about 4.6 MiB) and every GPU that loads the library holds it until the process exits.
 *   - Set-up: the first call on each device resolves the array's device address (with that
 *     device current) and caches it.  Make that first call outside any stream capture.
 *   - Sharing: all calls on a device use the same array, which keeps whatever the previous
 *     call left in it (each call overwrites every element it later reads, so nothing needs
 *     clearing).  Two calls that overlap on the GPU - different streams without an ordering
 *     between them - race on the array; serialise them.
 *   - No allocation: the function calls no cudaMalloc / cudaFree / stream-ordered
 *     allocation and no library routine that could.  Inputs and outputs are the caller's.
 *
 * Arguments and results are those of ceo_rmsnorm_bwd minus `partial_scratch`:
 *   dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x) (+ dres),   dw (+)= sum_rows dy * x * rstd
 */
#ifndef CEO_NOALLOC_H
#define CEO_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CEO_NOALLOC_MAX_D 2048
#define CEO_ERR_NOALLOC_TOO_LARGE (-6)

int ceo_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                            const void* dres, void* dx, float* dw, int dw_accumulate, int rows,
                            int D, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CEO_NOALLOC_H */
