/* An entry point for callers that cannot allocate device memory.
 *
 * This has no counterpart in the reference: it exists for programs that embed
 * the kernel library in a place where cudaMalloc is off limits.  Examples: a
 * plugin that runs inside someone else's serving process under a fixed memory
 * budget, a real-time loop that must not take the allocator's locks or its
 * implicit device synchronisation, a process whose memory pool was handed out
 * completely at start-up.  Such a caller still owns its inputs and outputs; what
 * it cannot provide is the scratch space that the split-K matrix product needs
 * for its partial sums.
 *
 * srlm_gemm_tn_tcgen05_static computes C[M,N] = X[M,K] . W[N,K]^T (bfloat16
 * operands, float32 accumulation) exactly like srlm_gemm_tn_tcgen05, but takes
 * no workspace argument: the partial sums and the tile counters live in a
 * file-scope device array of SRLM_STATIC_SCRATCH_BYTES that is part of the
 * library image.  Every GPU that loads the library holds that array until the
 * process exits.
 *
 * Rules for the caller:
 *  - With more than one split the partial sums lie in whole tiles of 128 weight
 *    rows by bn tokens, bn being M rounded up to 16, 32, 64, 128 or 256 (the
 *    smallest that holds M, else 256).  The scratch need is
 *        65536 + splits * ceil(N / 128) * ceil(M / bn) * 128 * bn * 4  bytes
 *    (up to twice splits * M * N * 4: M = 33 gives bn = 64), and there may be at
 *    most 16384 tiles.  Sizes whose need exceeds the array are refused with a
 *    negative status and a message from srlm_last_error(); nothing is launched.
 *    A single split needs no scratch.
 *  - The first call on a device looks the array's device address up (and sets a
 *    kernel attribute).  Make that first call outside any stream capture.
 *  - All calls share the one array and it keeps the last call's contents; the
 *    entry point clears the part that has to start at zero on the given stream
 *    before it launches.  Two calls that may overlap on the GPU (different
 *    streams, no dependency between them) race on the array: serialise them.
 *  - No cudaMalloc, cudaFree or allocating library routine is called.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SRLM_STATIC_SCRATCH_BYTES (65536 + (8 << 20))

/* c_dtype: 0 float32, 1 bfloat16.  ldx/ldw/ldc: leading dimensions in elements.  splits >= 1.
 * err_flag_out: optional host pointer; if not NULL the call synchronises the stream and stores the
 * kernel's error flag there (0 = every wait completed).  Returns 0, a cudaError_t, or a negative refusal. */
int srlm_gemm_tn_tcgen05_static(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                long long ldx, long long ldw, long long ldc, int splits, int* err_flag_out,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
