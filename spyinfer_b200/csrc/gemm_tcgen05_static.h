// Entry point of libspy_gemm_tcgen05.so for callers that cannot allocate device memory.
// It has no counterpart in the reference (spymaster2h/spyinfer allocates with cudaMalloc
// wherever it needs a buffer, even per call: src/backends/cuda/cublas/sgemm.cu:57-80).
//
//   C[M, N] = A[M, K] . W[N, K]^T     A, W bfloat16 (rows lda / ldw elements apart, K a multiple
//                                     of 8, 16-byte aligned), C bfloat16 (c_dtype 1) or float32
//                                     (c_dtype 0), rows ldc apart; when K is split, ldc == N.
//
// The caller passes inputs and outputs only.  The split-K partial sums go to a device array
// inside the library (SPY_GEMM_STATIC_SCRATCH_FLOATS floats on every GPU that loads it), so
// the call makes no cudaMalloc, no cudaFree and no call into an allocating library.
//
// What the array is used for depends on the number of tokens M (three classes):
// * Few tokens (at most 256, decoding): K may be split `splits` ways, splits x M x N floats of
//   partial products; the plans of that class need less than the array.
// * 257 tokens or more with fewer 128 x 256 tiles than SMs: the K blocks are shared out over
//   the SMs, one partial tile of 128 x 256 floats a block, over as many blocks as the array
//   holds tiles for (128): such a product always fits, with fewer blocks if need be.
// * 512 tokens or more with 8 or more, but fewer than SMs / 4, tiles of 256 x 256 (o and down
//   projections at a few hundred to a thousand tokens): K is cut into two to four ranges on
//   pairs of blocks, ranges x M x N floats.  512 x 4096 in two ranges fills the array exactly;
//   1,536 x 1,536 in two ranges does not fit.
// A plan that needs more than the array is refused before anything is launched (return 1; the
// message, with both sizes, is at spy_gemm_tcgen05_last_error()); it is not run another way.
// The sizes a plan needs are what spy_gemm_tcgen05_plan(M, N, K, limit, &splits, &floats) says.
// * The first call on a device looks the array's device address up (cudaGetSymbolAddress);
//   make it before any stream capture.
// * The one-time set-up under the entry point (the array's address, the kernels' shared-memory
//   attributes, the number of SMs) is kept per device, so one process may use several devices,
//   each made current before its calls.
// * All calls on a device share the array.  Nothing needs clearing between calls; calls that
//   overlap on the GPU race and must be ordered by the caller.  The same holds between this
//   entry point and the ordinary ones (spy_gemm_tcgen05, spy_gemm_tcgen05_ex) for products of
//   the second class: the flags by which their blocks signal a finished partial tile are one
//   array per device for the whole library, whichever scratch the caller gave.
// * After a status of 4 (a wait ran out) call spy_gemm_tcgen05_reset(stream) before the next
//   product: the one that gave up may have left such flags raised.
// * status: null, or two ints on the device that receive a code if a bounded wait inside the
//   kernel runs out.
#pragma once
#include <cuda_runtime.h>

#define SPY_GEMM_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif
int spy_gemm_tcgen05_static_scratch(const void* A, long long lda, const void* W, long long ldw, void* C, int c_dtype, long long ldc, int M,
                                    int N, int K, int* status, cudaStream_t stream);
int spy_gemm_tcgen05_reset(cudaStream_t stream);
int spy_gemm_tcgen05_plan(int M, int N, int K, long long scratch_limit, int* splits_out, long long* scratch_floats_out);
const char* spy_gemm_tcgen05_last_error();
#ifdef __cplusplus
}
#endif
