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
// * Few tokens (at most 64): K may be split, and the plans of that class need less than the
//   array; a plan that needed more would be refused (return 1; the message is at
//   spy_gemm_tcgen05_last_error()).  A few hundred tokens with fewer tiles than SMs: the K
//   blocks are shared out over the SMs, one partial tile of 128 x 256 floats a block, over as
//   many blocks as the array holds tiles for (128).
// * The first call on a device looks the array's device address up (cudaGetSymbolAddress);
//   make it before any stream capture.
// * All calls on a device share the array.  Nothing needs clearing between calls; calls that
//   overlap on the GPU race and must be ordered by the caller.
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
const char* spy_gemm_tcgen05_last_error();
#ifdef __cplusplus
}
#endif
