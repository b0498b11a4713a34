// Plain matrix product on the CUDA cores, any sizes and any mix of 32-bit and bfloat16
// storage:  C[M, N] = A[M, K] . W[N, K]^T, every product and sum in 32-bit (FFMA; no tensor
// cores, no TF32).  It is the float32 path's matrix product (bfloat16 weights are widened
// exactly on the fly, so the weights are kept once) and the bfloat16 path's fallback for
// shapes the tensor-core kernel refuses.  Each output element is one thread's sum over k in
// ascending order, so a row's result does not depend on M or on what else is in the batch.
// The reference's counterpart on this path is its CPU Linear (spymaster2h/spyinfer
// src/backends/cpu/x64/kernels.cpp:95-166); its CUDA path calls cuBLAS in half precision.
#include "common.cuh"

SPY_MODULE(spy_gemm_simt)

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, long long ldw, TC* __restrict__ C, long long ldc,
                 int M, int N, int K)
{
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_enter();
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // each thread stages four consecutive k of one row of each tile
    const int lr = tid / 4, lk = (tid % 4) * 4;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + i][lr] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + i][lr] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

// Row strides lda/ldw/ldc are in elements.
extern "C" int spy_gemm_simt(const void* A, int a_dtype, long long lda, const void* W, int w_dtype, long long ldw, void* C, int c_dtype,
                             long long ldc, int M, int N, int K, cudaStream_t stream)
{
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) SPY_FAIL("gemm: K %d must be positive", K);
    if (lda < K || ldw < K || ldc < N) SPY_FAIL("gemm: row strides %lld/%lld/%lld are shorter than the rows", lda, ldw, ldc);
    const long long gy = ((long long)M + BM - 1) / BM;
    if (gy > 65535) SPY_FAIL("gemm: M %d exceeds the grid limit of this kernel (%d rows)", M, 65535 * BM);
    dim3 grid((N + BN - 1) / BN, (unsigned)gy);
    SPY_DISPATCH_DTYPE(a_dtype, TA, {
        SPY_DISPATCH_DTYPE(w_dtype, TW, {
            SPY_DISPATCH_DTYPE(c_dtype, TC, {
                spy_launch(gemm_simt_kernel<TA, TW, TC>, grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K);
            })
        })
    })
    SPY_CHECK_LAUNCH("gemm_simt");
    return 0;
}
