// Token embedding: out[t, :] = table[ids[t], :], widened to the 32-bit residual stream.
// Replaces the reference's __cuda_embedding_kernel (spymaster2h/spyinfer
// src/backends/cuda/native/common.cuh:45-55): same gather, no scaling.
#include "common.cuh"

SPY_MODULE(spy_embedding)

template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, int* status)
{
    pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_TOKEN, t);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]);
}

extern "C" int spy_embedding(const void* table, int table_dtype, const int* ids, float* out, int tokens, int hidden, int vocab,
                             int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) SPY_FAIL("embedding: hidden %d and vocab %d must be positive", hidden, vocab);
    SPY_DISPATCH_DTYPE(table_dtype, TW, {
        spy_launch(embedding_kernel<TW>, dim3(tokens), dim3(256), 0, stream, (const TW*)table, ids, out, hidden, vocab, status);
    })
    SPY_CHECK_LAUNCH("embedding");
    return 0;
}
