// Next-token choice from 32-bit logits, one block per row.
//   temperature == 0: argmax, lowest index on ties (the reference's only sampler:
//     spymaster2h/spyinfer src/engine/model_runner.cpp:120-134, std::max_element on the host).
//   temperature  > 0: a draw from softmax(logits / temperature) by the Gumbel-max rule:
//     argmax_i (logits[i] / temperature - log(-log(u_i))), u_i uniform in (0, 1) from a
//     counter-based generator keyed by (seed, draw, i).  A row's token depends only on its
//     logits, seed and draw number, never on the rest of the batch.
#include "common.cuh"

SPY_MODULE(spy_sampling)

__device__ __forceinline__ uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float uniform_open(uint64_t seed, uint64_t draw, uint32_t index)
{
    const uint64_t r = mix64(mix64(seed ^ mix64(draw)) + index);
    return ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // 24 bits, never 0 or 1
}

__global__ void sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
                              const long long* __restrict__ seed, const long long* __restrict__ draw, int* __restrict__ tokens)
{
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const uint64_t sd = seed ? (uint64_t)seed[r] : 0, dr = draw ? (uint64_t)draw[r] : 0;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = row[i];
        if (temp > 0.f) v = v / temp - logf(-logf(uniform_open(sd, dr, (uint32_t)i)));
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarps ? best_v[lane] : -INFINITY;
        bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) tokens[r] = bi == 0x7fffffff ? 0 : bi;
    }
}

// logits: [rows, vocab] floats, rows row_stride apart.  temperature/seed/draw: per row, or
// null for greedy.  tokens: [rows] int32 out.
extern "C" int spy_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature, const long long* seed,
                          const long long* draw, int* tokens, cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) SPY_FAIL("sample: vocab %d must be positive and fit the row stride %lld", vocab, row_stride);
    sample_kernel<<<rows, 1024, 0, stream>>>(logits, row_stride, vocab, temperature, seed, draw, tokens);
    SPY_CHECK_LAUNCH("sample");
    return 0;
}
