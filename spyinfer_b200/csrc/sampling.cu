// Next-token choice from 32-bit logits.
//   temperature == 0: argmax, lowest index on ties (the reference's only sampler:
//     spymaster2h/spyinfer src/engine/model_runner.cpp:120-134, std::max_element on the host).
//   temperature  > 0: a draw from softmax(logits / temperature) by the Gumbel-max rule:
//     argmax_i (logits[i] / temperature - log(-log(u_i))), u_i uniform in (0, 1) from a
//     counter-based generator keyed by (seed, draw, i).  A row's token depends only on its
//     logits, seed and draw number, never on the rest of the batch.
// Two stages so that a row of a large vocabulary is read by many blocks: every block finds
// the best of its slice of the row, then one block per row picks among the slices' bests.
#include "common.cuh"

SPY_MODULE(spy_sampling)

__device__ __forceinline__ uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float uniform_open(uint64_t key, uint32_t index)
{
    const uint64_t r = mix64(key + index);
    return ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // 24 bits, never 0 or 1
}

constexpr int NONE = 0x7fffffff;

__device__ __forceinline__ void take_better(float& bv, int& bi, float ov, int oi)
{
    if (oi != NONE && (bi == NONE || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
}

// Reduces (value, index) over the block; thread 0 gets the result.
__device__ __forceinline__ void block_best(float& bv, int& bi)
{
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarps ? best_v[lane] : -INFINITY;
        bi = lane < nwarps ? best_i[lane] : NONE;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    }
}

__global__ void sample_slices_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int slice, const float* __restrict__ temperature,
                                     const long long* __restrict__ seed, const long long* __restrict__ draw, float* __restrict__ slice_v,
                                     int* __restrict__ slice_i)
{
    pdl_enter();
    const int r = blockIdx.y, lo = blockIdx.x * slice, hi = min(vocab, lo + slice);
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const uint64_t key = mix64((seed ? (uint64_t)seed[r] : 0) ^ mix64(draw ? (uint64_t)draw[r] : 0));
    float bv = -INFINITY;
    int bi = NONE;
    auto take = [&](float v, int i) {
        if (temp > 0.f) v = v / temp - logf(-logf(uniform_open(key, (uint32_t)i)));
        if (bi == NONE || v > bv) { bv = v; bi = i; }   // ascending i: the lowest index is kept on ties
    };
    if (((reinterpret_cast<uintptr_t>(row) | (uintptr_t)lo * 4) & 15) == 0) {
        // 16-byte loads; a thread's indices still ascend
        const int quads = (hi - lo) / 4;
        for (int q = threadIdx.x; q < quads; q += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(row + lo + 4 * q);
            take(v.x, lo + 4 * q);
            take(v.y, lo + 4 * q + 1);
            take(v.z, lo + 4 * q + 2);
            take(v.w, lo + 4 * q + 3);
        }
        for (int i = lo + 4 * quads + threadIdx.x; i < hi; i += blockDim.x) take(row[i], i);
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) take(row[i], i);
    }
    block_best(bv, bi);
    if (threadIdx.x == 0) {
        slice_v[(size_t)r * gridDim.x + blockIdx.x] = bv;
        slice_i[(size_t)r * gridDim.x + blockIdx.x] = bi;
    }
}

__global__ void sample_pick_kernel(const float* __restrict__ slice_v, const int* __restrict__ slice_i, int slices, int* __restrict__ tokens)
{
    pdl_enter();
    const int r = blockIdx.x;
    float bv = -INFINITY;
    int bi = NONE;
    for (int s = threadIdx.x; s < slices; s += blockDim.x) take_better(bv, bi, slice_v[(size_t)r * slices + s], slice_i[(size_t)r * slices + s]);
    block_best(bv, bi);
    if (threadIdx.x == 0) tokens[r] = bi == NONE ? 0 : bi;
}

// How many slices a row of `vocab` logits is cut into.
extern "C" int spy_sample_slices(int vocab) { return vocab <= 4096 ? 1 : (vocab + 4095) / 4096; }

// logits: [rows, vocab] floats, rows row_stride apart.  temperature/seed/draw: per row, or
// null for greedy.  tokens: [rows] int32 out.  slice_v / slice_i: rows * spy_sample_slices(vocab)
// floats / ints of scratch.
extern "C" int spy_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature, const long long* seed,
                          const long long* draw, int* tokens, float* slice_v, int* slice_i, cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) SPY_FAIL("sample: vocab %d must be positive and fit the row stride %lld", vocab, row_stride);
    if (rows > 65535) SPY_FAIL("sample: %d rows exceed the grid limit", rows);
    const int slices = spy_sample_slices(vocab);
    const int slice = ((vocab + slices - 1) / slices + 3) / 4 * 4;   // a multiple of 4: slices start on 16-byte boundaries
    dim3 grid(slices, rows);
    spy_launch(sample_slices_kernel, grid, dim3(256), 0, stream, logits, row_stride, vocab, slice, temperature, seed, draw, slice_v, slice_i);
    SPY_CHECK_LAUNCH("sample (slices)");
    spy_launch(sample_pick_kernel, dim3(rows), dim3(64), 0, stream, slice_v, slice_i, slices, tokens);
    SPY_CHECK_LAUNCH("sample (pick)");
    return 0;
}
