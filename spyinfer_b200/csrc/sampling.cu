// Next-token choice from 32-bit logits.
//   temperature == 0: argmax, lowest index on ties (the reference's only sampler:
//     spymaster2h/spyinfer src/engine/model_runner.cpp:120-134, std::max_element on the host).
//   temperature  > 0: a draw from softmax(logits / temperature) by the Gumbel-max rule:
//     argmax_i (logits[i] / temperature - log(-log(u_i))), u_i uniform in (0, 1) from a
//     counter-based generator keyed by (seed, draw, i).  A row's token depends only on its
//     logits, seed and draw number, never on the rest of the batch.
//   top_k > 0 (with a temperature): the draw is among the row's k largest logits only.  A
//     kernel ahead finds the row's k-th largest value by a radix select on the floats' bit
//     patterns (four passes of eight bits); logits below it take no part.  Logits equal to the
//     k-th value all stay, so a tie at the edge keeps more than k.
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

// Bit pattern of a float as an unsigned integer whose order is the floats' order.
__device__ __forceinline__ uint32_t ordered_bits(float v)
{
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// One block per row: floor[r] = the row's top_k[r]-th largest logit (-inf where top_k[r] <= 0
// or top_k[r] >= vocab: every logit takes part).
__global__ void topk_floor_kernel(const float* __restrict__ logits, long long row_stride, int vocab, const int* __restrict__ top_k,
                                  float* __restrict__ floor_out)
{
    pdl_enter();
    __shared__ unsigned int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_want;
    const int r = blockIdx.x;
    const int k = top_k[r];
    if (k <= 0 || k >= vocab) {
        if (threadIdx.x == 0) floor_out[r] = -INFINITY;
        return;
    }
    const float* row = logits + (size_t)r * row_stride;
    uint32_t prefix = 0;   // the bits of the k-th largest key found so far (from the top)
    int want = k;          // its rank among the keys that share the prefix
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask = pass == 0 ? 0u : 0xffffffffu << (shift + 8);
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const uint32_t key = ordered_bits(row[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int left = want, d = 255;
            for (; d > 0; --d) {
                if ((int)hist[d] >= left) break;
                left -= (int)hist[d];
            }
            s_prefix = prefix | ((uint32_t)d << shift);
            s_want = left;
        }
        __syncthreads();
        prefix = s_prefix;
        want = s_want;
        __syncthreads();
    }
    if (threadIdx.x == 0) floor_out[r] = from_ordered_bits(prefix);
}

__global__ void sample_slices_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int slice, const float* __restrict__ temperature,
                                     const long long* __restrict__ seed, const long long* __restrict__ draw, const float* __restrict__ floor_in,
                                     float* __restrict__ slice_v, int* __restrict__ slice_i)
{
    pdl_enter();
    const int r = blockIdx.y, lo = blockIdx.x * slice, hi = min(vocab, lo + slice);
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const float floor_v = (floor_in && temp > 0.f) ? floor_in[r] : -INFINITY;
    const uint64_t key = mix64((seed ? (uint64_t)seed[r] : 0) ^ mix64(draw ? (uint64_t)draw[r] : 0));
    float bv = -INFINITY;
    int bi = NONE;
    auto take = [&](float v, int i) {
        if (v < floor_v) return;   // outside the row's top k
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
// null for greedy.  top_k: per row (0 or less: the whole row), or null; floor_v: [rows] floats of
// scratch when top_k is given.  tokens: [rows] int32 out.  slice_v / slice_i:
// rows * spy_sample_slices(vocab) floats / ints of scratch.
extern "C" int spy_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature, const long long* seed,
                          const long long* draw, const int* top_k, float* floor_v, int* tokens, float* slice_v, int* slice_i,
                          cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) SPY_FAIL("sample: vocab %d must be positive and fit the row stride %lld", vocab, row_stride);
    if (rows > 65535) SPY_FAIL("sample: %d rows exceed the grid limit", rows);
    const int slices = spy_sample_slices(vocab);
    const int slice = ((vocab + slices - 1) / slices + 3) / 4 * 4;   // a multiple of 4: slices start on 16-byte boundaries
    dim3 grid(slices, rows);
    const float* floor_in = nullptr;
    if (top_k && temperature) {
        if (!floor_v) SPY_FAIL("sample: top_k needs its scratch of %d floats", rows);
        spy_launch(topk_floor_kernel, dim3(rows), dim3(1024), 0, stream, logits, row_stride, vocab, top_k, floor_v);
        SPY_CHECK_LAUNCH("sample (top-k floor)");
        floor_in = floor_v;
    }
    spy_launch(sample_slices_kernel, grid, dim3(256), 0, stream, logits, row_stride, vocab, slice, temperature, seed, draw, floor_in, slice_v,
               slice_i);
    SPY_CHECK_LAUNCH("sample (slices)");
    spy_launch(sample_pick_kernel, dim3(rows), dim3(64), 0, stream, slice_v, slice_i, slices, tokens);
    SPY_CHECK_LAUNCH("sample (pick)");
    return 0;
}
