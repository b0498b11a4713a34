// Attention over the paged cache for any mix of queries: one block per (query token, head).
// This is the plain kernel: it takes every head size (a multiple of 4 elements), every page
// size, 32-bit or bfloat16 storage, and computes everything in 32-bit with expf.  It is the
// engine's float32 path and the fallback of the bfloat16 path for sizes its fast kernels
// refuse.
//
// A query at position p of sequence s sees the keys j with lo <= j <= p, lo = 0 or
// p - window + 1; key j lies in page block_table[s, j / page_size], slot j % page_size.
// kv head = head / (nh / nkv); score = (q . k) * scale; p = exp(score - max) / sum;
// o = sum p v.  Formula: spymaster2h/spyinfer src/backends/cpu/cpu_attention.cpp:89-135.
// Keys are processed in chunks of 128 that start at multiples of 128 of the absolute
// position, so the result of a query does not depend on how the batch was cut.
#include "common.cuh"

SPY_MODULE(spy_attention_generic)

constexpr int CHUNK = 128;

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4])
    {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(CHUNK)
attention_generic_kernel(const TA* __restrict__ q, long long q_row_stride, TA* __restrict__ out, const TC* __restrict__ pages,
                         const int* __restrict__ block_table, int table_width, int page_size, int num_pages, int nh, int nkv, int hd,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token, int window, float scale, int* status)
{
    extern __shared__ float smem[];
    pdl_enter();
    float* q_s = smem;                       // hd
    float* p_s = q_s + hd;                   // CHUNK
    long long* row_s = (long long*)(p_s + CHUNK);  // CHUNK offsets of K rows (elements); 8-byte aligned: hd % 4 == 0, CHUNK even
    float* scratch = (float*)(row_s + CHUNK);      // 33

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)seq * table_width;
    const long long v_offset = (long long)nkv * page_size * hd;  // from a K row to its V row

    const TA* q_row = q + (size_t)t * q_row_stride + (size_t)h * hd;
    for (int d = tid; d < hd; d += CHUNK) q_s[d] = to_f32(q_row[d]);

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // dims tid, tid+128, tid+256, tid+384
    __syncthreads();

    for (int c = lo / CHUNK; c <= pos / CHUNK; ++c) {
        const int j = c * CHUNK + tid;
        bool valid = j >= lo && j <= pos;
        long long row = 0;
        if (valid) {
            const int lp = j / page_size;
            const int page = lp < table_width ? bt[lp] : -1;
            if (page < 0 || page >= num_pages) {
                report_status(status, SPY_STATUS_BAD_PAGE, t);
                valid = false;
            } else {
                row = ((((long long)page * 2) * nkv + kvh) * page_size + j % page_size) * hd;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const TC* k = pages + row;
            float dot = 0.f;
            for (int d = 0; d < hd; d += 4) {
                float kv[4];
                Vec4<TC>::load(k + d, kv);
                dot = fmaf(q_s[d], kv[0], dot);
                dot = fmaf(q_s[d + 1], kv[1], dot);
                dot = fmaf(q_s[d + 2], kv[2], dot);
                dot = fmaf(q_s[d + 3], kv[3], dot);
            }
            s = dot * scale;
        }
        const float chunk_max = block_max(s, scratch);
        const float m_new = fmaxf(m, chunk_max);
        if (m_new == -INFINITY) continue;  // every key of the chunk was refused: nothing to add (uniform over the block)
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        row_s[tid] = row;
        const float chunk_sum = block_sum(p, scratch);  // its barriers also publish p_s and row_s
        l = l * alpha + chunk_sum;
        m = m_new;
        const int first = max(lo, c * CHUNK) - c * CHUNK, last = min(pos, c * CHUNK + CHUNK - 1) - c * CHUNK;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int d = tid + r * CHUNK;
            if (d < hd) {
                float a = acc[r] * alpha;
                for (int jj = first; jj <= last; ++jj) a = fmaf(p_s[jj], to_f32(pages[row_s[jj] + v_offset + d]), a);
                acc[r] = a;
            }
        }
        __syncthreads();  // p_s and row_s are rewritten by the next chunk
    }
    TA* o_row = out + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int d = tid + r * CHUNK;
        if (d < hd) o_row[d] = from_f32<TA>(l > 0.f ? acc[r] / l : 0.f);
    }
}

// q: [T, ...] rows of q_row_stride elements whose first nh*hd elements are the query heads;
// out: [T, nh*hd]; pages: one cache [num_pages][2][nkv][page_size][hd] of cache_dtype.
extern "C" int spy_attention_generic(const void* q, long long q_row_stride, void* out, int act_dtype, const void* pages, int cache_dtype,
                                     const int* block_table, int table_width, int page_size, int num_pages, int nh, int nkv, int hd,
                                     const int* positions, const int* seq_of_token, int tokens, int window, float scale, int* status,
                                     cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) SPY_FAIL("attention: %d query heads do not group over %d key/value heads", nh, nkv);
    if (hd <= 0 || hd % 4 != 0 || hd > 4 * CHUNK) SPY_FAIL("attention: head_dim %d must be a multiple of 4, at most %d", hd, 4 * CHUNK);
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("attention: page_size, num_pages and table_width must be positive");
    if (window < 0) SPY_FAIL("attention: window %d must be 0 (none) or positive", window);
    if (nh > 65535) SPY_FAIL("attention: %d heads exceed the grid limit", nh);
    const size_t smem = (size_t)(hd + CHUNK + 33) * sizeof(float) + (size_t)CHUNK * sizeof(long long);
    dim3 grid(tokens, nh);
    SPY_DISPATCH_DTYPE(act_dtype, TA, {
        SPY_DISPATCH_DTYPE(cache_dtype, TC, {
            spy_launch(attention_generic_kernel<TA, TC>, grid, dim3(CHUNK), smem, stream,
                (const TA*)q, q_row_stride, (TA*)out, (const TC*)pages, block_table, table_width, page_size, num_pages, nh, nkv, hd,
                positions, seq_of_token, window, scale, status);
        })
    })
    SPY_CHECK_LAUNCH("attention_generic");
    return 0;
}
