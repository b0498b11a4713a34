// RMSNorm, optionally fused with the residual sum and with a row gather.
//   v   = x[row] (+ delta[row], itself possibly a sum of split-K partial products)   32-bit sums
//   x[row] = v                                    when write_back (the residual stream)
//   out = v * (1 / sqrt(mean(v^2) + eps)) * w     32-bit statistics, plain weight
// Formula of the reference: spymaster2h/spyinfer src/backends/cpu/x64/kernels.cpp:168-180
// (its CUDA twin: src/backends/cuda/native/common.cuh:57-188, which needs len % 8 == 0 and
// launches a separate add kernel for the residual).  Any row length works here; rows whose
// length is a multiple of 4 take 16- and 8-byte accesses.
#include "common.cuh"

SPY_MODULE(spy_rmsnorm)

template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4])
    {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4])
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<uint32_t*>(&a);
        x.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};


template <typename TX, typename TD, typename TW, typename TO, bool VEC>
__global__ void __launch_bounds__(1024) rmsnorm_kernel(TX* x, const TD* __restrict__ delta, int delta_splits, long long delta_split_stride, const int* __restrict__ rows,
                               const TW* __restrict__ w, TO* __restrict__ out, int len, float eps, int write_back)
{
    extern __shared__ float row_buf[];  // len floats, then 33 of scratch
    // The weight depends on no kernel ahead in the stream: the first quad of it (all of it when
    // the block spans the row, as in decoding) is loaded before the wait for those kernels.
    pdl_launch_dependents();
    float w_first[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (VEC) {
        if ((int)threadIdx.x * 4 < len) Quad<TW>::load(w + threadIdx.x * 4, w_first);
    }
    pdl_wait();
    float* scratch = row_buf + len;
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    TX* xr = x + (size_t)src_row * len;
    const TD* dr = delta ? delta + (size_t)src_row * len : nullptr;
    TO* orow = out + (size_t)blockIdx.x * len;
    float ss = 0.f;
    if constexpr (VEC) {
        for (int i = threadIdx.x * 4; i < len; i += blockDim.x * 4) {
            float v[4];
            Quad<TX>::load(xr + i, v);
            if (dr) {
                // the partial products are added in their order; four loads are in flight at a time
                for (int s0 = 0; s0 < delta_splits; s0 += 4) {
                    float d[4][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (s0 + j < delta_splits) Quad<TD>::load(dr + (size_t)(s0 + j) * delta_split_stride + i, d[j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (s0 + j < delta_splits) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[e] += d[j][e];
                        }
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                row_buf[i + e] = v[e];
                ss += v[e] * v[e];
            }
            if (write_back) Quad<TX>::store(xr + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            float v = to_f32(xr[i]);
            if (dr)
                for (int s = 0; s < delta_splits; ++s) v += to_f32(dr[(size_t)s * delta_split_stride + i]);
            row_buf[i] = v;
            ss += v * v;
            if (write_back) xr[i] = from_f32<TX>(v);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
    if constexpr (VEC) {
        for (int i = threadIdx.x * 4; i < len; i += blockDim.x * 4) {
            float wv[4], o[4];
            if (i == (int)threadIdx.x * 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) wv[e] = w_first[e];
            } else {
                Quad<TW>::load(w + i, wv);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = (inv * row_buf[i + e]) * wv[e];
            Quad<TO>::store(orow + i, o);
        }
    } else {
        for (int i = threadIdx.x; i < len; i += blockDim.x) orow[i] = from_f32<TO>((inv * row_buf[i]) * to_f32(w[i]));
    }
}


// Few rows (decoding): one block per row, the row in registers (QUADS quads of four elements per
// thread), no shared row buffer, at most 48 registers: a block of 1,024 threads then leaves
// room on its SM for the blocks of the product that follows, which start streaming their
// weights before this kernel has finished.  All partial products of a thread's elements are
// requested together, six quads at a time.
template <typename TX, typename TD, typename TW, typename TO, int QUADS>
__global__ void __maxnreg__(QUADS <= 2 ? 48 : 80) rmsnorm_row_kernel(TX* x, const TD* __restrict__ delta, int delta_splits, long long delta_split_stride,
                                                   const int* __restrict__ rows, const TW* __restrict__ w, TO* __restrict__ out, int len, float eps,
                                                   int write_back)
{
    __shared__ float scratch[33];
    pdl_launch_dependents();
    // the weight depends on no kernel ahead in the stream: it is loaded before the wait for them
    float wv[QUADS][4];
#pragma unroll
    for (int q = 0; q < QUADS; ++q) {
        const int i = (q * blockDim.x + threadIdx.x) * 4;
        if (i < len) Quad<TW>::load(w + i, wv[q]);
    }
    pdl_wait();
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    TX* xr = x + (size_t)src_row * len;
    const TD* dr = delta ? delta + (size_t)src_row * len : nullptr;
    TO* orow = out + (size_t)blockIdx.x * len;
    float v[QUADS][4];
#pragma unroll
    for (int q = 0; q < QUADS; ++q) {
        const int i = (q * blockDim.x + threadIdx.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[q][e] = 0.f;
        if (i < len) Quad<TX>::load(xr + i, v[q]);
    }
    if (dr) {
        constexpr int B = QUADS <= 2 ? 6 / QUADS : 1;
        for (int s0 = 0; s0 < delta_splits; s0 += B) {
            float d[B][QUADS][4];
#pragma unroll
            for (int j = 0; j < B; ++j)
#pragma unroll
                for (int q = 0; q < QUADS; ++q) {
                    const int i = (q * blockDim.x + threadIdx.x) * 4;
                    if (s0 + j < delta_splits && i < len) Quad<TD>::load(dr + (size_t)(s0 + j) * delta_split_stride + i, d[j][q]);
                }
#pragma unroll
            for (int j = 0; j < B; ++j)
#pragma unroll
                for (int q = 0; q < QUADS; ++q) {
                    const int i = (q * blockDim.x + threadIdx.x) * 4;
                    if (s0 + j < delta_splits && i < len) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[q][e] += d[j][q][e];
                    }
                }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < QUADS; ++q) {
        const int i = (q * blockDim.x + threadIdx.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += v[q][e] * v[q][e];
        if (write_back && i < len) Quad<TX>::store(xr + i, v[q]);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
#pragma unroll
    for (int q = 0; q < QUADS; ++q) {
        const int i = (q * blockDim.x + threadIdx.x) * 4;
        if (i < len) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = (inv * v[q][e]) * wv[q][e];
            Quad<TO>::store(orow + i, o);
        }
    }
}

template <typename TX, typename TD, typename TW, typename TO>
static int launch(void* x, const void* delta, int delta_splits, long long delta_split_stride, const int* rows, const void* w, void* out, int n,
                  int len, float eps, int write_back, cudaStream_t stream)
{
    const size_t smem = (size_t)(len + 33) * sizeof(float);
    const bool vec = len % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(w) |
                                       reinterpret_cast<uintptr_t>(out)) & 15) == 0 && delta_split_stride % 4 == 0;
    if (vec && (n < 512 ? len <= 8192 : len <= 16384)) {
        // the row lives in registers.  Few rows: one or two quads per thread, the row spread as wide as it goes;
        // many rows: four quads per thread, all their loads in flight together, several blocks an SM
        const int quads = n >= 512 ? 4 : (len <= 4096 ? 1 : 2);
        int threads = ((len / 4 + quads - 1) / quads + 31) / 32 * 32;
        if (threads < 64) threads = 64;
#define SPY_RMS_ROW(Q_)                                                                                                                          \
    spy_launch(rmsnorm_row_kernel<TX, TD, TW, TO, Q_>, dim3(n), dim3(threads), 0, stream, (TX*)x, (const TD*)delta, delta_splits, delta_split_stride, \
               rows, (const TW*)w, (TO*)out, len, eps, write_back)
        if (quads == 1) SPY_RMS_ROW(1);
        else if (quads == 2) SPY_RMS_ROW(2);
        else SPY_RMS_ROW(4);
#undef SPY_RMS_ROW
        SPY_CHECK_LAUNCH("rmsnorm (row in registers)");
        return 0;
    }
    auto kernel = vec ? rmsnorm_kernel<TX, TD, TW, TO, true> : rmsnorm_kernel<TX, TD, TW, TO, false>;
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) SPY_FAIL("rmsnorm: a row of %d elements does not fit in shared memory (limit %d)", len, (227 * 1024) / 4 - 33);
        SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
#ifndef SPY_RMS_ELEMS
#define SPY_RMS_ELEMS 4
#endif
    // many rows: fewer threads per row, several 16-byte loads each, more blocks per SM, so that rows in their load
    // phase overlap rows in their store phase; few rows (decoding): one load per thread, the row spread as wide as it goes
    const int per_thread = vec ? (n >= 512 ? SPY_RMS_ELEMS * 4 : 4) : 1;
    int threads = (len / per_thread + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : (threads + 31) / 32 * 32);
    spy_launch(kernel, dim3(n), dim3(threads), smem, stream, (TX*)x, (const TD*)delta, delta_splits, delta_split_stride, rows, (const TW*)w, (TO*)out, len, eps,
                                         write_back);
    SPY_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// x: [*, len] of x_dtype; delta: null or delta_splits stacked [*, len] arrays of delta_dtype
// (delta_split_stride elements apart), all added to x in order; rows: null or n row indices
// (gather); w: [len] of w_dtype; out: [n, len] of out_dtype.  write_back stores the sum into
// x and needs rows == null.
extern "C" int spy_rmsnorm(void* x, int x_dtype, const void* delta, int delta_dtype, int delta_splits, long long delta_split_stride,
                           const int* rows, const void* w, int w_dtype, void* out, int out_dtype, int n, int len, float eps, int write_back,
                           cudaStream_t stream)
{
    if (n <= 0) return 0;
    if (len <= 0) SPY_FAIL("rmsnorm: row length %d must be positive", len);
    if (write_back && rows) SPY_FAIL("rmsnorm: write_back with a row gather is not defined");
    if (delta && delta_splits <= 0) SPY_FAIL("rmsnorm: delta_splits %d must be positive", delta_splits);
    if (write_back && !delta) write_back = 0;
    if (!delta) { delta_dtype = x_dtype; delta_splits = 0; delta_split_stride = 0; }
    SPY_DISPATCH_DTYPE(x_dtype, TX, {
        SPY_DISPATCH_DTYPE(delta_dtype, TD, {
            SPY_DISPATCH_DTYPE(w_dtype, TW, {
                SPY_DISPATCH_DTYPE(out_dtype, TO, {
                    return launch<TX, TD, TW, TO>(x, delta, delta_splits, delta_split_stride, rows, w, out, n, len, eps, write_back, stream);
                })
            })
        })
    })
    return 0;
}
