// RMSNorm, optionally fused with the residual sum and with a row gather.
//   v   = x[row] (+ delta[row])                   32-bit sum
//   x[row] = v                                    when write_back (the residual stream)
//   out = v * (1 / sqrt(mean(v^2) + eps)) * w     32-bit statistics, plain weight
// Formula of the reference: spymaster2h/spyinfer src/backends/cpu/x64/kernels.cpp:168-180
// (its CUDA twin: src/backends/cuda/native/common.cuh:57-188, which needs len % 8 == 0 and
// launches a separate add kernel for the residual).  Any row length works here.
#include "common.cuh"

SPY_MODULE(spy_rmsnorm)

template <typename TX, typename TD, typename TW, typename TO>
__global__ void rmsnorm_kernel(TX* x, const TD* __restrict__ delta, const int* __restrict__ rows, const TW* __restrict__ w,
                               TO* __restrict__ out, int len, float eps, int write_back)
{
    extern __shared__ float row_buf[];  // len floats, then 33 of scratch
    float* scratch = row_buf + len;
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    TX* xr = x + (size_t)src_row * len;
    const TD* dr = delta ? delta + (size_t)src_row * len : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        float v = to_f32(xr[i]);
        if (dr) v += to_f32(dr[i]);
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
    TO* orow = out + (size_t)blockIdx.x * len;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float v = row_buf[i];
        if (write_back) xr[i] = from_f32<TX>(v);
        orow[i] = from_f32<TO>((inv * v) * to_f32(w[i]));
    }
}

template <typename TX, typename TD, typename TW, typename TO>
static int launch(void* x, const void* delta, const int* rows, const void* w, void* out, int n, int len, float eps, int write_back,
                  cudaStream_t stream)
{
    const size_t smem = (size_t)(len + 33) * sizeof(float);
    auto kernel = rmsnorm_kernel<TX, TD, TW, TO>;
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) SPY_FAIL("rmsnorm: a row of %d elements does not fit in shared memory (limit %d)", len, (227 * 1024) / 4 - 33);
        SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    const int threads = len >= 2048 ? 512 : (len >= 512 ? 256 : 128);
    kernel<<<n, threads, smem, stream>>>((TX*)x, (const TD*)delta, rows, (const TW*)w, (TO*)out, len, eps, write_back);
    SPY_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// x: [*, len] of x_dtype; delta: null or [*, len] of delta_dtype, added to x; rows: null or
// n row indices (gather); w: [len] of w_dtype; out: [n, len] of out_dtype.  write_back
// stores the sum into x and needs rows == null.
extern "C" int spy_rmsnorm(void* x, int x_dtype, const void* delta, int delta_dtype, const int* rows, const void* w, int w_dtype,
                           void* out, int out_dtype, int n, int len, float eps, int write_back, cudaStream_t stream)
{
    if (n <= 0) return 0;
    if (len <= 0) SPY_FAIL("rmsnorm: row length %d must be positive", len);
    if (write_back && rows) SPY_FAIL("rmsnorm: write_back with a row gather is not defined");
    if (write_back && !delta) write_back = 0;
    if (!delta) delta_dtype = x_dtype;
    SPY_DISPATCH_DTYPE(x_dtype, TX, {
        SPY_DISPATCH_DTYPE(delta_dtype, TD, {
            SPY_DISPATCH_DTYPE(w_dtype, TW, {
                SPY_DISPATCH_DTYPE(out_dtype, TO, {
                    return launch<TX, TD, TW, TO>(x, delta, rows, w, out, n, len, eps, write_back, stream);
                })
            })
        })
    })
    return 0;
}
