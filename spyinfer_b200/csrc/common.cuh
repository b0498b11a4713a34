// Shared helpers of the kernel modules.  Every module is one .cu file built into one shared
// library with a C interface: functions return 0 on success, and on failure a non-zero code
// after storing a message that `<module>_last_error()` returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

typedef __nv_bfloat16 bf16;

// dtype codes of the C interface
enum { SPY_F32 = 0, SPY_BF16 = 1 };

// Codes a kernel stores in the engine's device status word when it meets an index that
// would leave its buffers; the access is skipped and the host raises after the step.
enum {
    SPY_STATUS_OK = 0,
    SPY_STATUS_BAD_TOKEN = 1,
    SPY_STATUS_BAD_POSITION = 2,
    SPY_STATUS_BAD_PAGE = 3,
    SPY_STATUS_WAIT_TIMEOUT = 4,
};

#define SPY_MODULE(name)                                                                   \
    static thread_local char g_spy_error[512] = "";                                        \
    extern "C" const char* name##_last_error() { return g_spy_error; }

#define SPY_FAIL(...)                                                                      \
    do {                                                                                   \
        snprintf(g_spy_error, sizeof(g_spy_error), __VA_ARGS__);                           \
        return 1;                                                                          \
    } while (0)

#define SPY_CHECK_LAUNCH(what)                                                             \
    do {                                                                                   \
        cudaError_t e_ = cudaGetLastError();                                               \
        if (e_ != cudaSuccess) SPY_FAIL("%s: launch failed: %s", what, cudaGetErrorString(e_)); \
    } while (0)

#define SPY_CUDA(call)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) SPY_FAIL("%s: %s", #call, cudaGetErrorString(e_));          \
    } while (0)

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ void report_status(int* status, int code, int detail)
{
    if (status != nullptr && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 33 floats; every thread gets the
// result.  The order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Calls `body` with a value of the C++ type that a dtype code stands for.
#define SPY_DISPATCH_DTYPE(code, T, ...)                                                   \
    if ((code) == SPY_F32) { typedef float T; __VA_ARGS__ }                                 \
    else if ((code) == SPY_BF16) { typedef bf16 T; __VA_ARGS__ }                            \
    else SPY_FAIL("unknown dtype code %d", (int)(code));
