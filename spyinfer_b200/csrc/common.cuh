// Shared helpers of the kernel modules.  Every module is one .cu file built into one shared
// library with a C interface: functions return 0 on success, and on failure a non-zero code
// after storing a message that `<module>_last_error()` returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

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
        cudaError_t e_ = spy_take_launch_error();                                          \
        if (e_ != cudaSuccess) SPY_FAIL("%s: launch failed: %s", what, cudaGetErrorString(e_)); \
    } while (0)

#define SPY_CUDA(call)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) SPY_FAIL("%s: %s", #call, cudaGetErrorString(e_));          \
    } while (0)

// ---- what CUDA keeps per device ----------------------------------------------------------------
// Function attributes (the dynamic shared memory a kernel may use), occupancy figures and the
// number of SMs belong to a device, not to the process: set-up that is done "once" is done once
// per device, with that device current, and remembered by the device's index.
constexpr int SPY_MAX_DEVICES = 64;

static inline int spy_device()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= SPY_MAX_DEVICES) d = 0;
    return d;
}

// The current device's number of SMs (at least 1), asked once per device.
static inline int spy_sm_count()
{
    static int sms[SPY_MAX_DEVICES] = {};
    const int d = spy_device();
    if (sms[d] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 1;
        sms[d] = n;
    }
    return sms[d];
}

// Opens a block that runs once per device:  SPY_ONCE_PER_DEVICE { ...set-up... }
#define SPY_ONCE_PER_DEVICE                                                                \
    static bool spy_done_[SPY_MAX_DEVICES] = {};                                           \
    const int spy_dev_ = spy_device();                                                     \
    for (bool spy_run_ = !spy_done_[spy_dev_]; spy_run_; spy_run_ = false, spy_done_[spy_dev_] = true)

// ---- launches with programmatic dependent launch --------------------------------------------
// Every kernel of this library is launched with the programmatic-stream-serialization
// attribute: it may begin while the kernel before it in the stream is still finishing.  In
// return every kernel calls pdl_wait() before it reads or writes anything another kernel
// touches (the wait returns when all earlier kernels are complete and their memory is visible),
// and pdl_launch_dependents() as early as it can, which lets the next kernel start its
// prologue.  A kernel may do work that depends on no other kernel before its wait: the
// tensor-core product uses that to prefetch weights.  SPYINFER_PDL=0 in the environment
// turns the attribute off (the two instructions are then no-ops).
static thread_local cudaError_t g_spy_launch_error = cudaSuccess;

static inline bool spy_pdl_enabled()
{
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("SPYINFER_PDL");
        enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

static inline cudaError_t spy_take_launch_error()
{
    cudaError_t e = g_spy_launch_error;
    g_spy_launch_error = cudaSuccess;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e;
}

template <typename... KArgs, typename... Args>
static inline void spy_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = spy_pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) g_spy_launch_error = e;
}

// The same for a kernel whose blocks form clusters of `cluster` along x.
template <typename... KArgs, typename... Args>
static inline void spy_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = spy_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) g_spy_launch_error = e;
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// the usual opening of a kernel that has nothing to do before its inputs are ready
__device__ __forceinline__ void pdl_enter()
{
    pdl_launch_dependents();
    pdl_wait();
}

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
