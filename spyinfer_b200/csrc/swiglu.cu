// SwiGLU on a fused gate|up activation: out[t, i] = silu(x[t, i]) * x[t, inter + i],
// silu(g) = g / (1 + exp(-g)), computed in 32-bit.  Replaces the reference's
// __cuda_swiglu_fp16 (spymaster2h/spyinfer src/backends/cuda/native/common.cu:56-73), which
// works in half arithmetic on separate gate and up tensors.
#include "common.cuh"

SPY_MODULE(spy_swiglu)

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long row = i / inter;
        const int col = (int)(i - row * inter);
        const T* src = gate_up + row * 2 * inter;
        const float g = to_f32(src[col]);
        const float u = to_f32(src[inter + col]);
        out[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

extern "C" int spy_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (inter <= 0) SPY_FAIL("swiglu: intermediate size %d must be positive", inter);
    const long long total = (long long)tokens * inter;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        spy_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, inter, total);
    })
    SPY_CHECK_LAUNCH("swiglu");
    return 0;
}

// out[t, c] += bias[c], in 32-bit: the bias of a product whose kernel has no bias term of its own
// (the reference's linear adds one when it is bound, spymaster2h/spyinfer
// src/backends/cpu/cpu_operator.cpp:150-186; its model binds none, src/models/qwen3.hpp:39, 143).
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ out, const TB* __restrict__ bias, int cols, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) out[i] = from_f32<T>(to_f32(out[i]) + to_f32(bias[i % cols]));
}

extern "C" int spy_add_bias(void* out, int dtype, const void* bias, int bias_dtype, int rows, int cols, cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (cols <= 0) SPY_FAIL("add_bias: %d columns", cols);
    const long long total = (long long)rows * cols;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        SPY_DISPATCH_DTYPE(bias_dtype, TB, {
            spy_launch(add_bias_kernel<T, TB>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const TB*)bias, cols, total);
        })
    })
    SPY_CHECK_LAUNCH("add_bias");
    return 0;
}

