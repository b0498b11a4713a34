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
