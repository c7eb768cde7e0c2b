// SwiGLU gate:  out[t,j] = silu(g) * u with g = gu[t,2j], u = gu[t,2j+1], silu(g) = g / (1 + expf(-g))
// (formula of src/operators/cuda/cuda_elementwise.cu:34-41).  The gate and up projections are stored
// with their rows interleaved, so one GEMM yields [T, 2I] with each (gate, up) pair adjacent.
#include "common.cuh"

namespace {

template <typename TOut>
__global__ void silu_mul_interleaved_kernel(const float* __restrict__ gu, TOut* __restrict__ out, size_t n) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float2 p = reinterpret_cast<const float2*>(gu)[i];
    out[i] = forge::from_float<TOut>(p.x / (1.0f + expf(-p.x)) * p.y);
}

}  // namespace

extern "C" int forge_silu_mul_interleaved(const float* gu, void* out, int out_dtype, int T, int I,
                                          cudaStream_t stream) {
    if (T < 0 || I <= 0) return forge::fail(FORGE_ERR_ARG, "silu_mul: bad sizes T=%d I=%d", T, I);
    const size_t n = (size_t)T * I;
    if (n == 0) return FORGE_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(silu_mul_interleaved_kernel<TO>, dim3(blocks), dim3(256), 0, stream, 1, gu, (TO*)out, n));
    return forge::check_launch("silu_mul_interleaved", e);
}
