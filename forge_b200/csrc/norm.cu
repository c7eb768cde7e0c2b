// RMSNorm over rows of the fp32 residual stream:  y = x * rsqrt(mean(x^2) + eps) * w.
// Formula of the reference (src/operators/cuda/cuda_rms_norm.cu:10-36, src/operators/cpu/norm.cpp:98-112),
// but the sum of squares uses a fixed reduction tree instead of atomicAdd on one shared float, so a
// row's result never depends on timing or on the other rows of the batch.  All arithmetic is fp32;
// only the store rounds to the output type.  `rows` (optional) picks which input rows are normed:
// the final norm runs only on the rows whose logits are wanted.
#include "common.cuh"

namespace {

constexpr int kNormThreads = 256;

template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ out,
               const int32_t* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
    }
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TOut* o = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += kNormThreads) o[c] = forge::from_float<TOut>(xr[c] * inv * w[c]);
}

}  // namespace

extern "C" int forge_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int32_t* rows,
                             int R, int H, float eps, cudaStream_t stream) {
    if (R < 0 || H <= 0) return forge::fail(FORGE_ERR_ARG, "rmsnorm: bad sizes R=%d H=%d", R, H);
    if (R == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(rmsnorm_kernel<TO>, dim3(R), dim3(kNormThreads), 0, stream, 1, x, w, (TO*)out, rows, H, eps));
    return forge::check_launch("rmsnorm", e);
}
