// RMSNorm over rows of the fp32 residual stream:  y = x * rsqrt(mean(x^2) + eps) * w.
// Formula of the reference (src/operators/cuda/cuda_rms_norm.cu:10-36, src/operators/cpu/norm.cpp:98-112),
// but the sum of squares uses a fixed reduction tree instead of atomicAdd on one shared float, so a
// row's result never depends on timing or on the other rows of the batch.  All arithmetic is fp32;
// only the store rounds to the output type.  `rows` (optional) picks which input rows are normed:
// the final norm runs only on the rows whose logits are wanted.
#include "common.cuh"

namespace {

constexpr int kNormThreads = 128;

template <typename TOut> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
};

// One CTA per row.  With H a multiple of 4 a thread reads float4s (the first kKeep of them stay in registers
// for the second pass, beside the weights they meet there) and writes four outputs at a time; any other H goes
// element by element.
template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ out,
               const int32_t* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    constexpr int kKeep = 4;
    forge::pdl_launch_dependents();
    // the norm's weights do not depend on the kernel before: a thread's first kKeep float4s of them are read ahead of
    // the dependency wait instead of after the row's reduction, where the load's latency stood in the open
    float4 gain[kKeep];
    if ((H & 3) == 0) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            gain[i] = c < (H >> 2) ? reinterpret_cast<const float4*>(w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    forge::pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    TOut* o = out + (size_t)r * H;
    if ((H & 3) == 0) {
        const int n4 = H >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        float4 keep[kKeep];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            keep[i] = c < n4 ? x4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += (keep[i].x * keep[i].x + keep[i].y * keep[i].y) + (keep[i].z * keep[i].z + keep[i].w * keep[i].w);
        }
        for (int c = threadIdx.x + kKeep * kNormThreads; c < n4; c += kNormThreads) {
            const float4 v = x4[c];
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        ss = forge::block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            if (c < n4) {
                const float4 g = gain[i];
                Pack4<TOut>::store(o + 4 * c, keep[i].x * inv * g.x, keep[i].y * inv * g.y, keep[i].z * inv * g.z, keep[i].w * inv * g.w);
            }
        }
        for (int c = threadIdx.x + kKeep * kNormThreads; c < n4; c += kNormThreads) {
            const float4 v = x4[c], g = w4[c];
            Pack4<TOut>::store(o + 4 * c, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
    }
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
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
