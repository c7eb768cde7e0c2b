// Shared helpers of the forge_b200 CUDA libraries (sm_100a).
//
// Every exported entry point is `extern "C" int forge_<name>(..., cudaStream_t stream)`:
// it validates its arguments on the host, launches on `stream`, and returns 0 or a negative
// error code after storing a message that forge_last_error() returns.  Nothing here allocates
// device memory; callers pass every buffer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#define FORGE_OK 0
#define FORGE_ERR_ARG (-1)
#define FORGE_ERR_LAUNCH (-2)
#define FORGE_ERR_UNSUPPORTED (-3)

enum ForgeDType { FORGE_F32 = 0, FORGE_BF16 = 1 };

namespace forge {

inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// cudaFuncSetAttribute and the like hold for the device that was current when they ran: one "done" flag
// per device.  current() is the flag of the device that is current now (a device index beyond the table
// shares a flag that never stays set, so its set-up simply runs again).
struct PerDeviceFlag {
    static constexpr int kMax = 64;
    bool done[kMax + 1] = {};
    bool& current() {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMax) {
            done[kMax] = false;
            return done[kMax];
        }
        return done[dev];
    }
};

inline int check_launch(const char* what, cudaError_t launch_result = cudaSuccess) {
    cudaError_t e = launch_result != cudaSuccess ? launch_result : cudaGetLastError();
    if (e != cudaSuccess) return fail(FORGE_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return FORGE_OK;
}

// Programmatic dependent launch.  Every kernel of these libraries is launched with the attribute that lets
// it start while its predecessor in the stream is still draining; it tells the scheduler at once that its
// own successor may be set up (launch_dependents), does whatever does not depend on earlier kernels
// (barrier set-up, weight prefetch), and executes pdl_wait() before it touches memory that an earlier
// kernel wrote or still reads.  Because every kernel waits, completion is transitive along the stream.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("FORGE_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

// Launches `kernel` with programmatic stream serialization (and an optional cluster size).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          int cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed tree (warp shuffles, then warp 0 over the per-warp sums):
// the order of additions depends only on blockDim, never on timing.
__device__ __forceinline__ float block_sum(float v, float* smem /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nwarps) ? smem[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) smem[0] = t;
    }
    __syncthreads();
    return smem[0];
}
__device__ __forceinline__ float block_max(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nwarps) ? smem[threadIdx.x] : -INFINITY;
    if (warp == 0) {
        t = warp_max(t);
        if (lane == 0) smem[0] = t;
    }
    __syncthreads();
    return smem[0];
}

}  // namespace forge

#define FORGE_DISPATCH_DTYPE(code, T, ...)                                            \
    do {                                                                              \
        if ((code) == FORGE_F32) { using T = float; __VA_ARGS__; }                    \
        else if ((code) == FORGE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }      \
        else return forge::fail(FORGE_ERR_ARG, "unknown dtype code %d", (int)(code)); \
    } while (0)
