// Token embedding gather: out[t,:] = table[ids[t],:], written to the fp32 residual stream.
// Replaces the reference's embedding_kernel (src/operators/cuda/cuda_embedding.cu:9-34); like it,
// an id outside [0,V) gives a row of zeros, and here it also raises bit 0 of *status.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V, int* status) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = forge::to_float(row[c]);
}

}  // namespace

extern "C" int forge_embedding(const int32_t* ids, const void* table, int table_dtype, float* out,
                               int T, int H, int V, int* status, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return FORGE_OK;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(table_dtype, TT,
        e = forge::launch(embedding_kernel<TT>, dim3(T), dim3(threads), 0, stream, 1, ids, (const TT*)table, out, H, V, status));
    return forge::check_launch("embedding", e);
}
