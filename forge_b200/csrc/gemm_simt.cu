// C[M,N] (fp32) = A[M,K] . W[N,K]^T (+ bias[N]) (+ C), by fp32 FMA on the CUDA cores.
//
// This is the engine's true 32-bit matrix product: operands are widened to fp32 when they are read,
// every product and sum is an fp32 FMA, and no tensor-core mode (TF32/BF16) is involved.  It stands in
// for the reference's gemm_tiled_kernel / gemv_transB_kernel / cuBLAS SGEMM trio
// (src/operators/cuda/cuda_gemm.cu:7-55, cuda_gemv.cu:9-40, cuda_quant.cu:582-599).  Each output element
// sums k = 0..K-1 in order, whatever M and N are, so a token's row does not depend on the batch around it.
// Any M, N, K >= 1 is accepted (edges are zero-filled in shared memory).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                 float* __restrict__ C, int M, int N, int K, int accumulate) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[TM][TN] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? forge::to_float(A[(size_t)gm * K + gk]) : 0.f;
        }
        for (int i = threadIdx.x; i < BN * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int gn = n0 + r, gk = k0 + c;
            Ws[c][r] = (gn < N && gk < K) ? forge::to_float(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            float* c = C + (size_t)gm * N + gn;
            *c = accumulate ? (*c + v) : v;
        }
    }
}

}  // namespace

// dtype: type of both A and W (FORGE_F32 or FORGE_BF16).  C is fp32.  accumulate != 0: C += A.W^T + bias.
extern "C" int forge_gemm_simt(const void* A, const void* W, const float* bias, float* C, int dtype,
                               int M, int N, int K, int accumulate, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return forge::fail(FORGE_ERR_ARG, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return FORGE_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_simt: M=%d too large", M);
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(gemm_simt_kernel<TT, TT>, grid, dim3(256), 0, stream, 1, (const TT*)A, (const TT*)W, bias, C, M, N, K, accumulate));
    return forge::check_launch("gemm_simt", e);
}
