// Token selection on the device, one thread block per row of fp32 logits [R, V].
//
//  * forge_argmax: greedy; the lowest index wins a tie (the reference's CPU scan keeps the first
//    maximum, src/inference/sampler.cpp:137-142; its device argmax, cuda_quant.cu:526-580, leaves the
//    tie order to the block layout).
//  * forge_repeat_penalty: logit > 0 -> /penalty else *penalty, once per occurrence of the token in the
//    request's history (src/inference/sampler.cpp:340-351); the host passes (token, count) pairs.
//  * forge_sample: the reference's temperature / top-k / top-p pipeline (src/inference/sampler.cpp:197-328):
//      w_i = expf((l_i - max) / temperature);  top-k keeps the k largest, top-p then keeps the smallest
//      set of largest weights whose share exceeds p; the token is the first index whose running sum of
//      kept weights reaches u * (sum of kept weights), u in [0,1] supplied per row by the caller's RNG.
//    Thresholds are found by a bitwise search over an order-preserving integer key of the logits, so no
//    sort and no scratch memory is needed; ties at a threshold are all kept (the reference's
//    partial_sort keeps an arbitrary subset of them).  All reductions use fixed trees: the same logits
//    and u always give the same token.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    int t = threadIdx.x < (kThreads >> 5) ? smem[threadIdx.x] : 0;
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) smem[0] = t;
    }
    __syncthreads();
    return smem[0];
}

__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += kThreads) {
        const float v = row[i];
        if (bi == 0x7fffffff || v > best) { best = v; bi = i; }
    }
    auto better = [](float v, int i, float w, int j) { return (w > v) || (w == v && j < i); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, best, o);
        const int j = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(best, bi, w, j)) { best = w; bi = j; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = sval[lane];
        bi = sidx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, best, o);
            const int j = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(best, bi, w, j)) { best = w; bi = j; }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

__global__ void repeat_penalty_kernel(float* __restrict__ logits, const int32_t* __restrict__ tokens,
                                      const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                                      const float* __restrict__ penalty, int V) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x;
    const float pen = penalty[r];
    if (pen == 1.0f) return;
    float* row = logits + (size_t)r * V;
    for (int i = offsets[r] + threadIdx.x; i < offsets[r + 1]; i += blockDim.x) {
        const int tok = tokens[i];
        if (tok < 0 || tok >= V) continue;
        float v = row[tok];
        for (int c = 0; c < counts[i]; ++c) v = v > 0.f ? v / pen : v * pen;
        row[tok] = v;   // tokens are unique within a row, so no two threads touch one logit
    }
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ u,
              int32_t* __restrict__ out, int V) {
    __shared__ float fred[32];
    __shared__ int ired[32];
    __shared__ float wsum[kThreads / 32];
    __shared__ int s_first, s_last;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * V;
    const float inv_t = 1.0f / temperature[r];

    float mx = -INFINITY;
    for (int i = tid; i < V; i += kThreads) mx = fmaxf(mx, row[i]);
    mx = forge::block_max(mx, fred);

    // weight of the kept set {key >= thr}
    auto mass_ge = [&](uint32_t thr) {
        float s = 0.f;
        for (int i = tid; i < V; i += kThreads) {
            const float l = row[i];
            if (order_key(l) >= thr) s += expf((l - mx) * inv_t);
        }
        return forge::block_sum(s, fred);
    };

    uint32_t thr = 0;
    const int k = top_k[r];
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = thr | (1u << bit);
            int c = 0;
            for (int i = tid; i < V; i += kThreads) c += order_key(row[i]) >= cand;
            if (block_sum_int(c, ired) >= k) thr = cand;
        }
    }
    float total = mass_ge(thr);
    const float p = top_p[r];
    if (p < 1.0f) {
        const float need = p * total;
        uint32_t t2 = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = t2 | (1u << bit);
            if (cand <= thr || mass_ge(cand > thr ? cand : thr) > need) t2 = cand;
        }
        if (t2 > thr) thr = t2;
        total = mass_ge(thr);
    }

    // first index whose running kept weight reaches u * total; each thread owns a contiguous chunk
    const float target = u[r] * total;
    const int chunk = (V + kThreads - 1) / kThreads;
    const int lo = min(tid * chunk, V), hi = min(lo + chunk, V);
    float local = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float l = row[i];
        if (order_key(l) >= thr) { local += expf((l - mx) * inv_t); last_kept = i; }
    }
    // exclusive scan of `local` over threads: warp scan, then scan of warp totals
    const int lane = tid & 31, warp = tid >> 5;
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (tid == 0) { s_first = kThreads; s_last = -1; }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = wsum[lane], acc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, acc, o);
            if (lane >= o) acc += v;
        }
        wsum[lane] = acc - w;   // exclusive prefix of warp totals
    }
    __syncthreads();
    const float excl = wsum[warp] + incl - local;
    if (last_kept >= 0) {
        atomicMax(&s_last, last_kept);
        if (excl + local >= target) atomicMin(&s_first, tid);
    }
    __syncthreads();
    if (s_first == kThreads) {          // rounding left the target just above the total
        if (tid == 0) out[r] = s_last < 0 ? 0 : s_last;
        return;
    }
    if (tid == s_first) {
        float c = excl;
        int pick = last_kept;
        for (int i = lo; i < hi; ++i) {
            const float l = row[i];
            if (order_key(l) >= thr) {
                c += expf((l - mx) * inv_t);
                if (c >= target) { pick = i; break; }
            }
        }
        out[r] = pick;
    }
}

}  // namespace

extern "C" int forge_argmax(const float* logits, int32_t* out, int R, int V, cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "argmax: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    return forge::check_launch("argmax", forge::launch(argmax_kernel, dim3(R), dim3(kThreads), 0, stream, 1, logits, out, V));
}

extern "C" int forge_repeat_penalty(float* logits, const int32_t* tokens, const int32_t* counts,
                                    const int32_t* offsets, const float* penalty, int R, int V,
                                    cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "repeat_penalty: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    return forge::check_launch("repeat_penalty", forge::launch(repeat_penalty_kernel, dim3(R), dim3(256), 0, stream, 1, logits, tokens, counts, offsets, penalty, V));
}

// temperature[r] must be > 0 (the caller routes temperature <= 0 to forge_argmax).
extern "C" int forge_sample(const float* logits, const float* temperature, const int32_t* top_k,
                            const float* top_p, const float* u, int32_t* out, int R, int V,
                            cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "sample: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    return forge::check_launch("sample", forge::launch(sample_kernel, dim3(R), dim3(kThreads), 0, stream, 1, logits, temperature, top_k, top_p, u, out, V));
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
