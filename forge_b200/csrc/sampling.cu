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
//    Thresholds are found by a search, four bits at a time, over an order-preserving integer key of the
//    logits, so no sort and no scratch memory is needed; ties at a threshold are all kept (the reference's
//    partial_sort keeps an arbitrary subset of them).  All sums have a fixed order: the same logits and u
//    always give the same token.
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

// Temperature / top-k / top-p selection of one row per thread block.  The k-th largest key is found four bits at a
// time (8 histograms of 16 bins, counters packed four to a word); with top-k the few kept entries are gathered (in index
// order, by a scan, so every sum below has a fixed order) and top-p is decided among them: its threshold is the largest
// kept key whose tail weight exceeds p of the kept weight; without top-k the same threshold is found a digit at a time
// from per-bin weights.  A vocabulary of up to 49,152 entries has its keys read once into shared memory (SMEM); larger
// ones are walked in global memory (L2) once per digit.  (A first version searched both thresholds bit by bit, 66 walks
// and block-wide sums for top-k with top-p: 170 us for 8 rows of 32,000 against 48 us now.)
constexpr int kMaxSmemKeys = 49152;
constexpr int kListCap = 2048;
#define KEY_AT(i) ((i) + ((i) >> 5))

// The repeat penalty from a history that lives on the device: counts [slots, V] holds, per request slot, how often
// each token was generated; a row's logits are penalised once per occurrence, as in repeat_penalty_kernel.  With the
// history on the device a step's tokens can be drawn, and the next step launched, before the host has seen them.
__global__ void history_penalty_kernel(float* __restrict__ logits, const int32_t* __restrict__ counts,
                                       const int32_t* __restrict__ slot_of_row, const float* __restrict__ penalty, int V) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.y;
    const float pen = penalty[r];
    if (pen == 1.0f) return;
    const int32_t* hist = counts + (size_t)slot_of_row[r] * V;
    float* row = logits + (size_t)r * V;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
        const int c = hist[i];
        if (c > 0) {
            float v = row[i];
            for (int k = 0; k < c; ++k) v = v > 0.f ? v / pen : v * pen;
            row[i] = v;
        }
    }
}

// counts[slot of row r][tokens[r]] += 1 for the rows whose requests have a penalty (one thread per row).
__global__ void history_add_kernel(int32_t* __restrict__ counts, const int32_t* __restrict__ slot_of_row,
                                   const int32_t* __restrict__ tokens, const float* __restrict__ penalty, int R, int V) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R || penalty[r] == 1.0f) return;
    const int t = tokens[r];
    if (t >= 0 && t < V) counts[(size_t)slot_of_row[r] * V + t] += 1;      // a slot belongs to one row of a step
}

template <bool SMEM>
__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ u,
              int32_t* __restrict__ out, int V) {
    // [V] order keys of the row, one unused word after every 32: a thread that walks a contiguous chunk of 32 keys
    // (the gathering and the draw below) would otherwise hit one bank with all its lanes
    extern __shared__ uint32_t s_key[];
    __shared__ float fred[32];
    __shared__ int ired[32];
    __shared__ int hist_w[kThreads / 32][16];
    __shared__ int hist[16];
    __shared__ float mass_w[kThreads / 32][16];
    __shared__ float mass[16];
    __shared__ float wsum[kThreads / 32];
    __shared__ int s_first, s_last;
    __shared__ uint32_t list_key[kListCap];
    __shared__ float list_w[kListCap];
    __shared__ int iscan[kThreads / 32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * V;
    const float inv_t = 1.0f / temperature[r];

    float mx = -INFINITY;
    for (int i = tid; i < V; i += kThreads) {
        const float l = row[i];
        mx = fmaxf(mx, l);
        if (SMEM) s_key[KEY_AT(i)] = order_key(l);
    }
    mx = forge::block_max(mx, fred);                       // (its barriers also publish the keys)
    auto key_at = [&](int i) -> uint32_t { return SMEM ? s_key[KEY_AT(i)] : order_key(row[i]); };
    auto weight_of = [&](uint32_t key) {                   // the entry's weight from its key (the key maps back to the logit)
        const uint32_t bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
        return expf((__uint_as_float(bits) - mx) * inv_t);
    };
    auto mass_ge = [&](uint32_t thr) {
        float sum = 0.f;
        for (int i = tid; i < V; i += kThreads)
            { const uint32_t key = key_at(i); if (key >= thr) sum += weight_of(key); }
        return forge::block_sum(sum, fred);
    };

    uint32_t thr = 0;
    const int k = top_k[r];
    const bool with_k = k > 0 && k < V;
    if (with_k) {
        // the k-th largest key, a hexadecimal digit at a time from the top
        int remaining = k;
        uint32_t prefix = 0;
        for (int shift = 28; shift >= 0; shift -= 4) {
            // sixteen counters of 16 bits in four words (a thread counts at most 48 keys, a block 49,152)
            unsigned long long h[4] = {0ull, 0ull, 0ull, 0ull};
            const uint32_t high_mask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
            for (int i = tid; i < V; i += kThreads) {
                const uint32_t key = key_at(i);
                if ((key & high_mask) == (prefix & high_mask)) {
                    const int d = (key >> shift) & 15;
                    const unsigned long long one = 1ull << (16 * (d & 3));
#pragma unroll
                    for (int q = 0; q < 4; ++q) h[q] += (d >> 2) == q ? one : 0ull;
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                unsigned long long v = h[q];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) hist_w[warp][4 * q + e] = (int)((v >> (16 * e)) & 0xffffull);
                }
            }
            __syncthreads();
            if (tid < 16) {
                int t = 0;
                for (int w = 0; w < kThreads / 32; ++w) t += hist_w[w][tid];
                hist[tid] = t;
            }
            __syncthreads();
            for (int d = 15; d >= 0; --d) {
                const int c = hist[d];
                if (c >= remaining) { prefix |= (uint32_t)d << shift; break; }
                remaining -= c;
            }
            __syncthreads();                              // hist is rewritten in the next round
        }
        thr = prefix;
    }
    float total = 0.f;
    const float p = top_p[r];
    bool decided = false;
    if (p < 1.0f && with_k) {
        // gather the kept entries in index order: a count per thread over its contiguous chunk, a scan of the counts
        const int chunk = (V + kThreads - 1) / kThreads;
        const int lo = min(tid * chunk, V), hi = min(lo + chunk, V);
        int mine = 0;
        for (int i = lo; i < hi; ++i) mine += key_at(i) >= thr;
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) iscan[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int w = iscan[lane];
            int acc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, acc, o);
                if (lane >= o) acc += v;
            }
            iscan[lane] = acc - w;
            if (lane == 31) ired[0] = acc;                // how many are kept
        }
        __syncthreads();
        const int n = ired[0];
        if (n <= kListCap) {
            int pos = iscan[warp] + incl - mine;
            for (int i = lo; i < hi; ++i) {
                const uint32_t key = key_at(i);
                if (key >= thr) { list_key[pos] = key; list_w[pos] = weight_of(key); ++pos; }
            }
            __syncthreads();
            float all = 0.f;
            for (int j = 0; j < n; ++j) all += list_w[j];  // every thread the same sum in the same order
            const float need = p * all;
            // the largest kept key whose tail (the weights of keys at least as large) exceeds p of the kept weight
            uint32_t best = 0;
            for (int i = tid; i < n; i += kThreads) {
                const uint32_t key = list_key[i];
                float tail = 0.f;
                for (int j = 0; j < n; ++j) tail += list_key[j] >= key ? list_w[j] : 0.f;
                if (tail > need && key > best) best = key;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
            __syncthreads();
            if (lane == 0) ired[warp] = (int)best;
            __syncthreads();
            if (warp == 0) {
                uint32_t t = (uint32_t)ired[lane];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t = max(t, __shfl_xor_sync(0xffffffffu, t, o));
                if (lane == 0) ired[0] = (int)t;
            }
            __syncthreads();
            const uint32_t t2 = (uint32_t)ired[0];
            if (t2 > thr) thr = t2;
            decided = true;
            __syncthreads();
        }
    }
    if (p < 1.0f && !decided) {
        // no top-k (or too many ties to gather): the largest threshold whose tail weight exceeds p of the kept weight,
        // a hexadecimal digit at a time: per digit the weight of the keys that share the digits found so far, by bin
        total = mass_ge(thr);
        const float need = p * total;
        uint32_t prefix = 0;
        float above = 0.f;                                 // weight of the keys above every key that shares the prefix
        for (int shift = 28; shift >= 0; shift -= 4) {
            float m[16];
#pragma unroll
            for (int d = 0; d < 16; ++d) m[d] = 0.f;
            const uint32_t high_mask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
            for (int i = tid; i < V; i += kThreads) {
                const uint32_t key = key_at(i);
                if (key >= thr && (key & high_mask) == (prefix & high_mask)) {
                    const int d = (key >> shift) & 15;
                    const float w = weight_of(key);
#pragma unroll
                    for (int q = 0; q < 16; ++q) m[q] += d == q ? w : 0.f;
                }
            }
#pragma unroll
            for (int d = 0; d < 16; ++d) {
                float v = m[d];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) mass_w[warp][d] = v;
            }
            __syncthreads();
            if (tid < 16) {
                float t = 0.f;
                for (int w = 0; w < kThreads / 32; ++w) t += mass_w[w][tid];
                mass[tid] = t;
            }
            __syncthreads();
            float tail = above;
            int d = 15;
            for (; d > 0; --d) {
                if (tail + mass[d] > need) break;          // the threshold lies among the keys with this digit
                tail += mass[d];
            }
            prefix |= (uint32_t)d << shift;
            above = tail;
            __syncthreads();                              // mass is rewritten in the next round
        }
        if (prefix > thr) thr = prefix;
    }
    total = mass_ge(thr);

    // first index whose running kept weight reaches u * total; each thread owns a contiguous chunk
    const float target = u[r] * total;
    const int chunk = (V + kThreads - 1) / kThreads;
    const int lo = min(tid * chunk, V), hi = min(lo + chunk, V);
    float local = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = key_at(i);
        if (key >= thr) { local += weight_of(key); last_kept = i; }
    }
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
            const uint32_t key = key_at(i);
            if (key >= thr) {
                c += weight_of(key);
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

// counts int32 [slots, V]; slot_of_row int32 [R]; penalty fp32 [R] (1 = none).
extern "C" int forge_history_penalty(float* logits, const int32_t* counts, const int32_t* slot_of_row, const float* penalty,
                                     int R, int V, cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "history_penalty: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    return forge::check_launch("history_penalty", forge::launch(history_penalty_kernel, dim3((V + 1023) / 1024, R), dim3(256), 0, stream, 1,
                                                                logits, counts, slot_of_row, penalty, V));
}

extern "C" int forge_history_add(int32_t* counts, const int32_t* slot_of_row, const int32_t* tokens, const float* penalty,
                                 int R, int V, cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "history_add: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    return forge::check_launch("history_add", forge::launch(history_add_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, 1,
                                                            counts, slot_of_row, tokens, penalty, R, V));
}

// temperature[r] must be > 0 (the caller routes temperature <= 0 to forge_argmax).
extern "C" int forge_sample(const float* logits, const float* temperature, const int32_t* top_k,
                            const float* top_p, const float* u, int32_t* out, int R, int V,
                            cudaStream_t stream) {
    if (R < 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "sample: bad sizes R=%d V=%d", R, V);
    if (R == 0) return FORGE_OK;
    if (V <= kMaxSmemKeys) {
        static forge::PerDeviceFlag configured_on;
        bool& configured = configured_on.current();
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (kMaxSmemKeys + kMaxSmemKeys / 32 + 1) * 4);
            if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "sample: %s", cudaGetErrorString(e));
            configured = true;
        }
        return forge::check_launch("sample", forge::launch(sample_kernel<true>, dim3(R), dim3(kThreads), (size_t)(V + V / 32 + 1) * 4, stream, 1, logits,
                                                           temperature, top_k, top_p, u, out, V));
    }
    return forge::check_launch("sample", forge::launch(sample_kernel<false>, dim3(R), dim3(kThreads), 0, stream, 1, logits, temperature, top_k, top_p, u, out, V));
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
