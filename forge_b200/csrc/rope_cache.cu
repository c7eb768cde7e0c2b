// Rotary position encoding of q and k fused with the write of k and v into the paged cache.
//
// Input is the fp32 result of the fused QKV projection, [T, (NH + 2*NKV) * HD] (q heads, then k heads,
// then v heads).  The rotation is the reference's half-split form (src/operators/cuda/cuda_rope.cu:8-34):
//   freq_d = 1 / powf(theta, 2d/HD),  a = pos * freq_d  (fp32),
//   (x[d], x[d+HD/2]) <- (x[d] cos a - x[d+HD/2] sin a,  x[d] sin a + x[d+HD/2] cos a)
// with full-precision powf/sincosf.  q is stored as [T, NH*HD] in the activation type; k (rotated) and
// v go to the slot slot_mapping[t] = page * page_size + offset of a cache laid out as
// [num_pages, 2 (k,v), NKV, page_size, HD].  A negative slot skips the cache write (layers that read
// another layer's cache).  `rotary == 0` copies without rotating (a model without rotary encoding).
#include "common.cuh"
#include "checks.cuh"

namespace {

// cos/sin of every (token, pair) of a step: the angles depend on the position and the pair only, so one small
// kernel per step serves every head of every layer.  table[t, d] = (cos, sin) of positions[t] / theta^(2d/HD); with
// `by_pair` the table is laid out [d, t] instead, for a reader whose neighbouring threads hold neighbouring tokens.
__global__ void rope_table_kernel(const int32_t* __restrict__ positions, float2* __restrict__ table, int T, int HD, float theta,
                                  int by_pair) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x, half = HD >> 1;
    if (i >= T * half) return;
    const int t = by_pair ? i % T : i / half, d = by_pair ? i / T : i % half;
    const float freq = 1.0f / powf(theta, (2.0f * (float)d) / (float)HD);
    float s, c;
    sincosf((float)positions[t] * freq, &s, &c);
    table[i] = make_float2(c, s);
}

// One thread per pair (d, d + HD/2) of one head of one token: q and k heads are rotated, v heads copied.
// `table` (optional): the step's cos/sin from rope_table_kernel; without it the angles are computed here.
template <typename TAct, typename TCache>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ positions,
                     const int32_t* __restrict__ slot_mapping, TAct* __restrict__ q_out,
                     TCache* __restrict__ kv_cache, int NH, int NKV, int HD, int page_size,
                     float theta, int rotary, const float2* __restrict__ table) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const int half = HD >> 1;
    const int w = blockIdx.y * blockDim.x + threadIdx.x;
    if (w >= (NH + 2 * NKV) * half) return;
    const int h = w / half, d = w % half;
    const float* row = qkv + (size_t)t * (NH + 2 * NKV) * HD;
    float x0 = row[h * HD + d], x1 = row[h * HD + d + half];
    if (rotary && h < NH + NKV) {
        float s, c;
        if (table) {
            const float2 cs = table[(size_t)t * half + d];
            c = cs.x;
            s = cs.y;
        } else {
            const float freq = 1.0f / powf(theta, (2.0f * (float)d) / (float)HD);
            sincosf((float)positions[t] * freq, &s, &c);
        }
        const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
        x0 = y0;
        x1 = y1;
    }
    if (h < NH) {
        TAct* q = q_out + (size_t)t * NH * HD + h * HD;
        q[d] = forge::from_float<TAct>(x0);
        q[d + half] = forge::from_float<TAct>(x1);
        return;
    }
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot < 0 || !FORGE_SLOT_OK(slot)) return;
    const int page = slot / page_size, off = slot % page_size;
    const int is_v = h >= NH + NKV, kvh = h - NH - (is_v ? NKV : 0);
    TCache* dst = kv_cache + (((size_t)page * 2 + is_v) * NKV + kvh) * page_size * HD + (size_t)off * HD;
    dst[d] = forge::from_float<TCache>(x0);
    dst[d + half] = forge::from_float<TCache>(x1);
}

template <typename T> struct Store4;
template <> struct Store4<float> {
    static __device__ __forceinline__ void put(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Store4<__nv_bfloat16> {
    static __device__ __forceinline__ void put(__nv_bfloat16* p, const float (&v)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
};

// The same for head sizes that are a multiple of 8: a thread takes four neighbouring pairs of one head (two
// float4 loads, two 8- or 16-byte stores); a CTA takes kTokens tokens so that prompts do not launch one small
// CTA per token and 128 pairs.  Needs the step's cos/sin table.
constexpr int kRopeTokens = 4;
template <typename TAct, typename TCache>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ slot_mapping, TAct* __restrict__ q_out,
                         TCache* __restrict__ kv_cache, int T, int NH, int NKV, int HD, int page_size, int rotary,
                         const float2* __restrict__ table) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int half = HD >> 1, quads = half >> 2;                   // quads of pairs per head
    const int per_token = (NH + 2 * NKV) * quads;
    for (int i = threadIdx.x; i < kRopeTokens * per_token; i += blockDim.x) {
        const int t = blockIdx.x * kRopeTokens + i / per_token;
        if (t >= T) break;
        const int wq = i % per_token, h = wq / quads, d = (wq % quads) * 4;
        const float* row = qkv + (size_t)t * (NH + 2 * NKV) * HD + h * HD;
        const float4 a = *reinterpret_cast<const float4*>(row + d), b = *reinterpret_cast<const float4*>(row + d + half);
        float x0[4] = {a.x, a.y, a.z, a.w}, x1[4] = {b.x, b.y, b.z, b.w};
        if (rotary && h < NH + NKV) {
            const float4* cs = reinterpret_cast<const float4*>(table + (size_t)t * half + d);     // (c, s, c, s) x 2
            const float4 cs01 = cs[0], cs23 = cs[1];
            const float c[4] = {cs01.x, cs01.z, cs23.x, cs23.z}, sn[4] = {cs01.y, cs01.w, cs23.y, cs23.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float y0 = x0[j] * c[j] - x1[j] * sn[j], y1 = x0[j] * sn[j] + x1[j] * c[j];
                x0[j] = y0;
                x1[j] = y1;
            }
        }
        if (h < NH) {
            TAct* q = q_out + (size_t)t * NH * HD + h * HD;
            Store4<TAct>::put(q + d, x0);
            Store4<TAct>::put(q + d + half, x1);
            continue;
        }
        const int slot = slot_mapping ? slot_mapping[t] : -1;
        if (slot < 0 || !FORGE_SLOT_OK(slot)) continue;
        const int page = slot / page_size, off = slot % page_size;
        const int is_v = h >= NH + NKV, kvh = h - NH - (is_v ? NKV : 0);
        TCache* dst = kv_cache + (((size_t)page * 2 + is_v) * NKV + kvh) * page_size * HD + (size_t)off * HD;
        Store4<TCache>::put(dst + d, x0);
        Store4<TCache>::put(dst + d + half, x1);
    }
}

}  // namespace

// table: float [T, HD/2, 2] (cos, sin) for the step's tokens; by_pair != 0: [HD/2, T, 2].
extern "C" int forge_rope_table(const int32_t* positions, float* table, int T, int HD, float theta, int by_pair, cudaStream_t stream) {
    if (T < 0 || HD <= 0 || (HD & 1)) return forge::fail(FORGE_ERR_ARG, "rope_table: bad sizes T=%d HD=%d", T, HD);
    if (T == 0) return FORGE_OK;
    const long n = (long)T * (HD / 2);
    return forge::check_launch("rope_table", forge::launch(rope_table_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0,
                                                           stream, 1, positions, reinterpret_cast<float2*>(table), T, HD, theta, by_pair));
}

// table: optional cos/sin table from forge_rope_table for the same positions, HD and theta (null: compute here).
extern "C" int forge_rope_kv_write(const float* qkv, const int32_t* positions, const int32_t* slot_mapping,
                                   void* q_out, void* kv_cache, int dtype, int T, int NH, int NKV, int HD,
                                   int page_size, float theta, int rotary, const float* table, cudaStream_t stream) {
    if (T > 2147483647 / 2 || ((NH + 2 * NKV) * (HD / 2) + 127) / 128 > 65535)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "rope_kv_write: too many heads for one launch");
    if (T < 0 || NH <= 0 || NKV <= 0 || HD <= 0 || (HD & 1) || page_size <= 0)
        return forge::fail(FORGE_ERR_ARG, "rope_kv_write: bad sizes T=%d NH=%d NKV=%d HD=%d page=%d (HD must be even)",
                           T, NH, NKV, HD, page_size);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    if ((HD % 8) == 0 && (table != nullptr || !rotary) && T >= kRopeTokens) {
        FORGE_DISPATCH_DTYPE(dtype, TT,
            e = forge::launch(rope_kv_write_vec_kernel<TT, TT>, dim3((T + kRopeTokens - 1) / kRopeTokens), dim3(256), 0, stream, 1,
                              qkv, slot_mapping, (TT*)q_out, (TT*)kv_cache, T, NH, NKV, HD, page_size, rotary,
                              reinterpret_cast<const float2*>(table)));
        return forge::check_launch("rope_kv_write", e);
    }
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(rope_kv_write_kernel<TT, TT>, dim3(T, ((NH + 2 * NKV) * (HD / 2) + 127) / 128), dim3(128), 0, stream, 1,
                          qkv, positions, slot_mapping, (TT*)q_out, (TT*)kv_cache, NH, NKV, HD, page_size, theta, rotary,
                          reinterpret_cast<const float2*>(table)));
    return forge::check_launch("rope_kv_write", e);
}

// (checks build) the bounds that this library's kernels test page ids, slots and token indices against
FORGE_DEFINE_CHECKS_ENTRY(rope)
