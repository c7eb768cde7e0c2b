// Paged causal grouped-query attention on the CUDA cores, fp32 arithmetic throughout.
//
// One warp per (token, query head).  A token of request r at position p attends to the keys of r at
// positions max(0, p - window + 1) .. p, read from the paged cache through r's block table, in order,
// with an online softmax:  s_j = (q . k_j) / sqrt(HD);  o = sum_j softmax(s)_j v_j
// (formulas of src/operators/cuda/cuda_flash_attn.cu:154-248 and :297-439; kv head = q head / (NH/NKV)).
// Because a token's keys are always walked in the same order, its result does not depend on how the
// request was cut into steps or on what else is in the batch.  This kernel serves the true 32-bit path
// and any shape the tensor-core kernel refuses: any HD <= 256, any NH/NKV ratio, any page size.
#include "common.cuh"
#include "checks.cuh"

namespace {

template <int DPL, typename T>  // DPL = dims per lane = ceil(HD / 32)
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ kv_cache,
                            const int32_t* __restrict__ block_table, const int32_t* __restrict__ tok_req,
                            const int32_t* __restrict__ positions, T* __restrict__ out, int T_tokens, int NH,
                            int NKV, int HD, int page_size, int max_pages, int window, float scale) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int warp_global = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (warp_global >= T_tokens * NH) return;
    const int t = warp_global / NH, h = warp_global % NH;
    const int kvh = h / (NH / NKV);
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)tok_req[t] * max_pages;
    if (!FORGE_TOKEN_OK(t)) return;

    float qr[DPL], acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < HD ? forge::to_float(q[(size_t)t * NH * HD + h * HD + d]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    int j = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    while (j <= pos) {
        const int page_idx = j / page_size, off0 = j % page_size;
        const int page = table[page_idx];
        const int n_here = min(page_size - off0, pos - j + 1);
        if (!FORGE_PAGE_OK(page)) { j += n_here; continue; }          // (checks build) a page outside the pool is skipped
        const T* kp = kv_cache + (((size_t)page * 2 + 0) * NKV + kvh) * page_size * HD;
        const T* vp = kv_cache + (((size_t)page * 2 + 1) * NKV + kvh) * page_size * HD;
        for (int o = off0; o < off0 + n_here; ++o) {
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < HD) part = fmaf(qr[i], forge::to_float(kp[(size_t)o * HD + d]), part);
            }
            const float s = forge::warp_sum(part);
            const float m_new = fmaxf(m, s);
            const float alpha = expf(m - m_new);   // expf(-inf) = 0 on the first key
            const float p = expf(s - m_new);
            l = l * alpha + p;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                const float v = d < HD ? forge::to_float(vp[(size_t)o * HD + d]) : 0.f;
                acc[i] = fmaf(p, v, acc[i] * alpha);
            }
            m = m_new;
        }
        j += n_here;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < HD) out[(size_t)t * NH * HD + h * HD + d] = forge::from_float<T>(acc[i] * inv);
    }
}

template <typename T>
int launch(const void* q, const void* kv, const int32_t* bt, const int32_t* tok_req, const int32_t* positions,
           void* out, int T_tokens, int NH, int NKV, int HD, int page_size, int max_pages, int window,
           float scale, cudaStream_t stream) {
    const int warps = T_tokens * NH;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    const int dpl = (HD + 31) / 32;
    cudaError_t e = cudaSuccess;
#define FORGE_ATT_CASE(D)                                                                                  \
    case D:                                                                                                \
        e = forge::launch(paged_attention_simt_kernel<D, T>, dim3(blocks), dim3(128), 0, stream, 1,        \
            (const T*)q, (const T*)kv, bt, tok_req, positions, (T*)out, T_tokens, NH, NKV, HD, page_size,  \
            max_pages, window, scale);                                                                     \
        break;
    switch (dpl) {
        FORGE_ATT_CASE(1) FORGE_ATT_CASE(2) FORGE_ATT_CASE(3) FORGE_ATT_CASE(4)
        FORGE_ATT_CASE(5) FORGE_ATT_CASE(6) FORGE_ATT_CASE(7) FORGE_ATT_CASE(8)
        default: return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_simt: head_dim %d > 256", HD);
    }
#undef FORGE_ATT_CASE
    return forge::check_launch("paged_attention_simt", e);
}

}  // namespace

// window <= 0 means all keys.  scale is normally 1/sqrt(HD).
extern "C" int forge_paged_attention_simt(const void* q, const void* kv_cache, const int32_t* block_table,
                                          const int32_t* tok_req, const int32_t* positions, void* out, int dtype,
                                          int T, int NH, int NKV, int HD, int page_size, int max_pages, int window,
                                          float scale, cudaStream_t stream) {
    if (T < 0 || NH <= 0 || NKV <= 0 || HD <= 0 || page_size <= 0 || max_pages <= 0 || NH % NKV != 0)
        return forge::fail(FORGE_ERR_ARG, "paged_attention_simt: bad sizes T=%d NH=%d NKV=%d HD=%d page=%d max_pages=%d",
                           T, NH, NKV, HD, page_size, max_pages);
    if (T == 0) return FORGE_OK;
    if ((long long)T * NH > 0x7fffffffLL / 2) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_simt: T*NH too large");
    if (dtype == FORGE_F32) return launch<float>(q, kv_cache, block_table, tok_req, positions, out, T, NH, NKV, HD, page_size, max_pages, window, scale, stream);
    if (dtype == FORGE_BF16) return launch<__nv_bfloat16>(q, kv_cache, block_table, tok_req, positions, out, T, NH, NKV, HD, page_size, max_pages, window, scale, stream);
    return forge::fail(FORGE_ERR_ARG, "paged_attention_simt: unknown dtype %d", dtype);
}

// (checks build) the bounds that this file's kernel tests page ids and token indices against
FORGE_DEFINE_CHECKS_ENTRY(attention_simt)
