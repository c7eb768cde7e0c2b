// Paged causal grouped-query attention on the tensor cores (bf16 operands, fp32 softmax and accumulation),
// for portions of prompts and for decode tokens alike.
//
// A CTA works on one (request, kv head, tile of up to 64 query rows, slice of the keys).  A query row is a
// (token of the step, query head of this kv head's group) pair: row r <-> token r / G, head r % G with
// G = NH / NKV, so the G heads that share a kv head also share every K/V tile that is loaded.  Each warp
// owns 16 rows; a decode token (G <= 16 rows) is one warp.  Keys and values are fetched page by page
// through the request's block table with cp.async into double-buffered shared memory (rows padded by 16
// bytes: conflict-free ldmatrix for every head size that is a multiple of 16), scores and outputs come
// from mma.sync.m16n8k16, the softmax runs online in fp32 in the exp2 domain.
//   s_j = (q . k_j) / sqrt(HD) for keys max(0, p - window + 1) <= j <= p of the row's position p;
//   o = sum_j softmax(s)_j v_j          (formulas of src/operators/cuda/cuda_flash_attn.cu:154-248, 297-439)
// With num_splits > 1 the key range of a tile is cut into slices handled by different CTAs that write
// unnormalised partial results (o, running max, running sum) to scratch memory; a second kernel merges
// them.  That is how a single decode token with a long context fills the GPU.
#include <initializer_list>
#include <mma.h>

#include "attention_no_alloc.h"
#include "common.cuh"
#include "checks.cuh"
#include "mma_sync.cuh"

#ifndef FORGE_ATT_HD
#define FORGE_ATT_HD 64
#endif

namespace {

using namespace mma_sync;
constexpr int HD = FORGE_ATT_HD;

constexpr int BQ = 64;
constexpr int LD = HD + 8;                    // padded row length in shared memory (bf16 elements)
constexpr int CPR = HD / 8;                   // 16-byte chunks per row
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");

struct AttnParams {
    const __nv_bfloat16* q;       // [T, NH*HD]
    const __nv_bfloat16* kv;      // [pages, 2, NKV, page_size, HD]
    __nv_bfloat16* out;           // [T, NH*HD]
    float* part_o;                // [tiles, NKV, splits, part_rows, HD]   (num_splits > 1)
    float* part_ml;               // [tiles, NKV, splits, part_rows, 2]
    const int32_t* block_table;   // [S, max_pages]
    const int32_t* tile_req;      // [tiles] request row of each query tile
    const int32_t* tile_row0;     // [tiles] first query row (token * G + head) of the tile within its request
    const int32_t* q_start;       // [S+1]
    const int32_t* ctx_before;    // [S]
    int NH, NKV, page_size, max_pages, window, num_splits, part_rows;
    float scale_log2;
};

// Loads keys/values of token indices [t0, t0+BKV) of the request into one shared-memory buffer; rows
// outside [lo, hi) are zero-filled (their scores are masked and their values must not be NaN).
// Each lane first finds the cache row (page * 2 * NKV + kvh) * page_size + slot of tile rows `lane` and
// `lane + 32` through the block table; the copy loop then gets a row's index by shuffle, so the table is
// read once per row and not once per 16-byte chunk.
template <int BKV>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const AttnParams& p,
                                             const int32_t* table, int kvh, int t0, int lo, int hi) {
    const int lane = threadIdx.x & 31;
    int ridx[(BKV + 31) / 32];
#pragma unroll
    for (int i = 0; i < (BKV + 31) / 32; ++i) {
        const int t = t0 + lane + 32 * i;
        ridx[i] = -1;
        if (lane + 32 * i < BKV && t >= lo && t < hi) {
            const int page = table[t / p.page_size];
            if (FORGE_PAGE_OK(page)) ridx[i] = (page * 2 * p.NKV + kvh) * p.page_size + t % p.page_size;      // (checks build) else: zeros
        }
    }
    const int v_rows = p.NKV * p.page_size;                 // a page's values follow its keys
#pragma unroll 4
    for (int c = threadIdx.x; c < BKV * CPR; c += blockDim.x) {
        const int row = c / CPR, ch = c % CPR;
        int r = __shfl_sync(0xffffffffu, ridx[0], row & 31);
        if (BKV > 32) {
            const int r1 = __shfl_sync(0xffffffffu, ridx[(BKV + 31) / 32 - 1], row & 31);
            r = row < 32 ? r : r1;
        }
        __nv_bfloat16* kd = ks + row * LD + ch * 8;
        __nv_bfloat16* vd = vs + row * LD + ch * 8;
        if (r >= 0) {
            const __nv_bfloat16* kp = p.kv + (size_t)r * HD + ch * 8;
            cp_async16(kd, kp);
            cp_async16(vd, kp + (size_t)v_rows * HD);
        } else {
            *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
        }
    }
}

// BKV: keys per iteration; QROWS: query rows staged per CTA (64: four warps of 16 rows, portions of
// prompts; 16: one warp, decode tokens, where small buffers let many CTAs share an SM).
template <int BKV, int QROWS>
__global__ void __launch_bounds__(QROWS * 2)
paged_attention_mma_kernel(const AttnParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [QROWS][LD]
    __nv_bfloat16* ks = qs + QROWS * LD;                                 // [2][BKV][LD]
    __nv_bfloat16* vs = ks + 2 * BKV * LD;                               // [2][BKV][LD]

    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.NH / p.NKV;
    const int s = p.tile_req[tile], row0 = p.tile_row0[tile];
    const int qs0 = p.q_start[s], qlen = p.q_start[s + 1] - qs0, ctx = p.ctx_before[s];
    const int rows_here = min(BQ, qlen * G - row0);
    const int32_t* table = p.block_table + (size_t)s * p.max_pages;

    // key range of this tile and of this CTA's slice of it (slices are counted in tiles of 64 keys whatever
    // BKV is, so that the slicing does not depend on which instantiation runs)
    const int pos_lo = ctx + row0 / G, pos_hi = ctx + (row0 + rows_here - 1) / G;
    const int kv_hi = pos_hi + 1;
    const int kv_lo = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    const int t_begin = kv_lo / 64, t_end = (kv_hi + 63) / 64;
    const int per_split = (t_end - t_begin + p.num_splits - 1) / p.num_splits;
    const int my_begin = (t_begin + split * per_split) * (64 / BKV);
    const int my_end = min((t_begin + (split + 1) * per_split) * (64 / BKV), (kv_hi + BKV - 1) / BKV);

    // this thread's two rows (of the warp's 16): r_a = lane/4, r_b = r_a + 8
    const int wrow = warp * 16;
    const bool warp_active = wrow < rows_here;
    const int ra = row0 + wrow + (lane >> 2), rb = ra + 8;
    const int pos_a = ctx + ra / G, pos_b = ctx + rb / G;
    const bool valid_a = wrow + (lane >> 2) < rows_here, valid_b = wrow + (lane >> 2) + 8 < rows_here;
    // positions of the warp's first row and of its last valid row: a key tile wholly at or below the first
    // and wholly inside the window of the last needs no per-element mask
    const int wpos_first = ctx + (row0 + wrow) / G;
    const int wpos_last = ctx + (row0 + min(wrow + 15, rows_here - 1)) / G;

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    if (my_begin < my_end) {
        // stage the query tile: row r -> token r / G, head kvh * G + r % G
        for (int c = threadIdx.x; c < QROWS * CPR; c += blockDim.x) {
            const int row = c / CPR, ch = c % CPR;
            __nv_bfloat16* dst = qs + row * LD + ch * 8;
            if (row < rows_here) {
                const int r = row0 + row;
                cp_async16(dst, p.q + (size_t)(qs0 + r / G) * p.NH * HD + (size_t)(kvh * G + r % G) * HD + ch * 8);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        load_kv_tile<BKV>(ks, vs, p, table, kvh, my_begin * BKV, kv_lo, kv_hi);
        cp_async_commit();

        for (int t = my_begin; t < my_end; ++t) {
            const int buf = (t - my_begin) & 1;
            if (t + 1 < my_end) {
                load_kv_tile<BKV>(ks + (buf ^ 1) * BKV * LD, vs + (buf ^ 1) * BKV * LD, p, table, kvh, (t + 1) * BKV, kv_lo, kv_hi);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            if (warp_active) {
                const __nv_bfloat16* kb = ks + buf * BKV * LD;
                const __nv_bfloat16* vb = vs + buf * BKV * LD;
                float sc[BKV / 8][4];
#pragma unroll
                for (int i = 0; i < BKV / 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    uint32_t a[4];
                    ldmatrix_x4(a, qs + (wrow + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int nb = 0; nb < BKV / 16; ++nb) {
                        uint32_t b[4];
                        ldmatrix_x4(b, kb + (nb * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                        mma_bf16(sc[2 * nb], a, b[0], b[1]);
                        mma_bf16(sc[2 * nb + 1], a, b[2], b[3]);
                    }
                }
                // scale, mask, online softmax (exp2 domain)
                float mx_a = m_a, mx_b = m_b;
                const bool unmasked = t * BKV + BKV - 1 <= wpos_first && (p.window <= 0 || t * BKV > wpos_last - p.window);
                if (unmasked) {
#pragma unroll
                    for (int i = 0; i < BKV / 8; ++i) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc[i][e] *= p.scale_log2;
                        mx_a = fmaxf(mx_a, fmaxf(sc[i][0], sc[i][1]));
                        mx_b = fmaxf(mx_b, fmaxf(sc[i][2], sc[i][3]));
                    }
                } else {
                    const int j0 = t * BKV + 2 * (lane & 3);
#pragma unroll
                    for (int i = 0; i < BKV / 8; ++i) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int j = j0 + i * 8 + e;
                            const bool va = valid_a && j <= pos_a && (p.window <= 0 || j > pos_a - p.window);
                            const bool vb2 = valid_b && j <= pos_b && (p.window <= 0 || j > pos_b - p.window);
                            sc[i][e] = va ? sc[i][e] * p.scale_log2 : -INFINITY;
                            sc[i][2 + e] = vb2 ? sc[i][2 + e] * p.scale_log2 : -INFINITY;
                            mx_a = fmaxf(mx_a, sc[i][e]);
                            mx_b = fmaxf(mx_b, sc[i][2 + e]);
                        }
                    }
                }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                // a row that has seen no visible key yet keeps max -inf: use 0 as the reference so exp2 gives 0
                const float ref_a = mx_a == -INFINITY ? 0.f : mx_a, ref_b = mx_b == -INFINITY ? 0.f : mx_b;
                const float alpha_a = ex2_approx(m_a - ref_a), alpha_b = ex2_approx(m_b - ref_b);
                m_a = mx_a;
                m_b = mx_b;
                float sum_a = 0.f, sum_b = 0.f;
                uint32_t pfrag[BKV / 16][4];
#pragma unroll
                for (int i = 0; i < BKV / 8; ++i) {
                    const float p0 = ex2_approx(sc[i][0] - ref_a), p1 = ex2_approx(sc[i][1] - ref_a);
                    const float p2 = ex2_approx(sc[i][2] - ref_b), p3 = ex2_approx(sc[i][3] - ref_b);
                    sum_a += p0 + p1;
                    sum_b += p2 + p3;
                    pfrag[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
                    pfrag[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
                }
                l_a = l_a * alpha_a + sum_a;
                l_b = l_b * alpha_b + sum_b;
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    o_acc[i][0] *= alpha_a; o_acc[i][1] *= alpha_a;
                    o_acc[i][2] *= alpha_b; o_acc[i][3] *= alpha_b;
                }
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
                    for (int db = 0; db < HD / 16; ++db) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, vb + (kk * 16 + (lane & 15)) * LD + db * 16 + (lane >> 4) * 8);
                        mma_bf16(o_acc[2 * db], pfrag[kk], b[0], b[1]);
                        mma_bf16(o_acc[2 * db + 1], pfrag[kk], b[2], b[3]);
                    }
                }
            }
            __syncthreads();     // the buffer just read is the target of the next iteration's loads
        }
    }

    if (!warp_active) return;
    // row sums live spread over the 4 lanes of a row
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const int d0 = 2 * (lane & 3);
    if (p.num_splits == 1) {
        const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            if (valid_a)
                *reinterpret_cast<uint32_t*>(p.out + (size_t)(qs0 + ra / G) * p.NH * HD + (size_t)(kvh * G + ra % G) * HD + i * 8 + d0) =
                    pack_bf16(o_acc[i][0] * inv_a, o_acc[i][1] * inv_a);
            if (valid_b)
                *reinterpret_cast<uint32_t*>(p.out + (size_t)(qs0 + rb / G) * p.NH * HD + (size_t)(kvh * G + rb % G) * HD + i * 8 + d0) =
                    pack_bf16(o_acc[i][2] * inv_b, o_acc[i][3] * inv_b);
        }
    } else {
        const size_t slot = ((size_t)tile * p.NKV + kvh) * p.num_splits + split;
        float* po = p.part_o + slot * p.part_rows * HD;
        float* pml = p.part_ml + slot * p.part_rows * 2;
        const int la = wrow + (lane >> 2), lb = la + 8;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            if (valid_a) *reinterpret_cast<float2*>(po + la * HD + i * 8 + d0) = make_float2(o_acc[i][0], o_acc[i][1]);
            if (valid_b) *reinterpret_cast<float2*>(po + lb * HD + i * 8 + d0) = make_float2(o_acc[i][2], o_acc[i][3]);
        }
        if ((lane & 3) == 0) {
            if (valid_a) { pml[la * 2] = m_a; pml[la * 2 + 1] = l_a; }
            if (valid_b) { pml[lb * 2] = m_b; pml[lb * 2 + 1] = l_b; }
        }
    }
}

// One CTA of 1 to 8 warps per (tile, kv head, row) and 32 columns of the head: combines the slices' partial results.
// The slices are dealt to the CTA's threads (thread t takes slices t, t + threads, ...: with hundreds of slices, a
// long context spread over the whole GPU, a single warp walking them one after the other took 40 us).  A thread asks
// for its first slice's maximum, sum AND 32 columns at once, before the row's reference maximum is known (only the
// weights need it), so the kernel is one trip to L2 and two meetings of the CTA.  Every thread adds its slices'
// weighted results in index order, the lanes of a warp are summed by a butterfly and the warps in warp order: the
// order of additions is fixed, so the result does not depend on timing.
constexpr int kMergeWarps = 8;
__global__ void __launch_bounds__(32 * kMergeWarps)
attention_merge_kernel(const AttnParams p, int num_tiles) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    __shared__ float red_m[kMergeWarps], red_l[kMergeWarps], red_o[kMergeWarps][32];
    const int G = p.NH / p.NKV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5, threads = blockDim.x;
    const int PR = p.part_rows, S = p.num_splits;
    const int gw = blockIdx.x, c0 = blockIdx.y * 32;             // gw < num_tiles * NKV * PR by the launch
    const int row = gw % PR, kvh = (gw / PR) % p.NKV, tile = gw / (PR * p.NKV);
    const int s = p.tile_req[tile], row0 = p.tile_row0[tile];
    const int qs0 = p.q_start[s], qlen = p.q_start[s + 1] - qs0;
    if (tile >= num_tiles || row0 + row >= qlen * G) return;     // the same for every thread of the CTA
    const size_t slot0 = ((size_t)tile * p.NKV + kvh) * S;
    const float* ml = p.part_ml + (slot0 * PR + row) * 2;        // slice z: ml[z * PR * 2], + 1
    const float* po = p.part_o + (slot0 * PR + row) * HD + c0;   // slice z: po[z * PR * HD]
    // columns c0 .. c0 + 31 of slice z (the head size is a multiple of 16: whole float4s); a slice without a visible
    // key (maximum -inf) never wrote its partial result and counts as zeros
    auto load_cols = [&](int z, float m_z, float4 (&v)[8]) {
        const float4* src = reinterpret_cast<const float4*>(po + (size_t)z * PR * HD);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = (m_z != -INFINITY && c0 + 4 * i < HD) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    const int z_first = threadIdx.x;
    float m_first = -INFINITY, l_first = 0.f;
    float4 v_first[8];
    if (z_first < S) {
        m_first = ml[(size_t)z_first * PR * 2];
        l_first = ml[(size_t)z_first * PR * 2 + 1];
    }
    load_cols(z_first < S ? z_first : 0, m_first, v_first);
    // the row's reference: the largest of the slices' running maxima
    float M = m_first;
    for (int z = z_first + threads; z < S; z += threads) M = fmaxf(M, ml[(size_t)z * PR * 2]);
    M = forge::warp_max(M);
    if (lane == 0) red_m[warp] = M;
    __syncthreads();
    M = red_m[0];
    for (int w = 1; w < warps; ++w) M = fmaxf(M, red_m[w]);
    float acc[32];
    const float w_first = m_first == -INFINITY ? 0.f : exp2f(m_first - M);
    float L = w_first * l_first;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc[4 * i] = w_first * v_first[i].x; acc[4 * i + 1] = w_first * v_first[i].y;
        acc[4 * i + 2] = w_first * v_first[i].z; acc[4 * i + 3] = w_first * v_first[i].w;
    }
    for (int z = z_first + threads; z < S; z += threads) {       // more slices than threads: the rest, in index order
        const float m_z = ml[(size_t)z * PR * 2];
        if (m_z == -INFINITY) continue;
        const float w = exp2f(m_z - M);
        L += w * ml[(size_t)z * PR * 2 + 1];
        float4 v[8];
        load_cols(z, m_z, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[4 * i] += w * v[i].x; acc[4 * i + 1] += w * v[i].y; acc[4 * i + 2] += w * v[i].z; acc[4 * i + 3] += w * v[i].w;
        }
    }
    L = forge::warp_sum(L);
    if (lane == 0) red_l[warp] = L;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float t = forge::warp_sum(acc[i]);
        if (lane == i) red_o[warp][i] = t;
    }
    __syncthreads();
    if (threadIdx.x < 32 && c0 + threadIdx.x < HD) {
        float Lsum = red_l[0], v = red_o[0][threadIdx.x];
        for (int w = 1; w < warps; ++w) { Lsum += red_l[w]; v += red_o[w][threadIdx.x]; }
        const float inv = Lsum > 0.f ? 1.0f / Lsum : 0.f;
        const int r = row0 + row;
        p.out[(size_t)(qs0 + r / G) * p.NH * HD + (size_t)(kvh * G + r % G) * HD + c0 + threadIdx.x] = __float2bfloat16_rn(v * inv);
    }
}

// ---------------------------------------------------------------------------------------------------
// Decode step in one kernel: position encoding, cache write and attention of ONE new token per request.
//
// A CTA serves one (request, kv head).  It rotates the G query heads and the key head of the new token
// (fp32 angles, as rope_cache.cu does), writes the key and the value into the request's page, and attends
// over the request's keys: the key range is dealt to the CTA's warps in tiles of 32 keys (warp w takes
// tiles w, w + W, ...), each warp keeps an online softmax of its own over its tiles, and the warps' partial
// results are merged through shared memory in warp order.  One launch replaces three (rope + cache write,
// sliced attention, merge) and no partial result leaves the SM.
struct DecodeParams {
    const float* qkv;             // [S, (NH + 2 NKV) * HD] fp32: the new token's projections, one row per request
    __nv_bfloat16* kv;            // [pages, 2, NKV, page_size, HD]
    __nv_bfloat16* out;           // [S, NH*HD]
    const int32_t* block_table;   // [S, max_pages]
    const int32_t* positions;     // [S] position of the new token = tokens already cached
    const int32_t* slot_mapping;  // [S] page * page_size + offset of the new token
    int NH, NKV, page_size, max_pages, window, rotary;
    float theta, scale_log2;
    int ksplit;                   // CTAs of a cluster that share one (request, kv head) and deal its key tiles out
};

constexpr int DKV = 32;           // keys per tile

__device__ __forceinline__ uint32_t att_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void att_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float att_ld_peer(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int NWARPS, bool CLUSTER>
__global__ void __launch_bounds__(NWARPS * 32)
decode_attention_fused_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [16][LD]  (G heads, zero-padded)
    __nv_bfloat16* kvs = qs + 16 * LD;                                   // [NWARPS][2 buffers][K | V][DKV][LD]
    forge::pdl_launch_dependents();
    // ksplit CTAs (a cluster) share a (request, kv head): the key tiles go round all their warps, each CTA merges
    // its warps' results, and CTA 0 of the cluster merges the CTAs' through distributed shared memory.
    const int KS = CLUSTER ? p.ksplit : 1;             // without a cluster everything below folds to the one-CTA form
    const int rank = CLUSTER ? static_cast<int>(att_cluster_rank()) : 0;
    const int s = blockIdx.x / KS, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vwarp = rank * NWARPS + warp, vwarps = NWARPS * KS;        // this warp among all warps of the cluster
    const int G = p.NH / p.NKV;
    // The step's positions, slots and block tables were written before its first kernel started, and the keys
    // and values of earlier positions in earlier steps: all of that may be read before the dependency wait,
    // which only orders this kernel after the product that makes q, k and v.
    const int pos = p.positions[s];
    const int half = HD / 2;
    const float* row = p.qkv + (size_t)s * (p.NH + 2 * p.NKV) * HD;
    const int slot = p.slot_mapping[s];
    __nv_bfloat16* page_base = p.kv + ((size_t)(slot / p.page_size) * 2 * p.NKV + kvh) * p.page_size * HD + (size_t)(slot % p.page_size) * HD;

    const int32_t* table = p.block_table + (size_t)s * p.max_pages;
    const int kv_hi = pos + 1;
    const int kv_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int t_begin = kv_lo / DKV, t_end = (kv_hi + DKV - 1) / DKV;
    __nv_bfloat16* my_k = kvs + (size_t)warp * 4 * DKV * LD;             // [buffer][K | V]

    auto load_tile = [&](int buf, int t) {
        __nv_bfloat16* kd = my_k + (size_t)buf * 2 * DKV * LD;
        const int tk = t * DKV + lane;                                   // lane = row of the tile
        int ridx = -1;
        if (tk >= kv_lo && tk < kv_hi) {
            const int page = table[tk / p.page_size];
            if (FORGE_PAGE_OK(page)) ridx = (page * 2 * p.NKV + kvh) * p.page_size + tk % p.page_size;
        }
        const int v_rows = p.NKV * p.page_size;
#pragma unroll 4
        for (int c = lane; c < DKV * CPR; c += 32) {
            const int r_row = c / CPR, ch = c % CPR;
            const int r = __shfl_sync(0xffffffffu, ridx, r_row);
            __nv_bfloat16* dk = kd + r_row * LD + ch * 8;
            __nv_bfloat16* dv = dk + DKV * LD;
            if (r >= 0) {
                const __nv_bfloat16* src = p.kv + (size_t)r * HD + ch * 8;
                cp_async16(dk, src);
                cp_async16(dv, src + (size_t)v_rows * HD);
            } else {
                *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    // 0. this warp's first two tiles are requested now if they hold only earlier positions (the tile with the
    // new token is read after this kernel has written the token's key and value)
    int issued = 0;                                                      // tiles of this warp requested so far
    for (; issued < 2; ++issued) {
        const int t = t_begin + vwarp + issued * vwarps;
        if (t >= t_end - 1) break;
        load_tile(issued, t);
        cp_async_commit();
    }
    // the CTA whose warp gets the tile with the new token is the one that writes the token's key and value
    const bool writes_kv = ((t_end - 1 - t_begin) % vwarps) / NWARPS == rank;
    // the angles of the rotation depend on the position only: a thread's first few are computed here, while the
    // product that makes q, k and v still runs (powf and sincosf are some hundred instructions each).  Measured with
    // heads of 64: batch 8 +0.7 %, batch 1 +1.6 %; with heads of 128 (and in the kernel that streams the cache) the
    // registers held across the wait cost 1 to 3 %, so there the angles are computed where they are used.
    constexpr int kAnglesAhead = HD <= 64 ? 4 : 0;
    float cs_pre[kAnglesAhead > 0 ? kAnglesAhead : 1], sn_pre[kAnglesAhead > 0 ? kAnglesAhead : 1];
#pragma unroll
    for (int a = 0; a < kAnglesAhead; ++a) {
        const int i = threadIdx.x + a * blockDim.x;
        cs_pre[a] = 1.0f;
        sn_pre[a] = 0.0f;
        if (p.rotary && i < (G + 1) * half) {
            const float freq = 1.0f / powf(p.theta, (2.0f * (float)(i % half)) / (float)HD);
            sincosf((float)pos * freq, &sn_pre[a], &cs_pre[a]);
        }
    }
    forge::pdl_wait();

    // 1. rotate q (G heads) and k (one head), copy v; q to shared memory, k and v to the cache
    for (int i = threadIdx.x; i < 16 * CPR; i += blockDim.x)             // clear the padding rows of Q
        if (i / CPR >= G) *reinterpret_cast<uint4*>(qs + (i / CPR) * LD + (i % CPR) * 8) = make_uint4(0, 0, 0, 0);
    for (int a = 0, i = threadIdx.x; i < (G + 2) * half; ++a, i += blockDim.x) {
        const int h = i / half, d = i % half;                            // h < G: q head; G: k; G + 1: v
        const int src_head = h < G ? kvh * G + h : (h == G ? p.NH + kvh : p.NH + p.NKV + kvh);
        float x0 = row[src_head * HD + d], x1 = row[src_head * HD + d + half];
        if (p.rotary && h <= G) {
            float sn, cs;
            if (a < kAnglesAhead) {
                constexpr int k1 = kAnglesAhead > 1 ? 1 : 0, k2 = kAnglesAhead > 2 ? 2 : 0, k3 = kAnglesAhead > 3 ? 3 : 0;
                cs = a == 0 ? cs_pre[0] : (a == 1 ? cs_pre[k1] : (a == 2 ? cs_pre[k2] : cs_pre[k3]));
                sn = a == 0 ? sn_pre[0] : (a == 1 ? sn_pre[k1] : (a == 2 ? sn_pre[k2] : sn_pre[k3]));
            } else {
                const float freq = 1.0f / powf(p.theta, (2.0f * (float)d) / (float)HD);
                sincosf((float)pos * freq, &sn, &cs);
            }
            const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
            x0 = y0;
            x1 = y1;
        }
        if (h < G) {
            qs[h * LD + d] = __float2bfloat16_rn(x0);
            qs[h * LD + d + half] = __float2bfloat16_rn(x1);
        } else if (writes_kv && FORGE_SLOT_OK(slot)) {
            __nv_bfloat16* dst = page_base + (h == G ? 0 : (size_t)p.NKV * p.page_size * HD);
            dst[d] = __float2bfloat16_rn(x0);
            dst[d + half] = __float2bfloat16_rn(x1);
        }
    }
    __threadfence_block();        // the new key and value are read back below by whichever warp gets their tile
    __syncthreads();

    // 2. every warp walks its share of the key tiles
    const bool valid_a = (lane >> 2) < G, valid_b = (lane >> 2) + 8 < G;

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    int n_done = 0;
    for (int t = t_begin + vwarp; t < t_end; t += vwarps, ++n_done) {
        const int buf = n_done & 1;
        // tile n_done and, if there is one, the tile after it are on their way before this one is waited for
        for (; issued < n_done + 2 && t_begin + vwarp + issued * vwarps < t_end; ++issued) {
            load_tile(issued & 1, t_begin + vwarp + issued * vwarps);
            cp_async_commit();
        }
        if (issued == n_done + 2) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncwarp();
        const __nv_bfloat16* kb = my_k + (size_t)buf * 2 * DKV * LD;
        const __nv_bfloat16* vb = kb + DKV * LD;
        float sc[DKV / 8][4];
#pragma unroll
        for (int i = 0; i < DKV / 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < DKV / 16; ++nb) {
                uint32_t b[4];
                ldmatrix_x4(b, kb + (nb * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(sc[2 * nb], a, b[0], b[1]);
                mma_bf16(sc[2 * nb + 1], a, b[2], b[3]);
            }
        }
        float mx_a = m_a, mx_b = m_b;
        const bool unmasked = t * DKV + DKV - 1 <= pos && (p.window <= 0 || t * DKV > pos - p.window);
        const int j0 = t * DKV + 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < DKV / 8; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + i * 8 + e;
                const bool vis = unmasked || (j <= pos && (p.window <= 0 || j > pos - p.window));
                sc[i][e] = (vis && valid_a) ? sc[i][e] * p.scale_log2 : -INFINITY;
                sc[i][2 + e] = (vis && valid_b) ? sc[i][2 + e] * p.scale_log2 : -INFINITY;
                mx_a = fmaxf(mx_a, sc[i][e]);
                mx_b = fmaxf(mx_b, sc[i][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float ref_a = mx_a == -INFINITY ? 0.f : mx_a, ref_b = mx_b == -INFINITY ? 0.f : mx_b;
        const float alpha_a = ex2_approx(m_a - ref_a), alpha_b = ex2_approx(m_b - ref_b);
        m_a = mx_a;
        m_b = mx_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pfrag[DKV / 16][4];
#pragma unroll
        for (int i = 0; i < DKV / 8; ++i) {
            const float p0 = ex2_approx(sc[i][0] - ref_a), p1 = ex2_approx(sc[i][1] - ref_a);
            const float p2 = ex2_approx(sc[i][2] - ref_b), p3 = ex2_approx(sc[i][3] - ref_b);
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            pfrag[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
            pfrag[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * alpha_a + sum_a;
        l_b = l_b * alpha_b + sum_b;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o_acc[i][0] *= alpha_a; o_acc[i][1] *= alpha_a;
            o_acc[i][2] *= alpha_b; o_acc[i][3] *= alpha_b;
        }
#pragma unroll
        for (int kk = 0; kk < DKV / 16; ++kk) {
#pragma unroll
            for (int db = 0; db < HD / 16; ++db) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vb + (kk * 16 + (lane & 15)) * LD + db * 16 + (lane >> 4) * 8);
                mma_bf16(o_acc[2 * db], pfrag[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * db + 1], pfrag[kk], b[2], b[3]);
            }
        }
        __syncwarp();            // the buffer just read is the target of the load after next
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // 3. merge the warps' partial results in shared memory (the tile buffers are free now), in warp order
    __syncthreads();
    float* mo = reinterpret_cast<float*>(kvs);                           // [NWARPS][16][HD]
    float* ml = mo + NWARPS * 16 * HD;                                   // [NWARPS][16][2]
    {
        const int ra = lane >> 2, rb = ra + 8, d0 = 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + ra) * HD + i * 8 + d0) = make_float2(o_acc[i][0], o_acc[i][1]);
            *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + rb) * HD + i * 8 + d0) = make_float2(o_acc[i][2], o_acc[i][3]);
        }
        if ((lane & 3) == 0) {
            ml[(warp * 16 + ra) * 2] = m_a; ml[(warp * 16 + ra) * 2 + 1] = l_a;
            ml[(warp * 16 + rb) * 2] = m_b; ml[(warp * 16 + rb) * 2 + 1] = l_b;
        }
    }
    __syncthreads();
    float* cta_o = ml + NWARPS * 16 * 2;                                 // [16][HD] this CTA's un-normalised output
    float* cta_ml = cta_o + 16 * HD;                                     // [16][2]  its maximum and sum
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int r = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, ml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = ml[(w * 16 + r) * 2];
            const float wt = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += wt * ml[(w * 16 + r) * 2 + 1];
            acc += wt * mo[((size_t)w * 16 + r) * HD + d];
        }
        if (!CLUSTER) {
            p.out[(size_t)s * p.NH * HD + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            cta_o[r * HD + d] = acc;
            if (d == 0) { cta_ml[r * 2] = M; cta_ml[r * 2 + 1] = L; }
        }
    }
    if (CLUSTER) {
        // 4. the cluster's CTAs, in rank order, by CTA 0
        att_cluster_sync();
        if (rank == 0) {
            for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
                const int r = i / HD, d = i % HD;
                float M = -INFINITY;
                for (int q = 0; q < KS; ++q) M = fmaxf(M, att_ld_peer(cta_ml + r * 2, q));
                float L = 0.f, acc = 0.f;
                for (int q = 0; q < KS; ++q) {
                    const float mq = att_ld_peer(cta_ml + r * 2, q);
                    const float wt = mq == -INFINITY ? 0.f : exp2f(mq - M);
                    L += wt * att_ld_peer(cta_ml + r * 2 + 1, q);
                    acc += wt * att_ld_peer(cta_o + r * HD + d, q);
                }
                p.out[(size_t)s * p.NH * HD + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            }
        }
        att_cluster_sync();                  // nobody leaves while CTA 0 may still read its shared memory
    }
}

}  // namespace

// Scratch floats needed for num_splits > 1, with R = 16 if max_rows <= 16 else 64:
//   part_o = tiles*NKV*splits*R*HD, part_ml = tiles*NKV*splits*R*2.
// max_rows: the largest number of query rows (tokens * G) of any tile, which sets the CTA size (1..4 warps).
extern "C" int forge_paged_attention_mma(const void* q, const void* kv, void* out, float* part_o, float* part_ml,
                                         const int32_t* block_table, const int32_t* tile_req, const int32_t* tile_row0,
                                         const int32_t* q_start, const int32_t* ctx_before, int num_tiles, int max_rows,
                                         int NH, int NKV, int head_dim, int page_size, int max_pages, int window,
                                         int num_splits, float scale, cudaStream_t stream) {
    if (head_dim != HD) return forge::fail(FORGE_ERR_UNSUPPORTED, "this attention library was built for head_dim %d, got %d", HD, head_dim);
    if (num_tiles < 0 || NH <= 0 || NKV <= 0 || NH % NKV != 0 || page_size <= 0 || max_pages <= 0 || num_splits < 1 ||
        max_rows < 1 || max_rows > BQ)
        return forge::fail(FORGE_ERR_ARG, "paged_attention_mma: bad sizes tiles=%d NH=%d NKV=%d page=%d splits=%d rows=%d",
                           num_tiles, NH, NKV, page_size, num_splits, max_rows);
    if (num_tiles == 0) return FORGE_OK;
    if (num_splits > 1 && (!part_o || !part_ml)) return forge::fail(FORGE_ERR_ARG, "paged_attention_mma: splits need scratch");
    if (NKV > 65535 || num_splits > 65535) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_mma: grid too large");
    AttnParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)kv, (__nv_bfloat16*)out, part_o, part_ml, block_table,
                 tile_req, tile_row0, q_start, ctx_before, NH, NKV, page_size, max_pages, window, num_splits,
                 max_rows <= 16 ? 16 : BQ, scale * 1.4426950408889634f};
    // one warp of rows (decode tokens): small buffers, many CTAs per SM; otherwise four warps and 64-key tiles
    constexpr int smem_big = (64 + 4 * 64) * LD * 2, smem_small = (16 + 4 * 32) * LD * 2;
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_mma_kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_big);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(paged_attention_mma_kernel<32, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_small);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_mma: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaError_t le;
    if (max_rows <= 16)
        le = forge::launch(paged_attention_mma_kernel<32, 16>, dim3(num_tiles, NKV, num_splits), dim3(32), smem_small, stream, 1, p);
    else
        le = forge::launch(paged_attention_mma_kernel<64, 64>, dim3(num_tiles, NKV, num_splits),
                           dim3(32 * ((max_rows + 15) / 16)), smem_big, stream, 1, p);
    int rc = forge::check_launch("paged_attention_mma", le);
    if (rc != FORGE_OK || num_splits == 1) return rc;
    const long rows = (long)num_tiles * NKV * p.part_rows;
    const int merge_warps = num_splits >= 32 * kMergeWarps ? kMergeWarps : (num_splits + 31) / 32;     // a thread per slice, up to eight warps
    return forge::check_launch("attention_merge", forge::launch(attention_merge_kernel, dim3((unsigned)rows, (HD + 31) / 32),
                                                                dim3(32 * merge_warps), 0, stream, 1, p, num_tiles));
}

// ---------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_no_alloc.h): same kernels, scratch in a static array.
namespace {

static __device__ __align__(256) float g_static_scratch[FORGE_ATT_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_scratch_addr[kMaxDevices] = {nullptr};

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address of
// the array on the CURRENT device has to be asked for, once per device.
int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_mma_static: cannot tell the current device (%s)",
                           e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_mma_static: cudaGetSymbolAddress failed: %s",
                               cudaGetErrorString(e));
        g_static_scratch_addr[dev] = static_cast<float*>(ptr);
    }
    *out = g_static_scratch_addr[dev];
    return FORGE_OK;
}

}  // namespace

extern "C" int forge_paged_attention_mma_static(const void* q, const void* kv, void* out, const int32_t* block_table,
                                                const int32_t* tile_req, const int32_t* tile_row0,
                                                const int32_t* q_start, const int32_t* ctx_before, int num_tiles,
                                                int max_rows, int NH, int NKV, int head_dim, int page_size,
                                                int max_pages, int window, int num_splits, float scale,
                                                cudaStream_t stream) {
    if (num_tiles < 0 || NKV <= 0 || num_splits < 1 || max_rows < 1 || max_rows > BQ)
        return forge::fail(FORGE_ERR_ARG, "paged_attention_mma_static: bad sizes tiles=%d NKV=%d splits=%d rows=%d",
                           num_tiles, NKV, num_splits, max_rows);
    // with one slice the kernel writes its result straight to `out`: no scratch, nothing to fit, nothing to look up
    if (num_splits == 1)
        return forge_paged_attention_mma(q, kv, out, nullptr, nullptr, block_table, tile_req, tile_row0, q_start, ctx_before,
                                         num_tiles, max_rows, NH, NKV, head_dim, page_size, max_pages, window, 1, scale, stream);
    // the need is a product of four factors; each partial product is held against the array's size before the
    // next factor comes in, so that no product wraps round and slips under the limit
    constexpr unsigned long long kFloats = FORGE_ATT_STATIC_SCRATCH_FLOATS;
    unsigned long long rows = (unsigned long long)(max_rows <= 16 ? 16 : BQ);
    bool fits = true;
    for (unsigned long long factor : {(unsigned long long)num_tiles, (unsigned long long)NKV, (unsigned long long)num_splits}) {
        if (factor != 0 && rows > kFloats / factor) { fits = false; break; }
        rows *= factor;
    }
    if (!fits || rows * (HD + 2) > kFloats)
        return forge::fail(FORGE_ERR_UNSUPPORTED,
                           "paged_attention_mma_static: tiles %d x kv heads %d x slices %d x %d rows x %d scratch floats needed, "
                           "the built-in array holds %u; use fewer slices or forge_paged_attention_mma with your own scratch",
                           num_tiles, NKV, num_splits, max_rows <= 16 ? 16 : BQ, HD + 2, FORGE_ATT_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != FORGE_OK) return rc;
    // partial outputs first (rows * HD floats, a multiple of 16 floats), then the (max, sum) pairs
    return forge_paged_attention_mma(q, kv, out, scratch, scratch + rows * HD, block_table, tile_req, tile_row0, q_start,
                                     ctx_before, num_tiles, max_rows, NH, NKV, head_dim, page_size, max_pages, window,
                                     num_splits, scale, stream);
}

// One new token per request: rotary encoding (rotary != 0), cache write and attention in one launch.
// qkv fp32 [S, (NH + 2 NKV) * HD]; positions / slot_mapping int32 [S]; out bf16 [S, NH*HD].  NH / NKV <= 16.
extern "C" int forge_decode_attention_fused(const float* qkv, void* kv, void* out, const int32_t* block_table,
                                            const int32_t* positions, const int32_t* slot_mapping, int S, int NH, int NKV,
                                            int head_dim, int page_size, int max_pages, int window, int rotary,
                                            float theta, float scale, int max_context, cudaStream_t stream) {
    // max_context: an upper bound of the requests' cached tokens + 1 (0: unknown); it only steers how many CTAs
    // share a request's keys
    if (head_dim != HD) return forge::fail(FORGE_ERR_UNSUPPORTED, "this attention library was built for head_dim %d, got %d", HD, head_dim);
    if (S < 0 || NH <= 0 || NKV <= 0 || NH % NKV != 0 || page_size <= 0 || max_pages <= 0 || NKV > 65535)
        return forge::fail(FORGE_ERR_ARG, "decode_attention_fused: bad sizes S=%d NH=%d NKV=%d page=%d", S, NH, NKV, page_size);
    if (NH / NKV > 16) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_fused: %d query heads per kv head (at most 16)", NH / NKV);
    if (S == 0) return FORGE_OK;
    DecodeParams p{qkv, (__nv_bfloat16*)kv, (__nv_bfloat16*)out, block_table, positions, slot_mapping, NH, NKV, page_size,
                   max_pages, window, rotary, theta, scale * 1.4426950408889634f, 1};
    // eight warps while the CTAs are few (short latency per request), four when there are CTAs enough to fill the SMs
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    constexpr int kLimit = 227 * 1024;
    constexpr int need4 = (16 + 4 * 4 * DKV) * LD * 2, need8 = (16 + 8 * 4 * DKV) * LD * 2;   // tiles; the merge area is smaller
    if (need4 > kLimit) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_fused: head_dim %d needs %d bytes of shared memory", HD, need4);
    const int warps = ((long)S * NKV <= sms && need8 <= kLimit) ? 8 : 4;
    const int smem = warps == 8 ? need8 : need4;
    // while SMs are idle, 2 or 4 CTAs (a cluster) share a request's keys, as long as every warp keeps four tiles:
    // the cluster's hand-shakes cost about 1.4 us, which two tiles per warp do not pay back (measured at 8
    // requests: 640 cached tokens 0.837 -> 0.868 ms per step with 2 CTAs, 6,000 tokens 1.72 -> 1.10 ms with 4)
    // (a single request, 4 CTAs, gains from 4-way splitting already at 1,500 tokens: 0.88 -> 0.82 ms; below 64
    // tiles nothing gains)
    if (warps == 8 && max_context > 0) {
        const long tiles = (max_context + DKV - 1) / DKV, keep = (long)S * NKV >= 16 ? 4 : 2;
        while (tiles >= 64 && p.ksplit < 4 && (long)S * NKV * p.ksplit * 2 <= sms && tiles >= keep * warps * p.ksplit * 2) p.ksplit *= 2;
    }
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_fused_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, need4);
        if (e == cudaSuccess && need8 <= kLimit)
            e = cudaFuncSetAttribute(decode_attention_fused_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, need8);
        if (e == cudaSuccess && need8 <= kLimit)
            e = cudaFuncSetAttribute(decode_attention_fused_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, need8);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "decode_attention_fused: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaError_t le;
    if (p.ksplit > 1) le = forge::launch(decode_attention_fused_kernel<8, true>, dim3(S * p.ksplit, NKV), dim3(256), smem, stream, p.ksplit, p);
    else if (warps == 8) le = forge::launch(decode_attention_fused_kernel<8, false>, dim3(S, NKV), dim3(256), smem, stream, 1, p);
    else le = forge::launch(decode_attention_fused_kernel<4, false>, dim3(S, NKV), dim3(128), smem, stream, 1, p);
    return forge::check_launch("decode_attention_fused", le);
}

extern "C" int forge_attention_head_dim() { return HD; }
// (checks build) the bounds that this library's kernels test page ids and slots against
FORGE_DEFINE_CHECKS_ENTRY(attention_mma)
extern "C" const char* forge_last_error() { return forge::error_buffer(); }
