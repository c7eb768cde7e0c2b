// Paged causal grouped-query attention for prompt portions on the 5th-generation tensor cores (head size 64).
//
// One CTA = one tile of 128 query rows of one (request, kv head); a row is a (token, head of the kv head's
// group) pair, row r <-> token r / G, head r % G, so a tile is 128 / G tokens and the G heads share every
// key/value tile.  Per tile of 64 keys:
//   S = Q K^T      tcgen05.mma M=128 N=64 K=64, Q and K in shared memory (TMA, 128-byte swizzle), S in TMEM
//   softmax        128 threads, one row each, read S from TMEM, online max/sum in fp32 (exp2 domain), rescale
//                  the output accumulator in TMEM, write P as bf16 into shared memory in the MMA's layout
//   O += P V       tcgen05.mma M=128 N=64 K=64, P K-major, V MN-major (keys are rows of 128 bytes), O in TMEM
// Warp 0 feeds keys and values page by page through the request's block table (one TMA box per page and
// operand, two stages), warp 1 issues the MMAs, warps 2-5 are the softmax rows.  Three such CTAs fit an SM
// (64 KB of shared memory, 128 TMEM columns each), so one CTA's softmax overlaps another's MMAs.
//   s_j = (q . k_j) / sqrt(64) for keys max(0, p - window + 1) <= j <= p of the row's position p;
//   o = sum_j softmax(s)_j v_j        (formulas of src/operators/cuda/cuda_flash_attn.cu:154-248)
// Needs 128 % G == 0, 64 % page_size == 0 and page_size >= 8; everything else is served by attention_mma.cu.
#include "common.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int HD = 64, BQ = 128, BKV = 64, UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kTileBytes = BQ * 128;              // Q or P: 128 rows of 128 bytes
constexpr int kKVBytes = BKV * 128;               // K or V tile: 64 rows of 128 bytes
constexpr int kSmemBytes = kTileBytes * 2 + 4 * kKVBytes + 1024 + 1024;
constexpr int kTmemCols = 128;                    // S: columns 0..63, O: columns 64..127

struct AttnTcParams {
    __nv_bfloat16* out;           // [T, NH*HD]
    const int32_t* block_table;   // [S, max_pages]
    const int32_t* tile_req;      // [tiles]
    const int32_t* tile_row0;     // [tiles] first row (token * G + head) of the tile within its request
    const int32_t* q_start;       // [S+1]
    const int32_t* ctx_before;    // [S]
    int NH, NKV, page_size, max_pages, window;
    float scale_log2;
    int* status;
};

// 2^x by the special-function unit (2 ulp); the weights are rounded to bfloat16 right after
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kThreads, 3)
paged_attention_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                             const AttnTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                               // [128][64] bf16, K-major, swizzled
    uint8_t* p_s = smem + kTileBytes;                  // [128][64 keys] bf16, K-major, swizzled
    uint8_t* kv_s = smem + 2 * kTileBytes;             // [2 stages][K 8 KB | V 8 KB]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kTileBytes + 4 * kKVBytes);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;     // [2]
    uint64_t* kv_empty = bars + 3;    // [2]
    uint64_t* s_full = bars + 5;
    uint64_t* s_free = bars + 6;
    uint64_t* p_ready = bars + 7;
    uint64_t* o_done = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int G = p.NH / p.NKV;

    if (threadIdx.x == 0) {
        *abort = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(s_free, 128);
        mbar_init(p_ready, 128);
        mbar_init(o_done, 1);
        mbar_fence_init();
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_kv);
    }
    // key/value stages start as zeros: pages that are skipped (beyond the request, or released by the
    // window) leave their rows as they are, and those rows must hold finite numbers (their weights are 0)
    for (int i = threadIdx.x; i < 4 * kKVBytes / 16; i += kThreads) reinterpret_cast<uint4*>(kv_s)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    forge::pdl_launch_dependents();
    forge::pdl_wait();

    const int s_req = p.tile_req[tile], row0 = p.tile_row0[tile];
    const int qs0 = p.q_start[s_req], qlen = p.q_start[s_req + 1] - qs0, ctx = p.ctx_before[s_req];
    const int rows_here = min(BQ, qlen * G - row0);
    const int pos_lo = ctx + row0 / G, pos_hi = ctx + (row0 + rows_here - 1) / G;
    const int kv_hi = pos_hi + 1;
    const int kv_lo = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    const int t_begin = kv_lo / BKV, t_end = (kv_hi + BKV - 1) / BKV;
    const int n_iter = t_end - t_begin;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const int32_t* table = p.block_table + (size_t)s_req * p.max_pages;
            mbar_arrive_expect_tx(q_full, kTileBytes);
            tma_load_3d(q_s, &tmap_q, q_full, 0, kvh * G, qs0 + row0 / G);
            const int ppt = BKV / p.page_size;                           // pages per key tile
            const uint32_t page_bytes = p.page_size * 128;
            bool ok = true;
            for (int it = 0; it < n_iter && ok; ++it) {
                const int s = it & 1, t0 = (t_begin + it) * BKV;
                if (!(ok = mbar_wait(&kv_empty[s], ((it >> 1) & 1) ^ 1, abort, p.status, 1))) break;
                int pages[8], n_valid = 0;
                for (int i = 0; i < ppt; ++i) {
                    const int tp = t0 + i * p.page_size;
                    const bool live = tp < kv_hi && tp + p.page_size > kv_lo;
                    pages[i] = live ? table[tp / p.page_size] : -1;
                    n_valid += pages[i] >= 0;
                }
                mbar_arrive_expect_tx(&kv_full[s], n_valid * page_bytes * 2);
                uint8_t* k_dst = kv_s + s * 2 * kKVBytes;
                for (int i = 0; i < ppt; ++i) {
                    if (pages[i] < 0) continue;
                    const int row = (pages[i] * 2 * p.NKV + kvh) * p.page_size;
                    tma_load_2d(k_dst + i * page_bytes, &tmap_kv, &kv_full[s], 0, row);
                    tma_load_2d(k_dst + kKVBytes + i * page_bytes, &tmap_kv, &kv_full[s], 0, row + p.NKV * p.page_size);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(BQ, BKV);
            constexpr uint32_t idesc_pv = umma_idesc_bf16_f32_bmn(BQ, HD);
            const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
            bool ok = mbar_wait(q_full, 0, abort, p.status, 2);
            for (int it = 0; it < n_iter && ok; ++it) {
                const int s = it & 1;
                const uint32_t k_addr = smem_u32(kv_s + s * 2 * kKVBytes), v_addr = k_addr + kKVBytes;
                if (!(ok = mbar_wait(&kv_full[s], (it >> 1) & 1, abort, p.status, 3))) break;
                if (it > 0 && !(ok = mbar_wait(s_free, (it - 1) & 1, abort, p.status, 4))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < HD / UMMA_K; ++k)
                    umma_bf16(tmem_base, umma_desc_k_sw128(q_addr + k * 32), umma_desc_k_sw128(k_addr + k * 32), idesc_qk, k != 0);
                umma_commit(s_full);
                if (!(ok = mbar_wait(p_ready, it & 1, abort, p.status, 5))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < BKV / UMMA_K; ++k)
                    umma_bf16(tmem_base + 64, umma_desc_k_sw128(p_addr + k * 32), umma_desc_mn_sw128(v_addr + k * 2048, 0),
                              idesc_pv, (it | k) != 0);
                umma_commit(&kv_empty[s]);
                umma_commit(o_done);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax rows (warps 2..5)
        const int quarter = warp & 3;
        const int r_local = quarter * 32 + lane;                 // row of the tile = TMEM lane
        const int r = row0 + r_local;
        const bool valid = r_local < rows_here;
        const int pos = ctx + r / G;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint8_t* p_row = p_s + r_local * 128;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_iter && ok; ++it) {
            const int j0 = (t_begin + it) * BKV;
            if (!(ok = mbar_wait(s_full, it & 1, abort, p.status, 6))) break;
            tc_fence_after_sync();
            // rows whose keys of this tile are all visible skip the per-key tests (all tiles but the ones on
            // the diagonal or at the window's edge)
            const bool need_mask = !valid || j0 + BKV - 1 > pos || (p.window > 0 && j0 <= pos - p.window);
            // pass 1: the row's maximum over this tile
            float mx = m;
#pragma unroll
            for (int c = 0; c < BKV; c += 32) {
                uint32_t sv[32];
                tmem_ld_32x32b_x32(t_lane + c, sv);
                tmem_ld_wait();
                if (!need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]) * p.scale_log2);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int j = j0 + c + i;
                        const bool vis = valid && j <= pos && (p.window <= 0 || j > pos - p.window);
                        mx = fmaxf(mx, vis ? __uint_as_float(sv[i]) * p.scale_log2 : -INFINITY);
                    }
                }
            }
            const float ref = mx == -INFINITY ? 0.f : mx;
            const float alpha = ex2_approx(m - ref);
            m = mx;
            // the previous tile's P V must be complete before O is rescaled and P overwritten
            if (it > 0) {
                if (!(ok = mbar_wait(o_done, (it - 1) & 1, abort, p.status, 7))) break;
                tc_fence_after_sync();
                // the accumulator is rescaled only when some row of the warp got a new maximum (the TMEM
                // loads and stores are warp-wide, so the decision is the warp's)
                if (!__all_sync(0xffffffffu, alpha == 1.0f)) {
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t ov[32];
                        tmem_ld_32x32b_x32(t_lane + 64 + c, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                        tmem_st_32x32b_x32(t_lane + 64 + c, ov);
                    }
                    tmem_st_wait();
                }
            }
            // pass 2: weights, their sum, and P in the MMA's shared-memory layout (16-byte chunk ^ row % 8)
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < BKV; c += 32) {
                uint32_t sv[32];
                tmem_ld_32x32b_x32(t_lane + c, sv);
                tmem_ld_wait();
                uint32_t packed[16];
                if (!need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -ref));
                        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -ref));
                        sum += p0 + p1;
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float pr[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int j = j0 + c + i + e;
                            const bool vis = valid && j <= pos && (p.window <= 0 || j > pos - p.window);
                            pr[e] = vis ? ex2_approx(fmaf(__uint_as_float(sv[i + e]), p.scale_log2, -ref)) : 0.f;
                        }
                        sum += pr[0] + pr[1];
                        __nv_bfloat162 h = __floats2bfloat162_rn(pr[0], pr[1]);
                        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c >> 3) + q4;                        // 16-byte chunk of the row: 8 keys
                    *reinterpret_cast<uint4*>(p_row + ((chunk ^ (r_local & 7)) << 4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
            }
            l = l * alpha + sum;
            tc_fence_before_sync();
            mbar_arrive(s_free);                   // S may be overwritten by the next Q K^T
            fence_proxy_async();                   // P is in shared memory for the tensor core to read
            mbar_arrive(p_ready);
        }
        if (ok && n_iter > 0) ok = mbar_wait(o_done, (n_iter - 1) & 1, abort, p.status, 8);
        tc_fence_after_sync();
        if (ok && n_iter > 0) {
            // every lane takes part in the TMEM loads (they are warp-wide instructions); only valid rows store
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = p.out + (size_t)(qs0 + r / G) * p.NH * HD + (size_t)(kvh * G + r % G) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                tmem_ld_32x32b_x32(t_lane + 64 + c, ov);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * e]) * inv, __uint_as_float(ov[i + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

// q [T, NH*64] bf16, kv cache [pages, 2, NKV, page_size, 64] bf16, out [T, NH*64] bf16.  tile_req / tile_row0
// list tiles of 128 query rows (rows = tokens * G); q_start / ctx_before as for forge_paged_attention_mma.
extern "C" int forge_paged_attention_sm100(const void* q, const void* kv, void* out, const int32_t* block_table,
                                           const int32_t* tile_req, const int32_t* tile_row0, const int32_t* q_start,
                                           const int32_t* ctx_before, int* status, int num_tiles, int T, int num_pages,
                                           int NH, int NKV, int head_dim, int page_size, int max_pages, int window,
                                           float scale, cudaStream_t stream) {
    if (head_dim != HD) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: head_dim %d (only 64)", head_dim);
    if (NH <= 0 || NKV <= 0 || NH % NKV != 0 || BQ % (NH / NKV) != 0 || NH / NKV > BQ)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: group size %d/%d must divide 128", NH, NKV);
    if (page_size < 8 || BKV % page_size != 0)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: page size %d must be 8, 16, 32 or 64", page_size);
    if (num_tiles < 0 || T <= 0 || num_pages <= 0 || max_pages <= 0 || NKV > 65535)
        return forge::fail(FORGE_ERR_ARG, "paged_attention_sm100: bad sizes tiles=%d T=%d pages=%d", num_tiles, T, num_pages);
    if (num_tiles == 0) return FORGE_OK;
    const int G = NH / NKV;
    const char* err = nullptr;
    CUtensorMap tq, tkv;
    if (!bf16_q_map(q, T, NH, HD, BQ / G, G, &tq, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: q: %s", err);
    if (!bf16_tile_map(kv, num_pages * 2 * NKV * page_size, HD, page_size, &tkv, &err))
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: cache: %s", err);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_sm100: %s", cudaGetErrorString(e));
        configured = true;
    }
    AttnTcParams p{(__nv_bfloat16*)out, block_table, tile_req, tile_row0, q_start, ctx_before, NH, NKV, page_size,
                   max_pages, window, scale * 1.4426950408889634f, status};
    return forge::check_launch("paged_attention_sm100",
                               forge::launch(paged_attention_sm100_kernel, dim3(num_tiles, NKV), dim3(kThreads), kSmemBytes,
                                             stream, 1, tq, tkv, p));
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
