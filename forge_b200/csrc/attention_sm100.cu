// Paged causal grouped-query attention for prompt portions on the 5th-generation tensor cores (head sizes 64 and
// 128; the library is built per head size, -DFORGE_ATT_HD).
//
// One CTA = one tile of up to 128 query rows of one (request, kv head); a row is a (token, head of the kv head's
// group) pair, row r <-> token r / G, head r % G, so a tile is 128 / G tokens (rounded down: with a group that
// does not divide 128 the last rows of the tile stay empty) and the G heads share every key/value tile.  Per tile
// of 64 keys (HD = head size):
//   S = Q K^T      tcgen05.mma M=128 N=64 K=HD, Q and K in shared memory (TMA, 128-byte swizzle), S in TMEM
//                  (two buffers: the scores of tile it + 2 are computed while the rows work on tile it)
//   softmax        128 threads, one row each, hold the row's 64 scores in registers, online max/sum in fp32
//                  (exp2 domain, packed fp32 arithmetic), write P as bf16 into shared memory in the MMA's
//                  layout (two buffers); the output accumulator in TMEM is rescaled only when a row's
//                  reference exponent has to move (a maximum that grew by more than 2^8)
//   O += P V       tcgen05.mma M=128 N=64 K=64 per 64 columns of the head, P K-major, V MN-major (keys are rows of
//                  128 bytes), O in TMEM
// Warps 0-3 run one thread each: warp 0 feeds keys and values page by page through the request's block table
// (one TMA box per page and operand; key and value tiles have rings of three slots each, keys run ahead),
// warp 1 issues P V, warp 2 issues Q K^T; warps 4-7 are the softmax rows.  The first warpgroup hands most of
// its registers to the second (setmaxnreg).  With head size 64 two such CTAs fit an SM (99 KB of shared memory,
// 256 TMEM columns each); with 128 one does (163 KB).  Tiles are listed longest first and the kv heads of a tile are neighbouring CTAs, so the
// long tiles of all heads start in the first wave.
// A step with fewer tiles than the GPU has places for CTAs (a short portion on a long context) may list a tile several
// times, each entry with a share of the tile's key tiles (``tile_cut``): such a CTA leaves its sums unnormalised in
// fp32 with the row's reference exponent and sum, and a second kernel adds a tile's shares up in the order of the
// shares.
//   s_j = (q . k_j) * scale for keys max(0, p - window + 1) <= j <= p of the row's position p;
//   o = sum_j softmax(s)_j v_j        (formulas of src/operators/cuda/cuda_flash_attn.cu:154-248)
// Needs G <= 128, 64 % page_size == 0 and page_size >= 8; everything else is served by attention_mma.cu.
#include "common.cuh"
#include "checks.cuh"
#include "sm100.cuh"

#ifndef FORGE_ATT_HD
#define FORGE_ATT_HD 64
#endif

namespace {

using namespace sm100;

constexpr int HD = FORGE_ATT_HD, BQ = 128, BKV = 64, UMMA_K = 16;
static_assert(HD == 64 || HD == 128, "head size 64 or 128");
constexpr int KB = HD / 64;                       // 64-wide blocks of the head: Q, K and V tiles are KB swizzled blocks
constexpr int kThreads = 256;                     // warps 0-3: copies, P V, Q K^T, (idle); warps 4-7: the softmax rows
constexpr int kQkWarp = 2;
constexpr int kCtasPerSm = 2;                     // what the register budget is made for (head size 128: one fits, by shared memory)
constexpr int kLaunchRegs = 65536 / (kThreads * kCtasPerSm) / 8 * 8;     // what the compiler gives every thread at launch
constexpr int kRegsFew = 64, kRegsMany = 192;      // registers per thread of the two warpgroups after they trade
// setmaxnreg only moves registers inside the CTA's allocation: asking for more than it holds waits for ever
static_assert(kRegsFew + kRegsMany <= 2 * kLaunchRegs, "the two warpgroups cannot hold more registers than the CTA was given");
constexpr int kTileBytes = BQ * 128;              // P, or one block of Q: 128 rows of 128 bytes
constexpr int kQBytes = KB * kTileBytes;
constexpr int kKVBlock = BKV * 128;               // one block of a K or V tile: 64 keys of 128 bytes
constexpr int kKVBytes = KB * kKVBlock;
constexpr int kStages = 3;                        // ring slots for key tiles, and as many for value tiles
constexpr int kPageWindow = 256;                  // block-table entries staged in shared memory at a time
constexpr int kSmemBytes = kQBytes + 2 * kTileBytes + 2 * kStages * kKVBytes + 1024 + 1024 + kPageWindow * 4;
constexpr int kTmemCols = 256;                    // S of even / odd tiles: columns 0..63 / 64..127, O: 128..128+HD-1

struct AttnTcParams {
    __nv_bfloat16* out;           // [T, NH*HD]
    const int32_t* block_table;   // [S, max_pages]
    const int32_t* tile_req;      // [tiles]
    const int32_t* tile_row0;     // [tiles] first row (token * G + head) of the tile within its request
    const int32_t* tile_cut;      // [tiles][3] or null: this entry's share of the tile's keys (share, shares, first slot)
    float* part_o;                // [slots][NKV][128][HD] unnormalised sums of the entries that share a tile
    float* part_ml;               // [slots][NKV][128][2] reference exponent (exp2 domain) and sum of weights
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

// two fp32 lanes per instruction (the packed fp32 pipe): d = a * b + c and d = a + b on register pairs
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// A row's reference exponent moves only when its maximum has grown by more than this (in the exp2 domain):
// until then the weights are at most 2^8, which fp32 sums and bfloat16 weights hold with the same relative
// precision, and the accumulator in TMEM needs no rescaling.  The final division by the row's sum, taken
// with the same references, makes the result independent of when the reference moved.
constexpr float kRefSlack = 8.0f;

// score i of the row's 64 (i is a constant after unrolling)
#define SV(i) ((i) < 32 ? sv_lo[(i) & 31] : sv_hi[(i) & 31])

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
paged_attention_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                             const AttnTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                                            // [KB][128][64] bf16, K-major, swizzled
    uint8_t* p_s = smem + kQBytes;                                  // [2][128][64 keys] bf16, K-major, swizzled
    uint8_t* k_s = p_s + 2 * kTileBytes;                            // [kStages][KB][64 keys][64]
    uint8_t* v_s = k_s + kStages * kKVBytes;                        // [kStages][KB][64 keys][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + kStages * kKVBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                  // [kStages]
    uint64_t* k_empty = k_full + kStages;         // [kStages]
    uint64_t* v_full = k_empty + kStages;         // [kStages]
    uint64_t* v_empty = v_full + kStages;         // [kStages]
    uint64_t* s_full = v_empty + kStages;         // [2]
    uint64_t* p_ready = s_full + 2;               // [2]
    uint64_t* o_done = p_ready + 2;               // [2]
    uint64_t* s_free = o_done + 2;                // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int32_t* page_win = reinterpret_cast<int32_t*>(bars) + 256;     // [kPageWindow] block-table entries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles come longest first, and CTAs are handed out in the order of blockIdx.x: the kv heads of one tile are
    // neighbours, so that the long tiles of every head start in the first wave
    const int tile = blockIdx.x / p.NKV, kvh = blockIdx.x % p.NKV;
    const int G = p.NH / p.NKV;

    if (threadIdx.x == 0) {
        *abort = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&p_ready[b], 4);
            mbar_init(&s_free[b], 4);
            mbar_init(&o_done[b], 1);
        }
        mbar_fence_init();
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_kv);
    }
    // key/value stages start as zeros: pages that are skipped (beyond the request, or released by the
    // window) leave their rows as they are, and those rows must hold finite numbers (their weights are 0)
    for (int i = threadIdx.x; i < 2 * kStages * kKVBytes / 16; i += kThreads) reinterpret_cast<uint4*>(k_s)[i] = make_uint4(0, 0, 0, 0);
    // so do the rows of Q that a tile of fewer than 128 rows leaves unwritten
    for (int i = threadIdx.x; i < kQBytes / 16; i += kThreads) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
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

    // (the step's tile lists, request boundaries and block tables were written before its first kernel started: they
    // are read ahead of the dependency wait, which orders this kernel after the one that makes q and this step's keys)
    const int s_req = p.tile_req[tile], row0 = p.tile_row0[tile];
    const int qs0 = p.q_start[s_req], qlen = p.q_start[s_req + 1] - qs0, ctx = p.ctx_before[s_req];
    const int tile_rows = (BQ / G) * G;                             // rows of a full tile: whole tokens only
    const int rows_here = min(tile_rows, qlen * G - row0);
    const int pos_lo = ctx + row0 / G, pos_hi = ctx + (row0 + rows_here - 1) / G;
    const int kv_hi = pos_hi + 1;
    const int kv_lo = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    // this entry's share of the tile's key tiles (all of them unless the step cut the tile's keys)
    int share = 0, shares = 1, slot = 0;
    if (p.tile_cut != nullptr) {
        share = p.tile_cut[3 * tile];
        shares = p.tile_cut[3 * tile + 1];
        slot = p.tile_cut[3 * tile + 2] + share;
    }
    const int t_first = kv_lo / BKV, n_all = (kv_hi + BKV - 1) / BKV - t_first;
    const int t_begin = t_first + (int)((long long)n_all * share / shares);
    const int t_end = t_first + (int)((long long)n_all * (share + 1) / shares);
    const int n_iter = t_end - t_begin;
    forge::pdl_wait();

    // the softmax rows keep a row's 64 scores in registers; the other warpgroup runs single threads and gives
    // its registers up for that
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsFew));
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // The warp stages the request's block-table entries in shared memory, a window at a time (one coalesced
        // read instead of a dependent global load per page); lane 0 then issues the copies.
        const int32_t* table = p.block_table + (size_t)s_req * p.max_pages;
        const int ppt = BKV / p.page_size;                               // pages per key tile
        const int iters_per_win = kPageWindow / ppt;
        const uint32_t page_bytes = p.page_size * 128;
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, KB * tile_rows * 128);
            for (int kb = 0; kb < KB; ++kb) tma_load_3d(q_s + kb * kTileBytes, &tmap_q, q_full, kb * 64, kvh * G, qs0 + row0 / G);
        }
        bool ok = true;
        int st = 0, ph = 0;                                              // ring slot and its phase
        for (int it0 = 0; it0 < n_iter && ok; it0 += iters_per_win) {
            const int it1 = min(n_iter, it0 + iters_per_win);
            const int first_page = (t_begin + it0) * ppt;
            __syncwarp();
            for (int i = lane; i < (it1 - it0) * ppt; i += 32)
                page_win[i] = first_page + i < p.max_pages ? table[first_page + i] : -1;
            __syncwarp();
            if (lane == 0) {
                for (int it = it0; it < it1 && ok; ++it) {
                    const int t0 = (t_begin + it) * BKV;
                    int rows[8], n_valid = 0;
                    for (int i = 0; i < ppt; ++i) {
                        const int tp = t0 + i * p.page_size, page = page_win[(it - it0) * ppt + i];
                        const bool live = tp < kv_hi && tp + p.page_size > kv_lo && page >= 0 && FORGE_PAGE_OK(page);
                        rows[i] = live ? (page * 2 * p.NKV + kvh) * p.page_size : -1;
                        n_valid += live;
                    }
                    // keys first: Q K^T of a tile runs two tiles ahead of its P V
                    if (!(ok = mbar_wait<true>(&k_empty[st], ph ^ 1, abort, p.status, 1))) break;
                    mbar_arrive_expect_tx(&k_full[st], KB * n_valid * page_bytes);
                    for (int i = 0; i < ppt; ++i)
                        if (rows[i] >= 0)
                            for (int kb = 0; kb < KB; ++kb)
                                tma_load_2d(k_s + st * kKVBytes + kb * kKVBlock + i * page_bytes, &tmap_kv, &k_full[st], kb * 64, rows[i]);
                    if (!(ok = mbar_wait<true>(&v_empty[st], ph ^ 1, abort, p.status, 9))) break;
                    mbar_arrive_expect_tx(&v_full[st], KB * n_valid * page_bytes);
                    for (int i = 0; i < ppt; ++i)
                        if (rows[i] >= 0)
                            for (int kb = 0; kb < KB; ++kb)
                                tma_load_2d(v_s + st * kKVBytes + kb * kKVBlock + i * page_bytes, &tmap_kv, &v_full[st], kb * 64,
                                            rows[i] + p.NKV * p.page_size);
                    if (++st == kStages) { st = 0; ph ^= 1; }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ P V issuer
        if (lane == 0) {
            constexpr uint32_t idesc_pv = umma_idesc_bf16_f32_bmn(BQ, 64);        // one product per 64 columns of the head
            const uint32_t p_addr = smem_u32(p_s), v_addr = smem_u32(v_s);
            bool ok = true;
            int vst = 0, vph = 0;
            for (int it = 0; it < n_iter && ok; ++it) {
                const int b = it & 1;
                if (!(ok = mbar_wait<true>(&v_full[vst], vph, abort, p.status, 4))) break;
                if (!(ok = mbar_wait<true>(&p_ready[b], (it >> 1) & 1, abort, p.status, 5))) break;
                tc_fence_after_sync();
                const uint32_t pa = p_addr + b * kTileBytes, va = v_addr + vst * kKVBytes;
#pragma unroll
                for (int nb = 0; nb < KB; ++nb)
#pragma unroll
                    for (int k = 0; k < BKV / UMMA_K; ++k)
                        umma_bf16(tmem_base + 2 * BKV + nb * 64, umma_desc_k_sw128(pa + k * 32),
                                  umma_desc_mn_sw128(va + nb * kKVBlock + k * 2048, 0), idesc_pv, (it | k) != 0);
                umma_commit(&o_done[b]);
                umma_commit(&v_empty[vst]);
                if (++vst == kStages) { vst = 0; vph ^= 1; }
            }
        }
    } else if (warp == kQkWarp) {
        // ------------------------------------------------------------------ Q K^T issuer
        // A thread issues one tcgen05 instruction or barrier probe every 50 to 100 clocks, so the two products
        // have a thread each.  S has two buffers in TMEM, and the rows hold S of tile it in registers from
        // the start of their work on it: its buffer takes the scores of tile it + 2 while they compute.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(BQ, BKV);
            const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s);
            bool ok = mbar_wait<true>(q_full, 0, abort, p.status, 2);
            int kst = 0, kph = 0;
            for (int it = 0; it < n_iter && ok; ++it) {
                const int b = it & 1;
                if (!(ok = mbar_wait<true>(&k_full[kst], kph, abort, p.status, 3))) break;
                if (it >= 2 && !(ok = mbar_wait<true>(&s_free[b], ((it - 2) >> 1) & 1, abort, p.status, 11))) break;
                // P V of tile it - 2 has read its P buffer before these scores exist: the rows, who wait for the
                // scores, then need no probe of their own before they overwrite that buffer (a probe costs them
                // some 200 clocks of their dependent chain; this thread has the time)
                if (it >= 2 && !(ok = mbar_wait<true>(&o_done[b], ((it - 2) >> 1) & 1, abort, p.status, 10))) break;
                tc_fence_after_sync();
                const uint32_t ka = k_addr + kst * kKVBytes;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int k = 0; k < 64 / UMMA_K; ++k)
                        umma_bf16(tmem_base + b * BKV, umma_desc_k_sw128(q_addr + kb * kTileBytes + k * 32),
                                  umma_desc_k_sw128(ka + kb * kKVBlock + k * 32), idesc_qk, (kb | k) != 0);
                umma_commit(&s_full[b]);
                umma_commit(&k_empty[kst]);
                if (++kst == kStages) { kst = 0; kph ^= 1; }
            }
        }
    }
    } else {
        // ------------------------------------------------------------------ softmax rows (warps 4..7)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMany));
        const int quarter = warp & 3;                            // the quarter of TMEM's lanes that this warp may touch
        const int r_local = quarter * 32 + lane;                 // row of the tile = TMEM lane
        const int r = row0 + r_local;
        const bool valid = r_local < rows_here;
        const int pos = ctx + r / G;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t t_out = t_lane + 2 * BKV;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_iter && ok; ++it) {
            const int j0 = (t_begin + it) * BKV, b = it & 1;
            uint8_t* p_row = p_s + b * kTileBytes + r_local * 128;
            if (!(ok = mbar_wait<true>(&s_full[b], (it >> 1) & 1, abort, p.status, 6))) break;
            tc_fence_after_sync();
            // the row's 64 scores stay in registers for both passes
            uint32_t sv_lo[32], sv_hi[32];
            tmem_ld_32x32b_x32(t_lane + b * BKV, sv_lo);
            tmem_ld_32x32b_x32(t_lane + b * BKV + 32, sv_hi);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[b]);
            // rows whose keys of this tile are all visible skip the per-key tests (all tiles but the ones on the
            // diagonal or at the window's edge); masked scores become -inf here, once
            const bool need_mask = !valid || j0 + BKV - 1 > pos || (p.window > 0 && j0 <= pos - p.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < BKV; ++i) {
                    const int j = j0 + i;
                    const bool vis = valid && j <= pos && (p.window <= 0 || j > pos - p.window);
                    if (!vis) SV(i) = __float_as_uint(-INFINITY);
                }
            }
            // pass 1: the maximum of the raw scores (the scale is positive, so it commutes with the maximum),
            // in two independent chains of three-input maxima
            float a0 = -INFINITY, a1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < BKV; i += 4) {
                a0 = max3(a0, __uint_as_float(SV(i)), __uint_as_float(SV(i + 1)));
                a1 = max3(a1, __uint_as_float(SV(i + 2)), __uint_as_float(SV(i + 3)));
            }
            const float mx_tile = fmaxf(a0, a1) * p.scale_log2;
            // m is the reference of the row's exponents; -inf + slack is -inf, so the first visible key sets it
            const float m_new = mx_tile > m + kRefSlack ? mx_tile : m;
            const float alpha = m_new == m ? 1.0f : ex2_approx(m - m_new);
            m = m_new;
            const float ref = m == -INFINITY ? 0.f : m;
            // the accumulator is rescaled only when some row of the warp moved its reference (the TMEM loads
            // and stores are warp-wide, so the decision is the warp's); P V of the previous tile must be
            // complete by then
            if (it > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
                if (!(ok = mbar_wait<true>(&o_done[b ^ 1], ((it - 1) >> 1) & 1, abort, p.status, 7))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tmem_ld_32x32b_x32(t_out + c, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tmem_st_32x32b_x32(t_out + c, ov);
                }
                tmem_st_wait();
            }
            // (this P buffer was read by P V of the tile before the previous one: the thread that issued this
            // tile's Q K^T waited for that)
            // pass 2: weights (exp2 of -inf is 0), their sum, and P in the MMA's shared-memory layout
            // (16-byte chunk ^ row % 8)
            const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), nref2 = pack_f32x2(-ref, -ref);
            uint64_t acc_a = pack_f32x2(0.f, 0.f), acc_b = acc_a;
#pragma unroll
            for (int c = 0; c < BKV; c += 8) {
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 8; i += 4) {
                    float x0, x1, x2, x3;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(SV(c + i)), __uint_as_float(SV(c + i + 1))), scale2, nref2), x0, x1);
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(SV(c + i + 2)), __uint_as_float(SV(c + i + 3))), scale2, nref2), x2, x3);
                    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
                    acc_a = add_f32x2(acc_a, pack_f32x2(p0, p1));
                    acc_b = add_f32x2(acc_b, pack_f32x2(p2, p3));
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h0);
                    packed[(i >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
                *reinterpret_cast<uint4*>(p_row + (((c >> 3) ^ (r_local & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            float s0, s1, s2, s3;
            unpack_f32x2(acc_a, s0, s1);
            unpack_f32x2(acc_b, s2, s3);
            l = l * alpha + ((s0 + s1) + (s2 + s3));
            // one arrival per warp: P is in shared memory for the tensor core to read (and O, if it was
            // rescaled, is in TMEM)
            tc_fence_before_sync();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        if (ok && n_iter > 0) ok = mbar_wait<true>(&o_done[(n_iter - 1) & 1], ((n_iter - 1) >> 1) & 1, abort, p.status, 8);
        tc_fence_after_sync();
        if (shares > 1) {
            // one share of the tile's keys: the sums as they are, with the reference they were taken against
            // (a share without a visible key, or one that gave up waiting, counts as nothing)
            const bool have = __all_sync(0xffffffffu, ok) && n_iter > 0;
            const size_t prow = ((size_t)slot * p.NKV + kvh) * BQ + r_local;
            p.part_ml[prow * 2] = have ? m : -INFINITY;
            p.part_ml[prow * 2 + 1] = have ? l : 0.f;
            if (have) {
                float* dst = p.part_o + prow * HD;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tmem_ld_32x32b_x32(t_out + c, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(ov[i], ov[i + 1], ov[i + 2], ov[i + 3]);
                }
            }
        } else if (ok && n_iter > 0) {
            // every lane takes part in the TMEM loads (they are warp-wide instructions); only valid rows store
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = p.out + (size_t)(qs0 + r / G) * p.NH * HD + (size_t)(kvh * G + r % G) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                tmem_ld_32x32b_x32(t_out + c, ov);
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

// Adds up the shares of the tiles whose keys were cut: a thread per (row, four neighbouring columns), 256 / (HD / 4)
// rows per CTA.  The shares are walked in their order, so the sum does not depend on timing.
//   M = max_z m_z;  o = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z
constexpr int kMergeThreads = 256, kMaxShares = 32;
constexpr int kMergeRows = kMergeThreads / (HD / 4);             // rows per CTA
__global__ void __launch_bounds__(kMergeThreads)
attention_sm100_merge_kernel(const AttnTcParams p, const int32_t* __restrict__ merge_list) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int mt = blockIdx.x / p.NKV, kvh = blockIdx.x % p.NKV;
    const int G = p.NH / p.NKV;
    const int s_req = merge_list[4 * mt], row0 = merge_list[4 * mt + 1], slot0 = merge_list[4 * mt + 2];
    const int shares = min(merge_list[4 * mt + 3], kMaxShares);
    const int qs0 = p.q_start[s_req], qlen = p.q_start[s_req + 1] - qs0;
    const int rows_here = min((BQ / G) * G, qlen * G - row0);
    const int r_local = blockIdx.y * kMergeRows + threadIdx.x / (HD / 4), c = (threadIdx.x % (HD / 4)) * 4;
    if (r_local >= rows_here) return;
    const size_t prow0 = ((size_t)slot0 * p.NKV + kvh) * BQ + r_local, pstep = (size_t)p.NKV * BQ;     // share z: prow0 + z * pstep
    float M = -INFINITY;
    for (int z = 0; z < shares; ++z) M = fmaxf(M, p.part_ml[(prow0 + z * pstep) * 2]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int z = 0; z < shares; ++z) {
        const size_t prow = prow0 + z * pstep;
        const float m_z = p.part_ml[prow * 2], l_z = p.part_ml[prow * 2 + 1];
        // a share without a visible key never wrote its sums
        const float w = m_z == -INFINITY ? 0.f : exp2f(m_z - M);
        const float4 v = w != 0.f ? *reinterpret_cast<const float4*>(p.part_o + prow * HD + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        L += w * l_z;
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    const int r = row0 + r_local;
    __nv_bfloat16* dst = p.out + (size_t)(qs0 + r / G) * p.NH * HD + (size_t)(kvh * G + r % G) * HD + c;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), h1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
}

}  // namespace

// q [T, NH*HD] bf16, kv cache [pages, 2, NKV, page_size, HD] bf16, out [T, NH*HD] bf16.  tile_req / tile_row0
// list tiles of (128 / G) * G query rows (rows = tokens * G); q_start / ctx_before as for forge_paged_attention_mma.
// tile_cut (or null) [num_tiles][3]: entry i works on share tile_cut[i][0] of tile_cut[i][1] equal shares of its tile's
// key tiles and, with more than one share, leaves its sums in slot tile_cut[i][2] + share of part_o [slots][NKV][128][HD]
// and part_ml [slots][NKV][128][2]; merge_list [num_merge][4] = (request, first row, first slot, shares) names the
// tiles to add up afterwards (at most 32 shares each).
extern "C" int forge_paged_attention_sm100(const void* q, const void* kv, void* out, const int32_t* block_table,
                                           const int32_t* tile_req, const int32_t* tile_row0, const int32_t* tile_cut,
                                           void* part_o, void* part_ml, const int32_t* merge_list, int num_merge,
                                           const int32_t* q_start,
                                           const int32_t* ctx_before, int* status, int num_tiles, int T, int num_pages,
                                           int NH, int NKV, int head_dim, int page_size, int max_pages, int window,
                                           float scale, cudaStream_t stream) {
    if (head_dim != HD) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: this library was built for head_dim %d, got %d", HD, head_dim);
    if (NH <= 0 || NKV <= 0 || NH % NKV != 0 || NH / NKV > BQ)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: %d query heads per kv head (at most 128)", NKV > 0 ? NH / NKV : 0);
    if (page_size < 8 || BKV % page_size != 0)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: page size %d must be 8, 16, 32 or 64", page_size);
    if (!(scale > 0.f)) return forge::fail(FORGE_ERR_ARG, "paged_attention_sm100: scale %g must be positive", (double)scale);
    if (num_tiles < 0 || T <= 0 || num_pages <= 0 || max_pages <= 0)
        return forge::fail(FORGE_ERR_ARG, "paged_attention_sm100: bad sizes tiles=%d T=%d pages=%d", num_tiles, T, num_pages);
    if (num_merge < 0 || (num_merge > 0 && (!tile_cut || !part_o || !part_ml || !merge_list)))
        return forge::fail(FORGE_ERR_ARG, "paged_attention_sm100: %d tiles to add up need tile_cut, part_o, part_ml and merge_list", num_merge);
    if (num_tiles == 0) return FORGE_OK;
    const int G = NH / NKV;
    const char* err = nullptr;
    CUtensorMap tq, tkv;
    if (!bf16_q_map(q, T, NH, HD, BQ / G, G, &tq, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: q: %s", err);
    if (!bf16_tile_map(kv, num_pages * 2 * NKV * page_size, HD, page_size, &tkv, &err))
        return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: cache: %s", err);
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_sm100: %s", cudaGetErrorString(e));
        // the warpgroups trade registers inside what the CTA was given at launch; a build that gives less would wait
        // for registers that never come, so it is refused here
        cudaFuncAttributes attr;
        e = cudaFuncGetAttributes(&attr, paged_attention_sm100_kernel);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "paged_attention_sm100: %s", cudaGetErrorString(e));
        if (attr.numRegs * 2 < kRegsFew + kRegsMany)
            return forge::fail(FORGE_ERR_UNSUPPORTED, "paged_attention_sm100: built with %d registers per thread, needs %d",
                               attr.numRegs, (kRegsFew + kRegsMany + 1) / 2);
        configured = true;
    }
    AttnTcParams p{(__nv_bfloat16*)out, block_table, tile_req, tile_row0, tile_cut, (float*)part_o, (float*)part_ml,
                   q_start, ctx_before, NH, NKV, page_size, max_pages, window, scale * 1.4426950408889634f, status};
    int rc = forge::check_launch("paged_attention_sm100",
                                 forge::launch(paged_attention_sm100_kernel, dim3((unsigned)num_tiles * NKV), dim3(kThreads), kSmemBytes,
                                               stream, 1, tq, tkv, p));
    if (rc != FORGE_OK || num_merge == 0) return rc;
    return forge::check_launch("attention_sm100_merge",
                               forge::launch(attention_sm100_merge_kernel, dim3((unsigned)num_merge * NKV, BQ / kMergeRows), dim3(kMergeThreads), 0,
                                             stream, 1, p, merge_list));
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }

// (checks build) the bounds that this library's kernel tests page ids against
FORGE_DEFINE_CHECKS_ENTRY(attention_sm100)
