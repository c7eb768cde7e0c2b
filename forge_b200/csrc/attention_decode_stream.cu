// Decode step's attention for long contexts: the keys and values stream through a ring in shared memory.
//
// Same work as decode_attention_fused_kernel (attention_mma.cu): one new token per request; a CTA serves one
// (request, kv head), or one of the 2, 4 or 8 CTAs of a cluster that share one; it rotates the G query heads and
// the key head of the new token (fp32 angles), writes the key and the value into the request's page and attends
// over the request's keys with mma.sync.m16n8k16 and an online softmax in fp32 (exp2 domain).  What differs is
// how the cache reaches the SM.  There every warp fetches its own tiles of 32 keys with cp.async into two
// buffers, so a warp has one tile in flight while it computes on the other and waits out most of a memory
// latency per tile (3 TB/s at 8 requests x 8,192 tokens, 4.2-4.9 TB/s with 64 and more (request, kv head) pairs).
// Here two producer threads (of two warps: one thread's TMA instructions are taken one after the other) walk the
// block table and bring tiles of 64 keys by TMA, one box per page holding the page's keys AND values of this kv
// head (a 5-D view of the cache [pages, 2, kv heads, page, head]; 16 KB per instruction with pages of 64 tokens and
// heads of 64), into a ring of 4 or 8 tiles; the consumer warps take the tiles in turn.  A whole ring is in flight
// while the consumers compute, whatever a single warp's pace.
//   Tiles land with the 128-byte swizzle (16-byte chunk c of row r at chunk c ^ (r % 8)), which ldmatrix reads
// without bank conflicts; a head of 128 is two 64-wide blocks per tile.  The new token's key and value never
// travel through global memory on their way to this CTA's products: the warp that gets the last tile writes them
// into the tile's row after the tile has landed (the copy of that row may be older than this step's write).
// Every wait on a barrier is bounded (sm100.cuh).
//   s_j = (q . k_j) / sqrt(HD) for keys max(0, p - window + 1) <= j <= p of the token's position p;
//   o = sum_j softmax(s)_j v_j          (formulas of src/operators/cuda/cuda_flash_attn.cu:154-248, 297-439)
// Head sizes 64 and 128, pages of 16, 32 or 64 tokens, at most 16 query heads per kv head.
#include "common.cuh"
#include "checks.cuh"
#include "mma_sync.cuh"
#include "sm100.cuh"

#ifndef FORGE_ATT_HD
#define FORGE_ATT_HD 64
#endif

#if FORGE_ATT_HD == 64 || FORGE_ATT_HD == 128

namespace {

using namespace mma_sync;
using namespace sm100;

constexpr int HD = FORGE_ATT_HD, KB = HD / 64;      // 64-wide blocks of the head
constexpr int TK = 64;                              // keys per tile
constexpr int LDQ = HD + 8;                         // padded row of Q in shared memory (bf16 elements)
constexpr int kBlockBytes = TK * 128;               // one block of a tile's keys (or values): 64 rows of 128 bytes
constexpr int kTileBytes = 2 * KB * kBlockBytes;    // per 64-wide block: the keys, then the values
constexpr int kProducers = 2;                       // warps 0 and 1: one issuing thread each

struct StreamParams {
    const float* qkv;             // [S, (NH + 2 NKV) * HD] fp32: the new token's projections, one row per request
    __nv_bfloat16* kv;            // [pages, 2, NKV, page_size, HD]
    __nv_bfloat16* out;           // [S, NH*HD]
    const int32_t* block_table;   // [S, max_pages]
    const int32_t* positions;     // [S] position of the new token = tokens already cached
    const int32_t* slot_mapping;  // [S] page * page_size + offset of the new token
    int NH, NKV, page_size, max_pages, window, rotary;
    float theta, scale_log2;
    int ksplit;                   // CTAs of a cluster that share one (request, kv head) and deal its key tiles out
    int* status;
};

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ uint32_t stream_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void stream_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float stream_ld_peer(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Shared memory: [ring: R tiles, 1024-byte aligned][Q 16 x LDQ bf16][new key, new value: 2 x HD bf16][barriers]
template <int NC, int R> struct StreamCfg {
    static constexpr int kThreads = 32 * (kProducers + NC);
    static constexpr int kRingBytes = R * kTileBytes;
    static constexpr int kQBytes = 16 * LDQ * 2;
    static constexpr int kNewBytes = 2 * HD * 2;
    static constexpr int kMergeBytes = (NC * 16 * HD + NC * 16 * 2 + 16 * HD + 16 * 2) * 4;      // lives in the ring after the last tile
    static_assert(kMergeBytes <= kRingBytes, "the merge area must fit the ring");
    // A slot's successive tiles must go to the same consumer: a barrier's parity tells two phases apart, so a warp
    // whose FIRST tile were a slot's second would find "its" phase complete before the first tile has landed.
    static_assert(R % NC == 0, "the ring holds a whole number of tiles per consumer");
    static constexpr int kSmemBytes = 1024 + kRingBytes + kQBytes + kNewBytes + 2 * R * 8 + 64;
};

template <int NC, int R, bool CLUSTER>
__global__ void __launch_bounds__(32 * (kProducers + NC))
decode_attention_stream_kernel(const __grid_constant__ CUtensorMap tmap_kv, const StreamParams p) {
    using C = StreamCfg<NC, R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(ring + C::kRingBytes);                 // [16][LDQ], G heads, zero-padded
    __nv_bfloat16* kv_new = qs + 16 * LDQ;                                                      // [2][HD]: the new token's key and value
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(kv_new) + C::kNewBytes);   // [R] copies -> consumers
    uint64_t* empty = full + R;                                                                 // [R] consumer -> producers
    volatile int* abort = reinterpret_cast<volatile int*>(empty + R);

    forge::pdl_launch_dependents();
    const int KS = CLUSTER ? p.ksplit : 1;
    const int rank = CLUSTER ? static_cast<int>(stream_cluster_rank()) : 0;
    const int s = blockIdx.x / KS, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.NH / p.NKV;
    // The step's positions, slots and block tables were written before its first kernel started, and the keys and
    // values of earlier positions in earlier steps: all of that may be read before the dependency wait, which only
    // orders this kernel after the product that makes q, k and v.
    const int pos = p.positions[s];
    const int slot = p.slot_mapping[s];
    const int32_t* table = p.block_table + (size_t)s * p.max_pages;
    const int kv_hi = pos + 1;
    const int kv_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int t_begin = kv_lo / TK, t_end = (kv_hi + TK - 1) / TK;
    // the cluster's CTAs take the tiles in turn: this CTA's i-th tile is t_begin + rank + i * KS
    const int n_mine = (t_end - t_begin - rank + KS - 1) / KS;
    const int ppt = TK / p.page_size;                                    // pages per tile
    const uint32_t page_bytes = 2u * p.page_size * 128u;                 // one box: a page's keys and values, 64 columns

    if (threadIdx.x == 0) {
        *abort = 0;
        for (int i = 0; i < R; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_fence_init();
        prefetch_tensormap(&tmap_kv);
    }
    // Pages that a tile does not need (beyond the token, or released by the window) are not copied: their rows keep
    // what the ring held, which must be finite numbers because their weights are exact zeros.  With pages of 64
    // tokens a tile is one page and is copied whole or does not exist.
    if (ppt > 1) {
        for (int i = threadIdx.x; i < C::kRingBytes / 16; i += C::kThreads) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
    }
    __syncthreads();

    if (warp < kProducers) {
        // ------------------------------------------------------------------ producers: tiles i = warp, warp + 2, ...
        // The warp reads the block-table entries of its next 32 tiles at once (one coalesced trip instead of a
        // dependent load per page), lane 0 then issues the copies.
        bool ok = true;
        for (int i0 = warp; i0 < n_mine && ok; i0 += 32 * kProducers) {
            int pages[4];                                                 // the pages of this lane's tile (at most 4: pages of 16)
            const int i_lane = i0 + lane * kProducers;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                pages[j] = -1;
                if (j < ppt && i_lane < n_mine) {
                    const int t = t_begin + rank + i_lane * KS;
                    const int tp = t * TK + j * p.page_size;              // first token of the page
                    const int idx = tp / p.page_size;
                    if (tp < kv_hi && tp + p.page_size > kv_lo && idx < p.max_pages) {
                        const int pg = table[idx];
                        if (pg >= 0 && FORGE_PAGE_OK(pg)) pages[j] = pg;
                    }
                }
            }
            for (int l = 0; l < 32 && ok; ++l) {
                const int i = i0 + l * kProducers;
                if (i >= n_mine) break;
                int pg[4], n_valid = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    pg[j] = __shfl_sync(0xffffffffu, pages[j], l);
                    n_valid += pg[j] >= 0;
                }
                if (lane == 0) {
                    const int st = i % R;
                    if (!(ok = mbar_wait<true>(&empty[st], ((i / R) & 1) ^ 1, abort, p.status, 1))) {
                    } else {
                        mbar_arrive_expect_tx(&full[st], (uint32_t)(n_valid * KB) * page_bytes);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (j >= ppt || pg[j] < 0) continue;
                            for (int kb = 0; kb < KB; ++kb)
                                tma_load_5d(ring + st * kTileBytes + kb * 2 * kBlockBytes + j * page_bytes, &tmap_kv, &full[st],
                                            kb * 64, 0, 0, kvh, pg[j]);
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
        }
        forge::pdl_wait();                          // (nothing of this warp depends on the earlier kernel; it waits with the others)
    } else {
        // ------------------------------------------------------------------ consumers
        const int cw = warp - kProducers;            // consumer index: tiles i = cw, cw + NC, ...
        const int ct = threadIdx.x - 32 * kProducers, cthreads = 32 * NC;
        forge::pdl_wait();
        // 1. rotate q (G heads) and k (one head), copy v; q to shared memory, k and v to shared memory and the cache
        const float* row = p.qkv + (size_t)s * (p.NH + 2 * p.NKV) * HD;
        const int half = HD / 2;
        // the CTA that gets the tile with the new token writes the token's key and value into the cache
        const bool owns_last = (t_end - 1 - t_begin) % KS == rank;
        __nv_bfloat16* page_base = p.kv + ((size_t)(slot / p.page_size) * 2 * p.NKV + kvh) * p.page_size * HD + (size_t)(slot % p.page_size) * HD;
        for (int i = ct; i < 16 * (HD / 8); i += cthreads)               // clear the padding rows of Q
            if (i / (HD / 8) >= G) *reinterpret_cast<uint4*>(qs + (i / (HD / 8)) * LDQ + (i % (HD / 8)) * 8) = make_uint4(0, 0, 0, 0);
        for (int i = ct; i < (G + 2) * half; i += cthreads) {
            const int h = i / half, d = i % half;                         // h < G: q head; G: k; G + 1: v
            const int src_head = h < G ? kvh * G + h : (h == G ? p.NH + kvh : p.NH + p.NKV + kvh);
            float x0 = row[src_head * HD + d], x1 = row[src_head * HD + d + half];
            if (p.rotary && h <= G) {
                const float freq = 1.0f / powf(p.theta, (2.0f * (float)d) / (float)HD);
                float sn, cs;
                sincosf((float)pos * freq, &sn, &cs);
                const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
                x0 = y0;
                x1 = y1;
            }
            const __nv_bfloat16 b0 = __float2bfloat16_rn(x0), b1 = __float2bfloat16_rn(x1);
            if (h < G) {
                qs[h * LDQ + d] = b0;
                qs[h * LDQ + d + half] = b1;
            } else {
                kv_new[(h - G) * HD + d] = b0;
                kv_new[(h - G) * HD + d + half] = b1;
                if (owns_last && FORGE_SLOT_OK(slot)) {
                    __nv_bfloat16* dst = page_base + (h == G ? 0 : (size_t)p.NKV * p.page_size * HD);
                    dst[d] = b0;
                    dst[d + half] = b1;
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");       // the consumers only: Q and the new key/value are in place

        // 2. every consumer warp walks its share of the CTA's tiles
        const bool valid_a = (lane >> 2) < G, valid_b = (lane >> 2) + 8 < G;
        float o_acc[HD / 8][4];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
        bool ok = true;
        for (int i = cw; i < n_mine && ok; i += NC) {
            const int t = t_begin + rank + i * KS, st = i % R;
            uint8_t* tile = ring + st * kTileBytes;
            if (!(ok = mbar_wait<true>(&full[st], (i / R) & 1, abort, p.status, 2))) break;
            if (t == t_end - 1) {
                // the new token's row: what the copy brought for it may be older than this step's write
                const int r = pos - t * TK;
                if (lane < 2 * (HD / 8)) {
                    const int which = lane / (HD / 8), c = lane % (HD / 8);          // 0: key, 1: value; 16-byte chunk of the head
                    const int page_j = r / p.page_size, pr = r % p.page_size;
                    uint8_t* dst = tile + (c / 8) * 2 * kBlockBytes + page_j * page_bytes + which * p.page_size * 128 + pr * 128 +
                                   (((c % 8) ^ (pr & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(kv_new + which * HD + c * 8);
                }
                __syncwarp();
            }
            // row `key` of the tile's keys (which = 0) or values (1), 64-wide block kb: its 128 bytes
            auto row_ptr = [&](int key, int which, int kb) -> const uint8_t* {
                return tile + kb * 2 * kBlockBytes + (key / p.page_size) * page_bytes + which * p.page_size * 128 + (key % p.page_size) * 128;
            };
            float sc[TK / 8][4];
#pragma unroll
            for (int j = 0; j < TK / 8; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, qs + (lane & 15) * LDQ + kk * 16 + (lane >> 4) * 8);
                const int c = (kk % 4) * 2 + ((lane >> 3) & 1);           // 16-byte chunk inside the 64-wide block
#pragma unroll
                for (int nb = 0; nb < TK / 16; ++nb) {
                    const int key = nb * 16 + (lane >> 4) * 8 + (lane & 7);
                    uint32_t b[4];
                    ldmatrix_x4(b, row_ptr(key, 0, kk / 4) + ((c ^ (key & 7)) << 4));
                    mma_bf16(sc[2 * nb], a, b[0], b[1]);
                    mma_bf16(sc[2 * nb + 1], a, b[2], b[3]);
                }
            }
            float mx_a = m_a, mx_b = m_b;
            const bool unmasked = t * TK + TK - 1 <= pos && (p.window <= 0 || t * TK > pos - p.window);
            const int j0 = t * TK + 2 * (lane & 3);
#pragma unroll
            for (int j = 0; j < TK / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = j0 + j * 8 + e;
                    const bool vis = unmasked || (key <= pos && (p.window <= 0 || key > pos - p.window));
                    sc[j][e] = (vis && valid_a) ? sc[j][e] * p.scale_log2 : -INFINITY;
                    sc[j][2 + e] = (vis && valid_b) ? sc[j][2 + e] * p.scale_log2 : -INFINITY;
                    mx_a = fmaxf(mx_a, sc[j][e]);
                    mx_b = fmaxf(mx_b, sc[j][2 + e]);
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
            uint32_t pfrag[TK / 16][4];
#pragma unroll
            for (int j = 0; j < TK / 8; ++j) {
                const float p0 = ex2_approx(sc[j][0] - ref_a), p1 = ex2_approx(sc[j][1] - ref_a);
                const float p2 = ex2_approx(sc[j][2] - ref_b), p3 = ex2_approx(sc[j][3] - ref_b);
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                pfrag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                pfrag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_a = l_a * alpha_a + sum_a;
            l_b = l_b * alpha_b + sum_b;
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o_acc[j][0] *= alpha_a; o_acc[j][1] *= alpha_a;
                o_acc[j][2] *= alpha_b; o_acc[j][3] *= alpha_b;
            }
#pragma unroll
            for (int kk = 0; kk < TK / 16; ++kk) {
                const int key = kk * 16 + (lane & 15);
#pragma unroll
                for (int db = 0; db < HD / 16; ++db) {
                    const int c = (db % 4) * 2 + (lane >> 4);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, row_ptr(key, 1, db / 4) + ((c ^ (key & 7)) << 4));
                    mma_bf16(o_acc[2 * db], pfrag[kk], b[0], b[1]);
                    mma_bf16(o_acc[2 * db + 1], pfrag[kk], b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);                       // the tile's slot may take another tile
        }
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (!ok) { m_a = m_b = -INFINITY; l_a = l_b = 0.f; }              // a wait ran out: the status word says so, the output is zeros

        // 3. merge the consumers' partial results through the ring (every tile of this CTA has landed and been read
        // once all consumers are here), in warp order
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        float* mo = reinterpret_cast<float*>(ring);                      // [NC][16][HD]
        float* ml = mo + NC * 16 * HD;                                   // [NC][16][2]
        {
            const int ra = lane >> 2, rb = ra + 8, d0 = 2 * (lane & 3);
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                *reinterpret_cast<float2*>(mo + ((size_t)cw * 16 + ra) * HD + j * 8 + d0) = make_float2(o_acc[j][0], o_acc[j][1]);
                *reinterpret_cast<float2*>(mo + ((size_t)cw * 16 + rb) * HD + j * 8 + d0) = make_float2(o_acc[j][2], o_acc[j][3]);
            }
            if ((lane & 3) == 0) {
                ml[(cw * 16 + ra) * 2] = m_a; ml[(cw * 16 + ra) * 2 + 1] = l_a;
                ml[(cw * 16 + rb) * 2] = m_b; ml[(cw * 16 + rb) * 2 + 1] = l_b;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        float* cta_o = ml + NC * 16 * 2;                                 // [16][HD] this CTA's un-normalised output
        float* cta_ml = cta_o + 16 * HD;                                 // [16][2]  its maximum and sum
        for (int i = ct; i < G * HD; i += cthreads) {
            const int r = i / HD, d = i % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NC; ++w) M = fmaxf(M, ml[(w * 16 + r) * 2]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < NC; ++w) {
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
    }
    if (CLUSTER) {
        // 4. the cluster's CTAs, in rank order, by CTA 0
        float* cta_o = reinterpret_cast<float*>(ring) + NC * 16 * HD + NC * 16 * 2;
        float* cta_ml = cta_o + 16 * HD;
        stream_cluster_sync();
        if (rank == 0) {
            for (int i = threadIdx.x; i < G * HD; i += C::kThreads) {
                const int r = i / HD, d = i % HD;
                float M = -INFINITY;
                for (int q = 0; q < KS; ++q) M = fmaxf(M, stream_ld_peer(cta_ml + r * 2, q));
                float L = 0.f, acc = 0.f;
                for (int q = 0; q < KS; ++q) {
                    const float mq = stream_ld_peer(cta_ml + r * 2, q);
                    const float wt = mq == -INFINITY ? 0.f : exp2f(mq - M);
                    L += wt * stream_ld_peer(cta_ml + r * 2 + 1, q);
                    acc += wt * stream_ld_peer(cta_o + r * HD + d, q);
                }
                p.out[(size_t)s * p.NH * HD + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            }
        }
        stream_cluster_sync();                  // nobody leaves while CTA 0 may still read its shared memory
    }
}

// The cache [pages, 2, NKV, page_size, HD] seen as {HD, page_size, 2, NKV, pages}; a box {64, page_size, 2, 1, 1} is one
// page's keys and values of one kv head, 64 columns of the head, with the 128-byte swizzle.
bool cache_page_map(const void* kv, int num_pages, int NKV, int page_size, CUtensorMap* out, const char** err) {
    using Key = std::tuple<const void*, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{kv, num_pages, NKV, page_size};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    auto fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
    if (reinterpret_cast<uintptr_t>(kv) & 15) { *err = "TMA needs a 16-byte aligned cache"; return false; }
    CUtensorMap m;
    const cuuint64_t row = (cuuint64_t)HD * 2, head = row * page_size;
    const cuuint64_t dims[5] = {(cuuint64_t)HD, (cuuint64_t)page_size, 2u, (cuuint64_t)NKV, (cuuint64_t)num_pages};
    const cuuint64_t strides[4] = {row, head * NKV, head, head * NKV * 2};
    const cuuint32_t box[5] = {64u, (cuuint32_t)page_size, 2u, 1u, 1u};
    const cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(kv), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed (cache pages)"; return false; }
    if (cache.size() > 1024) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

template <int NC, int R, bool CLUSTER>
int launch_stream(const CUtensorMap& tkv, const StreamParams& p, int S, int NKV, cudaStream_t stream) {
    using C = StreamCfg<NC, R>;
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_stream_kernel<NC, R, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e == cudaSuccess && CLUSTER)      // one or two requests with very long contexts: clusters of 16
            e = cudaFuncSetAttribute(decode_attention_stream_kernel<NC, R, CLUSTER>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "decode_attention_stream: %s", cudaGetErrorString(e));
        configured = true;
    }
    return forge::check_launch("decode_attention_stream",
                               forge::launch(decode_attention_stream_kernel<NC, R, CLUSTER>, dim3(S * p.ksplit, NKV), dim3(C::kThreads),
                                             C::kSmemBytes, stream, p.ksplit, tkv, p));
}

}  // namespace

// As forge_decode_attention_fused, plus: num_pages (pages of the cache tensor), status (device int, bit 1 raised if a
// wait ran out), ksplit (0: choose; 1, 2, 4, 8, 16: CTAs that share a request's keys; 16 is a cluster size beyond the
// portable 8, which the kernel is marked for).
extern "C" int forge_decode_attention_stream(const float* qkv, void* kv, void* out, const int32_t* block_table,
                                             const int32_t* positions, const int32_t* slot_mapping, int* status, int S,
                                             int NH, int NKV, int head_dim, int page_size, int max_pages, int num_pages,
                                             int window, int rotary, float theta, float scale, int max_context, int ksplit,
                                             cudaStream_t stream) {
    if (head_dim != HD) return forge::fail(FORGE_ERR_UNSUPPORTED, "this attention library was built for head_dim %d, got %d", HD, head_dim);
    if (S < 0 || NH <= 0 || NKV <= 0 || NH % NKV != 0 || max_pages <= 0 || num_pages <= 0 || NKV > 65535)
        return forge::fail(FORGE_ERR_ARG, "decode_attention_stream: bad sizes S=%d NH=%d NKV=%d pages=%d", S, NH, NKV, num_pages);
    if (page_size != 16 && page_size != 32 && page_size != 64)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_stream: page size %d (16, 32 or 64)", page_size);
    if (NH / NKV > 16) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_stream: %d query heads per kv head (at most 16)", NH / NKV);
    if (ksplit != 0 && ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8 && ksplit != 16)
        return forge::fail(FORGE_ERR_ARG, "decode_attention_stream: %d CTAs per request (1, 2, 4, 8 or 16)", ksplit);
    if (S == 0) return FORGE_OK;
    const char* err = nullptr;
    CUtensorMap tkv;
    if (!cache_page_map(kv, num_pages, NKV, page_size, &tkv, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_stream: %s", err);
    StreamParams p{qkv, (__nv_bfloat16*)kv, (__nv_bfloat16*)out, block_table, positions, slot_mapping, NH, NKV, page_size,
                   max_pages, window, rotary, theta, scale * 1.4426950408889634f, 1, status};
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // few (request, kv head) pairs: eight consumer warps and a ring of eight tiles (six with heads of 128), one CTA per SM, and while SMs are
    // idle 2, 4 or 8 CTAs share a request's keys as long as each keeps a ring's worth of tiles; many pairs: four
    // consumers and four tiles, three CTAs per SM
    constexpr int kFew = HD == 64 ? 8 : 6;           // consumers = tiles of the ring: 128 / 192 KB
    const bool few = (long)S * NKV <= sms;
    if (ksplit > 0) {
        p.ksplit = ksplit;
    } else if (few && max_context > 0) {
        // a cluster lives inside one GPC: fewer CTAs run at once in clusters of 4 or 8 than there are SMs, and a
        // second wave would double the time
        static int resident[17] = {0};
        const long tiles = (max_context + TK - 1) / TK;
        for (int ks = 2; ks <= 16; ks *= 2) {
            if (resident[ks] == 0) {
                cudaFuncSetAttribute(decode_attention_stream_kernel<kFew, kFew, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     StreamCfg<kFew, kFew>::kSmemBytes);
                cudaFuncSetAttribute(decode_attention_stream_kernel<kFew, kFew, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(ks * 16);
                cfg.blockDim = dim3(StreamCfg<kFew, kFew>::kThreads);
                cfg.dynamicSmemBytes = StreamCfg<kFew, kFew>::kSmemBytes;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = ks;
                at[0].val.clusterDim.y = 1;
                at[0].val.clusterDim.z = 1;
                cfg.attrs = at;
                cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, decode_attention_stream_kernel<kFew, kFew, true>, &cfg) != cudaSuccess || n <= 0) {
                    cudaGetLastError();
                    n = ks > 8 ? 0 : (sms - sms / 8 * (ks > 2 ? (ks > 4 ? 2 : 1) : 0)) / ks;      // a guess on the safe side; no clusters of 16
                }
                resident[ks] = n > 0 ? n * ks : -1;
            }
            if ((long)S * NKV * ks <= resident[ks] && tiles >= (long)kFew * ks) p.ksplit = ks;
        }
    }
    if (p.ksplit > 1) return launch_stream<kFew, kFew, true>(tkv, p, S, NKV, stream);
    if (few) return launch_stream<kFew, kFew, false>(tkv, p, S, NKV, stream);
    return launch_stream<4, 4, false>(tkv, p, S, NKV, stream);
}

// (checks build) the bounds that this file's kernel tests page ids and slots against
FORGE_DEFINE_CHECKS_ENTRY(attention_decode_stream)

#else

FORGE_DEFINE_CHECKS_ENTRY(attention_decode_stream)
extern "C" int forge_decode_attention_stream(const float*, void*, void*, const int32_t*, const int32_t*, const int32_t*, int*, int, int,
                                             int, int, int, int, int, int, int, float, float, int, int, cudaStream_t) {
    return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_attention_stream: built for head sizes 64 and 128 only (this library: %d)", FORGE_ATT_HD);
}

#endif
