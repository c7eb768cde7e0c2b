// bf16 matrix product on the 5th-generation tensor cores:  C[M,N] = A[M,K] . W[N,K]^T, fp32 accumulation
// in tensor memory, operands brought to shared memory by TMA, epilogue fused.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0     TMA producer: for each (tile, k-block) waits for a free stage, arms the stage's barrier with
//              the byte count and issues two tile loads (A box 128 x 64, W box BN x 64, 128-byte swizzle).
//   warp 1     MMA issuer: owns the TMEM allocation (two accumulators of BN columns), waits for a full
//              stage, issues four tcgen05.mma (K = 16 each) per k-block and commits the stage's "empty"
//              barrier; after the last k-block commits the accumulator's "full" barrier.
//   warps 2-5  epilogue: each warp reads its quarter of the 128 TMEM lanes (one output row per thread),
//              32 columns at a time, applies the epilogue and stores to global memory, then releases the
//              accumulator.  Two accumulators let the epilogue of tile i overlap the MMAs of tile i+1.
// Tiles are walked with the row-tile index fastest, so CTAs that run together share a W tile in L2.
// Edges: TMA fills out-of-range rows and the K tail with zeros; the epilogue masks rows >= M, cols >= N.
//
// Epilogues (all arithmetic fp32):
//   0  C fp32  = acc + bias
//   1  C fp32 += acc + bias                      (the residual stream)
//   2  C bf16  = acc + bias
//   3  C bf16[M, N/2]: out[:, j] = silu(acc[:, 2j]) * acc[:, 2j+1]     (gate/up rows interleaved in W)
// Replaces the reference's cuBLAS GemmEx / tiled GEMM / GEMV trio and its separate bias-add, residual-add
// and silu-multiply launches (src/operators/cuda/cuda_quant.cu:582-599, cuda_gemm.cu:7-55,
// cuda_elementwise.cu:8-48).
#include "common.cuh"
#include "checks.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kSmemLimit = 227 * 1024;

enum Epilogue { EPI_STORE_F32 = 0, EPI_ACCUM_F32 = 1, EPI_STORE_BF16 = 2, EPI_SWIGLU_BF16 = 3, EPI_QKV_ROPE = 4 };

struct GemmParams {
    void* C;
    const float* bias;
    int M, N, K;
    int epilogue;
    int* status;
    int tma_out;        // fp32 results leave through shared memory and TMA stores / adds (the kernels that take a map of C)
    // EPI_QKV_ROPE: the product is a step's q, k, v; its epilogue rotates q and k and puts k and v into the paged cache
    const float* rope_table;         // [head_dim / 2, M, 2] (cos, sin) of each row's position, or null: no rotation
    const int32_t* slot_mapping;     // [M] page * page_size + offset of each row's token (negative or null: no cache write)
    __nv_bfloat16* kv_cache;         // [pages, 2, NKV, page_size, head_dim]
    int NH, NKV, head_dim, page_size;
};

template <int BN> struct Cfg {
    static constexpr int kStageBytes = (BM + BN) * BK * 2;
    // the wide tiles (many rows) send fp32 results through two [128 rows x 32 fp32] boxes in shared memory
    static constexpr int kOutBytes = BN >= 128 ? BM * 128 : 0;
    static constexpr int kRingLimit = kSmemLimit - 2048 - 2 * kOutBytes;
    static constexpr int kStages = kRingLimit / kStageBytes > 12 ? 12 : kRingLimit / kStageBytes;
    static constexpr int kTmemCols = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 1024 /*barriers*/ + 2 * kOutBytes;
};

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

// Applies the epilogue to 32 consecutive columns (n .. n+31) of output row m held in r (fp32 bits) and stores them.
template <int BN>
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, const uint32_t (&r)[32], int m, int n) {
    if (m < p.M && n < p.N) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        const int width = min(min(32, BN), p.N - n);
        if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (i < width) v[i] += p.bias[n + i];
        }
        if (p.epilogue == EPI_STORE_F32 || p.epilogue == EPI_ACCUM_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)m * p.N + n;
            const bool acc = p.epilogue == EPI_ACCUM_F32;
            if (width == 32 && (p.N & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    if (acc) {
                        const float4 old = *reinterpret_cast<const float4*>(dst + i);
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    *reinterpret_cast<float4*>(dst + i) = o;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) if (i < width) dst[i] = acc ? dst[i] + v[i] : v[i];
            }
        } else if (p.epilogue == EPI_STORE_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.N + n;
            if (width == 32 && (p.N & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]), h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), h3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                    uint4 o;
                    o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                    o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(dst + i) = o;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) if (i < width) dst[i] = __float2bfloat16_rn(v[i]);
            }
        } else {   // EPI_SWIGLU_BF16: N is even, pairs never straddle a 32-column chunk
            const int half_n = p.N >> 1;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * half_n + (n >> 1);
            if (width == 32 && (half_n & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 16; i += 8) {
                    uint32_t w4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int q = 2 * (i + 2 * j);
                        __nv_bfloat162 h = __floats2bfloat162_rn(silu(v[q]) * v[q + 1], silu(v[q + 2]) * v[q + 3]);
                        w4[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(dst + i) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (2 * i + 1 < width) dst[i] = __float2bfloat16_rn(silu(v[2 * i]) * v[2 * i + 1]);
            }
        }
    }
}

// EPI_QKV_ROPE for one row (token m) of a tile whose columns n0 .. n0 + BN - 1 are whole heads of the fused
// [q heads | k heads | v heads] projection: per head, the HD sums leave tensor memory, get their bias, q and k heads
// are rotated by the row's angles (half-split pairs d, d + HD/2, in fp32, as rope_cache.cu does), everything is
// rounded once to bfloat16, and q goes to C [M, NH*HD], k and v into the cache at the row's slot.  The product never
// exists in global memory in fp32.  (Formulas: src/operators/cuda/cuda_rope.cu:8-34; order of rotation and cache
// update: src/inference/engines/generic_engine.cpp:961-973.)  Control flow is the same for all lanes of a warp.
template <int BN, int HD>
__device__ __forceinline__ void qkv_rope_row(const GemmParams& p, uint32_t t_row, int m, int n0) {
    constexpr int half = HD / 2;
    const bool row_ok = m < p.M;
    int slot = (row_ok && p.slot_mapping && p.kv_cache) ? p.slot_mapping[m] : -1;
    if (slot >= 0 && !FORGE_SLOT_OK(slot)) slot = -1;             // (checks build) a slot outside the pool is not written
    // pair d of row m is at tab[d * M]: the 32 rows of a warp read 256 consecutive bytes per pair
    const float2* tab = p.rope_table ? reinterpret_cast<const float2*>(p.rope_table) + (row_ok ? m : 0) : nullptr;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += HD) {
        const int n = n0 + c0;
        if (n >= p.N) break;
        uint32_t r[HD / 32][32];
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) tmem_ld_32x32b_x32(t_row + c0 + 32 * c, r[c]);
        tmem_ld_wait();
        if (!row_ok) continue;
        const int head = n / HD;
        const bool is_q = head < p.NH, is_v = head >= p.NH + p.NKV;
        float v[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) v[i] = __uint_as_float(r[i / 32][i % 32]) + (p.bias ? __ldg(p.bias + n + i) : 0.f);
        if (!is_v && tab) {
#pragma unroll
            for (int d = 0; d < half; ++d) {
                const float2 cs = __ldg(tab + (size_t)d * p.M);
                const float x0 = v[d], x1 = v[d + half];
                v[d] = x0 * cs.x - x1 * cs.y;
                v[d + half] = x0 * cs.y + x1 * cs.x;
            }
        }
        __nv_bfloat16* dst;
        if (is_q) {
            dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.NH * HD + (size_t)head * HD;
        } else {
            if (slot < 0) continue;
            const int kvh = is_v ? head - p.NH - p.NKV : head - p.NH;
            dst = p.kv_cache + (((size_t)(slot / p.page_size) * 2 + (is_v ? 1 : 0)) * p.NKV + kvh) * p.page_size * HD +
                  (size_t)(slot % p.page_size) * HD;
        }
#pragma unroll
        for (int i = 0; i < HD; i += 8) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]), h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), h3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
            uint4 o;
            o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
            o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + i) = o;
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using C = Cfg<BN>;
    constexpr int kStages = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle pattern to line up with the descriptors
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes);
    uint8_t* out_s = smem + kStages * C::kStageBytes + 1024;      // [2][128 rows][32 fp32], swizzled (wide tiles only)
    uint64_t* full = bars;                       // [kStages]  TMA -> MMA
    uint64_t* empty = bars + kStages;            // [kStages]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * kStages;     // [2]        MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * kStages + 2;  // [2]      epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
        mbar_fence_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    forge::pdl_launch_dependents();
    // A, bias and C may come from (or still be read by) earlier kernels: the thread that copies and the warps that
    // write wait for them below.  W does not: the first tile's first k-blocks of it are asked for before the wait.

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;       // k-blocks issued so far, over all tiles
            bool ok = true;
            uint32_t ahead = 0;    // stages whose W is on its way already
            if ((int)blockIdx.x < num_tiles) {
                const int n0 = ((int)blockIdx.x / tiles_m) * BN;
                ahead = num_kb < kStages ? num_kb : kStages;
                for (uint32_t s = 0; s < ahead; ++s) {
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    tma_load_2d(tiles + s * C::kStageBytes + BM * BK * 2, &tmap_w, &full[s], s * BK, n0);
                }
            }
            forge::pdl_wait();
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    uint8_t* a_dst = tiles + s * C::kStageBytes;
                    if (it < ahead) {              // the first tile's k-block `it`: only A is still to come
                        tma_load_2d(a_dst, &tmap_a, &full[s], kb * BK, m0);
                        continue;
                    }
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&empty[s], ph ^ 1, abort, p.status))) break;
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    tma_load_2d(a_dst, &tmap_a, &full[s], kb * BK, m0);
                    tma_load_2d(a_dst + BM * BK * 2, &tmap_w, &full[s], kb * BK, n0);
                }
            }
            if (!ok) {
                // drain: wait (bounded) for the copies already issued so none lands after the CTA is gone
                const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0;
                for (uint32_t j = first; j < it; ++j) {
                    const unsigned long long t0 = global_ns();
                    while (!mbar_try_wait(&full[j % kStages], (j / kStages) & 1) && global_ns() - t0 < 100000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
            uint32_t it = 0;
            bool ok = true;
            int local = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int a = local & 1;
                const uint32_t aph = (local >> 1) & 1;
                if (!(ok = mbar_wait(&acc_empty[a], aph ^ 1, abort, p.status))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + a * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&full[s], ph, abort, p.status))) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + s * C::kStageBytes);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr), w_desc = umma_desc_k_sw128(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        umma_bf16(d_tmem, umma_desc_advance(a_desc, k * UMMA_K * 2), umma_desc_advance(w_desc, k * UMMA_K * 2),
                                  idesc, k != 0 || kb != 0);
                    }
                    umma_commit(&empty[s]);       // stage is free once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[a]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;              // TMEM lanes this warp may read: 32*quarter .. +31
        const int row_in_tile = quarter * 32 + lane;
        forge::pdl_wait();                         // bias and C: written or still read by earlier kernels
        bool ok = true;
        int local = 0, out_chunk = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int a = local & 1;
            const uint32_t aph = (local >> 1) & 1;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            if (!(ok = mbar_wait(&acc_full[a], aph, abort, p.status))) break;
            tc_fence_after_sync();
            const int m = m0 + row_in_tile;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN;
            if constexpr (C::kOutBytes > 0) {
                if (p.tma_out) {
                    // fp32 results: a chunk of 32 columns of all 128 rows goes to shared memory (the layout of a
                    // 128-byte-swizzled box) and from there to global memory with one TMA instruction, a store
                    // or an add that the L2 performs; the four warps meet at a named barrier around each chunk,
                    // and two buffers let a chunk be written while the previous one is read
                    const bool issuer = threadIdx.x == 64;
#pragma unroll 1
                    for (int c = 0; c < BN; c += 32) {
                        if (n0 + c >= p.N) break;
                        uint8_t* buf = out_s + (out_chunk++ & 1) * C::kOutBytes;
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(t_row + c, r);
                        if (issuer) bulk_wait_group_read<1>();      // the copy that read this buffer two chunks ago
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        tmem_ld_wait();
                        if (p.bias) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (n0 + c + i < p.N) r[i] = __float_as_uint(__uint_as_float(r[i]) + p.bias[n0 + c + i]);
                        }
                        uint8_t* row = buf + row_in_tile * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<uint4*>(row + ((j ^ (row_in_tile & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        fence_proxy_async();
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (issuer) {
                            if (p.epilogue == EPI_ACCUM_F32) tma_reduce_add_2d(&tmap_c, buf, n0 + c, m0);
                            else tma_store_2d(&tmap_c, buf, n0 + c, m0);
                            bulk_commit_group();
                        }
                    }
                    tc_fence_before_sync();
                    mbar_arrive(&acc_empty[a]);
                    continue;
                }
            }
            if constexpr (BN % 128 == 0) {
                if (p.epilogue == EPI_QKV_ROPE) {
                    if (p.head_dim == 64) qkv_rope_row<BN, 64>(p, t_row, m, n0);
                    else qkv_rope_row<BN, 128>(p, t_row, m, n0);
                    tc_fence_before_sync();
                    mbar_arrive(&acc_empty[a]);
                    continue;
                }
            }
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                if constexpr (BN >= 32) {
                    tmem_ld_32x32b_x32(t_row + c, r);
                } else {
                    uint32_t h[16];
                    tmem_ld_32x32b_x16(t_row + c, h);
#pragma unroll
                    for (int i = 0; i < 16; ++i) { r[i] = h[i]; r[i + 16] = 0; }
                }
                tmem_ld_wait();
                store_row_chunk<BN>(p, r, m, n0 + c);
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[a]);
        }
        if (C::kOutBytes > 0 && p.tma_out && threadIdx.x == 64) bulk_wait_group<0>();   // results are in global memory before the CTA leaves
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------
// Many rows, two CTAs on one tile (tcgen05 cta_group::2).
//
// A k-step of the single-CTA [128 x 256] tile moves 24 KB through an SM's shared memory (TMA writes 12 KB, the
// tensor core reads them) at 128 B per clock: 188 clocks for 128 clocks of arithmetic.  Here the two CTAs of a
// cluster share a [256 x 256] tile: CTA r stages rows r*128.. of A and rows r*128.. of W (half of the tile's N
// side), 8 KB per k-step each, and ONE thread of the even CTA issues MMAs of M = 256, N = 256 that read both
// CTAs' shared memory and accumulate rows r*128.. of the tile into CTA r's tensor memory.  Per SM that is
// 16 KB per 128 clocks: the arithmetic is the bound again (measured: 125 clocks per MMA in the main loop).
//   Barriers.  full[s] lives in the even CTA only: both CTAs' TMA loads complete their bytes on it (a
// cta_group::2 load may signal its pair's barrier), the even CTA's producer arms it with both CTAs' byte count.
// empty[s] and acc_full[a] exist in both CTAs and are arrived on by multicast commits.  acc_empty[a] lives in
// the even CTA and collects the 256 epilogue threads of both.  Two accumulators of 256 columns fill the tensor
// memory of each CTA, so the epilogue of one tile overlaps the MMAs of the next.
//   G: k-blocks per stage and TMA instruction (through the 3D k-block views); G = 0: 2D maps, one k-block per
// stage, for a K that is no multiple of 64.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
constexpr int kPairBN = 256;                                   // N of the pair's tile; each CTA stages half of it
// PBN: the tile's N (256; 128 or 192 where narrower tiles fill the last wave better)
template <int PBN> struct PairCfgT {
    static constexpr int kBlockBytes = (BM + PBN / 2) * BK * 2;             // one k-block per CTA: 32 KB at 256
    static constexpr int kRingBlocks = 6;                                   // 192 KB of stages at most, whatever their size
    static constexpr int kOutBytes = BM * 128;                              // a [128 rows x 32 fp32] box of results
    static constexpr int kSmemBytes = kRingBlocks * kBlockBytes + 1024 + 1024 + 2 * kOutBytes;
    static constexpr int kTmemCols = 512;
};
using PairCfg = PairCfgT<kPairBN>;

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Tile loads into this CTA's shared memory whose bytes complete on `bar_cluster_addr`, a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs of the pair once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int G, int PBN = kPairBN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_sm100_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                       const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using C = PairCfgT<PBN>;
    constexpr int g = G > 0 ? G : 1;
    constexpr int kStages = C::kRingBlocks / g, BNH = PBN / 2;
    constexpr int kABytes = g * BM * BK * 2, kStageBytes = g * C::kBlockBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;                         // [kStages][ g tiles of A | g tiles of this CTA's half of W ]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kRingBlocks * C::kBlockBytes);
    uint8_t* out_s = smem + C::kRingBlocks * C::kBlockBytes + 1024;       // [2][128 rows][32 fp32], swizzled
    uint64_t* full = bars;                         // [kStages]  both CTAs' TMA -> the even CTA's MMA thread
    uint64_t* empty = bars + kStages;              // [kStages]  MMA -> each CTA's TMA thread
    uint64_t* acc_full = bars + 2 * kStages;       // [2]        MMA -> each CTA's epilogue
    uint64_t* acc_empty = bars + 2 * kStages + 2;  // [2]        both CTAs' epilogues -> the even CTA's MMA thread
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles_n = (p.N + PBN - 1) / PBN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + BK - 1) / BK;
    const int num_groups = (num_kb + g - 1) / g;               // stages per tile; the last may hold fewer k-blocks

    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 256); }
        mbar_fence_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                    // both CTAs' barriers exist before either signals across
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    forge::pdl_launch_dependents();
    // A, bias and C may come from (or still be read by) earlier kernels: the threads that copy and the warps that
    // write wait for them below.  W does not: the first tile's first stages of it are asked for before the wait.

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint32_t full0 = map_to_cta(smem_u32(&full[0]), 0);
            uint32_t ahead = 0;                // stages whose W is on its way already
            if (pair < num_tiles) {
                const int n0 = (pair / tiles_m) * PBN + rank * BNH;
                ahead = num_groups < kStages ? num_groups : kStages;
                for (uint32_t s = 0; s < ahead; ++s) {
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kStageBytes);
                    const uint32_t bar = full0 + s * 8;
                    uint8_t* w_dst = tiles + s * kStageBytes + kABytes;
                    if constexpr (G > 0) tma_load_3d_pair(w_dst, &tmap_w, bar, 0, n0, (int)s * g);
                    else tma_load_2d_pair(w_dst, &tmap_w, bar, (int)s * BK, n0);
                }
            }
            forge::pdl_wait();
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile % tiles_m) * 2 * BM + rank * BM, n0 = (tile / tiles_m) * PBN + rank * BNH;
                for (int gi = 0; gi < num_groups; ++gi, ++it) {
                    const int s = it % kStages;
                    const uint32_t bar = full0 + s * 8;
                    uint8_t* a_dst = tiles + s * kStageBytes;
                    if (it < ahead) {              // the first tile's stage `it`: only A is still to come
                        if constexpr (G > 0) tma_load_3d_pair(a_dst, &tmap_a, bar, 0, m0, gi * g);
                        else tma_load_2d_pair(a_dst, &tmap_a, bar, gi * BK, m0);
                        continue;
                    }
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&empty[s], ph ^ 1, abort, p.status))) break;
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kStageBytes);   // k-blocks past K arrive as zeros
                    if constexpr (G > 0) {
                        tma_load_3d_pair(a_dst, &tmap_a, bar, 0, m0, gi * g);
                        tma_load_3d_pair(a_dst + kABytes, &tmap_w, bar, 0, n0, gi * g);
                    } else {
                        tma_load_2d_pair(a_dst, &tmap_a, bar, gi * BK, m0);
                        tma_load_2d_pair(a_dst + kABytes, &tmap_w, bar, gi * BK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (the even CTA's)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(2 * BM, PBN);
            uint32_t it = 0;
            bool ok = true;
            int local = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const int a = local & 1;
                const uint32_t aph = (local >> 1) & 1;
                if (!(ok = mbar_wait(&acc_empty[a], aph ^ 1, abort, p.status))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + a * PBN;
                for (int gi = 0; gi < num_groups; ++gi, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&full[s], ph, abort, p.status))) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + s * kStageBytes);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr), w_desc = umma_desc_k_sw128(a_addr + kABytes);
                    const int here = min(g, num_kb - gi * g);
#pragma unroll
                    for (int j = 0; j < g; ++j) {
                        if (j >= here) break;
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16_pair(d_tmem, umma_desc_advance(a_desc, j * (BM * BK * 2) + k * UMMA_K * 2),
                                           umma_desc_advance(w_desc, j * (BNH * BK * 2) + k * UMMA_K * 2), idesc,
                                           (j | k) != 0 || gi != 0);
                    }
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[a]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5 of each CTA)
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
        forge::pdl_wait();                         // bias, C and what the epilogue reads beside them: earlier kernels' to finish with
        bool ok = true;
        int local = 0, out_chunk = 0;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
            const int a = local & 1;
            const uint32_t aph = (local >> 1) & 1;
            const int m0 = (tile % tiles_m) * 2 * BM + rank * BM, n0 = (tile / tiles_m) * PBN;
            if (!(ok = mbar_wait(&acc_full[a], aph, abort, p.status))) break;
            tc_fence_after_sync();
            const int m = m0 + row_in_tile;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * PBN;
            if (p.tma_out) {
                // fp32 results: a chunk of 32 columns of all 128 rows goes to shared memory (the layout of a
                // 128-byte-swizzled box) and from there to global memory with one TMA instruction, a store or
                // an add that the L2 performs; the four warps meet at a named barrier around each chunk, and
                // two buffers let a chunk be written while the previous one is read
                const bool issuer = threadIdx.x == 64;
#pragma unroll 1
                for (int c = 0; c < PBN; c += 32) {
                    if (n0 + c >= p.N) break;
                    uint8_t* buf = out_s + (out_chunk++ & 1) * C::kOutBytes;      // the buffers alternate across tiles too
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_row + c, r);
                    if (issuer) bulk_wait_group_read<1>();          // the copy that read this buffer two chunks ago
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    tmem_ld_wait();
                    if (p.bias) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c + i < p.N) r[i] = __float_as_uint(__uint_as_float(r[i]) + p.bias[n0 + c + i]);
                    }
                    uint8_t* row = buf + row_in_tile * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(row + ((j ^ (row_in_tile & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    fence_proxy_async();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (issuer && m0 < p.M) {
                        if (p.epilogue == EPI_ACCUM_F32) tma_reduce_add_2d(&tmap_c, buf, n0 + c, m0);
                        else tma_store_2d(&tmap_c, buf, n0 + c, m0);
                        bulk_commit_group();
                    }
                }
            } else if (p.epilogue == EPI_QKV_ROPE) {
                // whole heads per tile: rotated and rounded once, q to C, k and v into the cache
                if (p.head_dim == 64) qkv_rope_row<PBN, 64>(p, t_row, m, n0);
                else if constexpr (PBN % 128 == 0) qkv_rope_row<PBN, 128>(p, t_row, m, n0);
            } else {
#pragma unroll 1
                for (int c = 0; c < PBN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_row + c, r);
                    tmem_ld_wait();
                    store_row_chunk<PBN>(p, r, m, n0 + c);
                }
            }
            tc_fence_before_sync();
            mbar_arrive_cluster(acc_empty0 + a * 8);
        }
        if (p.tma_out && threadIdx.x == 64) bulk_wait_group<0>();   // the results are in global memory before the CTA leaves
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                    // the pair's MMAs read both CTAs' shared memory: leave together
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
    }
}

__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------------------
// Some hundred rows, few tiles: K cut across a cluster.
//
// A product of 129 to about 1,000 rows onto a narrow matrix (the o and down projections of a prompt of 512 tokens:
// [512 x 2048]) makes 64 tiles of 128 x 128, so fewer than half of the SMs work, and each of them has to take in its
// whole share of both operands (1 MB a tile at K = 2048) at the 60 GB/s that an SM's copies deliver: 17 of the 20 us
// such a product takes.  Here the 2 or 4 CTAs of a cluster share one tile and cut K between them, so twice or four
// times the SMs take the operands in.  Each CTA parks its [128 x 128] fp32 partial in shared memory (the ring of
// stages is free by then; 16-byte chunk j of row m at chunk j ^ (m % 32), which both the writers, a row per thread,
// and the readers, a row per warp, touch without bank conflicts), the cluster synchronises, and every CTA then adds
// up, in rank order (so the result does not depend on timing), the rows it owns, adds the bias and writes C: a
// store, or one add per element into the residual stream.  fp32 results only (no bf16 or SwiGLU epilogue).
// G: k-blocks per TMA instruction and ring slot (the matrix seen as {64 columns, rows, K / 64 k-blocks}); G = 1 is the
// form for a K that is no multiple of 64 (plain 2-D maps).  Measured on the o-projection of 512 rows inside a prompt
// step: 14.7 us with one k-block per instruction, 13.9 with two, 11.2 with the reduction asking for four rows' shares
// before it uses the first.  Tiles of [128 x 256] cut four ways (a third fewer bytes per SM) were slower at every size
// tried (512 rows: o 13.5, down 21.5 against 19.6 us): a CTA's time here is a chain of short phases, not its bytes.
constexpr int kSplitBN = 128;
template <int G>
struct SplitKCfg {
    static constexpr int kStageBytes = G * (BM + kSplitBN) * BK * 2;        // 32 KB per k-block
    static constexpr int kStages = 6 / G;                                   // a ring of 192 KB
    static constexpr int kPartialBytes = BM * kSplitBN * 4;                 // 64 KB, parked in the ring once its slots are free
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
    static constexpr int kTmemCols = kSplitBN;
    static_assert(kPartialBytes <= kStages * kStageBytes, "the partial sums take the ring's place");
};

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
gemm_sm100_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                         const GemmParams p, const int ksplit) {
    using C = SplitKCfg<G>;
    constexpr int kStages = C::kStages, BN = kSplitBN;
    constexpr int kTileA = BM * BK * 2, kTileW = BN * BK * 2;                            // one k-block of either operand
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;                                                               // slot: G tiles of A, then G tiles of W
    float* partial = reinterpret_cast<float*>(smem);       // [128 rows][BN / 4 chunks of 4], swizzled; written when the last product has read the ring
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + kStages;
    uint64_t* acc_full = bars + 2 * kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());
    const int tiles_m = (p.M + BM - 1) / BM;
    const int tile = blockIdx.x / ksplit;
    const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
    const int num_kb = (p.K + BK - 1) / BK;
    const int kb_per = (num_kb + ksplit - 1) / ksplit;
    const int kb_begin = rank * kb_per, kb_end = min(kb_begin + kb_per, num_kb);
    const int my_kb = max(kb_end - kb_begin, 0);

    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        mbar_fence_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    forge::pdl_launch_dependents();

    const int my_groups = (my_kb + G - 1) / G;          // ring slots this CTA fills (the last may hold fewer k-blocks)
    // one operand's G k-blocks of slot `i`: one instruction (a box beyond this CTA's share or beyond K brings the
    // neighbour's k-blocks or zeros, which no product reads)
    auto load_a = [&](int i, uint64_t* bar) {
        uint8_t* dst = tiles + (i % kStages) * C::kStageBytes;
        if constexpr (G == 1) tma_load_2d(dst, &tmap_a, bar, (kb_begin + i) * BK, m0);
        else tma_load_3d(dst, &tmap_a, bar, 0, m0, kb_begin + i * G);
    };
    auto load_w = [&](int i, uint64_t* bar) {
        uint8_t* dst = tiles + (i % kStages) * C::kStageBytes + G * kTileA;
        if constexpr (G == 1) tma_load_2d(dst, &tmap_w, bar, (kb_begin + i) * BK, n0);
        else tma_load_3d(dst, &tmap_w, bar, 0, n0, kb_begin + i * G);
    };
    if (warp == 0) {
        if (lane == 0) {
            // the weights do not depend on earlier kernels: their first stages are requested before the wait
            const int first = min(my_groups, kStages);
            for (int i = 0; i < first; ++i) {
                mbar_arrive_expect_tx(&full[i], C::kStageBytes);
                load_w(i, &full[i]);
            }
            forge::pdl_wait();                    // the activations come from the previous kernel
            for (int i = 0; i < first; ++i) load_a(i, &full[i]);
            bool ok = true;
            for (int i = first; i < my_groups && ok; ++i) {
                const int s = i % kStages;
                if (!(ok = mbar_wait(&empty[s], ((i / kStages) - 1) & 1, abort, p.status))) break;
                mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                load_a(i, &full[s]);
                load_w(i, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
            bool ok = true;
            for (int i = 0; i < my_groups && ok; ++i) {
                const int s = i % kStages;
                if (!(ok = mbar_wait(&full[s], (i / kStages) & 1, abort, p.status))) break;
                tc_fence_after_sync();
                const uint32_t slot = smem_u32(tiles + s * C::kStageBytes);
                const int n_here = min(G, my_kb - i * G);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    if (g >= n_here) break;
                    const uint64_t a_desc = umma_desc_k_sw128(slot + g * kTileA), w_desc = umma_desc_k_sw128(slot + G * kTileA + g * kTileW);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(tmem_base, umma_desc_advance(a_desc, k * UMMA_K * 2), umma_desc_advance(w_desc, k * UMMA_K * 2),
                                  idesc, k != 0 || g != 0 || i != 0);
                }
                umma_commit(&empty[s]);
            }
            if (ok && my_kb > 0) umma_commit(acc_full);
        }
    } else {
        // warps 2..5: this CTA's partial sums out of tensor memory, a row per thread
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        forge::pdl_wait();                        // C and bias: written or still read by earlier kernels
        bool ok = true;
        if (my_kb > 0) ok = mbar_wait(acc_full, 0, abort, p.status);
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        float4* prow = reinterpret_cast<float4*>(partial) + row * (BN / 4);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
            uint32_t r[32];
            if (my_kb > 0 && ok) {
                tmem_ld_32x32b_x32(t_row + c, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                prow[((c >> 2) + j) ^ (row & 31)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();                       // every CTA's partial is in place and visible

    if (warp >= 2) {
        // this CTA owns rows [rank * 128 / ksplit, (rank + 1) * 128 / ksplit) of the tile; a warp takes a row at a
        // time, a lane 16 bytes of each 128 columns of it
        const int row_lo = rank * BM / ksplit, row_hi = (rank + 1) * BM / ksplit;
        const uint32_t partial_addr = smem_u32(partial);
        constexpr int kHalves = BN / 128;
        float4 b[kHalves];
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
            const int n = n0 + 128 * h + 4 * lane;
            b[h] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.bias) {
                if (n + 3 < p.N) b[h] = *reinterpret_cast<const float4*>(p.bias + n);
                else { if (n < p.N) b[h].x = p.bias[n]; if (n + 1 < p.N) b[h].y = p.bias[n + 1]; if (n + 2 < p.N) b[h].z = p.bias[n + 2]; }
            }
        }
        // several rows' shares are asked for before the first is used: a load from a peer's shared memory takes some
        // hundred clocks, and one row after the other was a chain of them
        constexpr int kAhead = 4 / kHalves;
        const bool accum = p.epilogue == EPI_ACCUM_F32;
        for (int first = row_lo + (warp - 2); first < row_hi; first += 4 * kAhead) {
            float4 v[kAhead][kHalves][4];
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int row = first + 4 * j;
                if (row >= row_hi) break;
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    const uint32_t at = partial_addr + (row * (BN / 4) + 32 * h + (lane ^ (row & 31))) * 16;
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (q < ksplit) v[j][h][q] = ld_dsmem_f32x4(at, q);
                }
            }
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int row = first + 4 * j, m = m0 + row;
                if (row >= row_hi) break;
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    const int n = n0 + 128 * h + 4 * lane;
                    float4 acc = b[h];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (q < ksplit) { acc.x += v[j][h][q].x; acc.y += v[j][h][q].y; acc.z += v[j][h][q].z; acc.w += v[j][h][q].w; }
                    if (m >= p.M || n >= p.N) continue;
                    float* dst = reinterpret_cast<float*>(p.C) + (size_t)m * p.N + n;
                    if (n + 3 < p.N && (p.N & 3) == 0) {
                        if (accum) atomicAdd(reinterpret_cast<float4*>(dst), acc);       // one add per element: the order of CTAs does not matter
                        else *reinterpret_cast<float4*>(dst) = acc;
                    } else {
                        const float e[4] = {acc.x, acc.y, acc.z, acc.w};
                        for (int i = 0; i < 4; ++i) {
                            if (n + i >= p.N) break;
                            if (accum) atomicAdd(dst + i, e[i]);
                            else dst[i] = e[i];
                        }
                    }
                }
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                       // nobody leaves while a peer may still read its partial
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------
// Few rows (decode): the weight matrix is the MMA's M operand.
//
// With M <= 64 tokens the product is a stream of weights through the SMs: what matters is that every SM
// has many bytes of W in flight and that no byte is loaded twice.  So here a CTA takes 128 rows of W
// (all 16 KB of each 128 x 64 tile are useful bytes; the tokens are the narrow N side, padded to 16/32/64
// by TMA's zero fill) and only a slice of K; the `kSplit` CTAs of a thread-block cluster share one row
// tile and cut K between them, which gives enough CTAs to cover the GPU even when N is small.  Their
// partial sums meet in distributed shared memory: every CTA parks its [tokens x 128] fp32 partial in its
// own shared memory, the cluster synchronises, and each CTA then adds up, in rank order (so the result
// does not depend on timing), the slice of rows it owns, applies the epilogue and writes C.  No scratch
// in global memory, no atomics.
//
// One TMA instruction keeps an SM's copy engine busy for about one memory latency (measured: ~0.4 us from
// DRAM, the same for boxes of 8, 16, 32 and 64 KB, and no faster with more instructions in flight), so an SM
// that asks for one 16 KB k-block at a time pulls 45 GB/s whatever the depth of its pipeline.  A stage here
// is therefore a GROUP of up to 4 consecutive k-blocks brought by one instruction per operand: the matrix
// [rows, K] is described to TMA as {64 columns, rows, K / 64 k-blocks} (k-block stride 128 bytes), and a box
// {64, 128, g} lands in shared memory as g standard 128-byte-swizzled [128 x 64] tiles one after the other.
// That needs K % 64 == 0; other K take the plain 2D map with one k-block per stage.
// Two threads issue the MMAs (warps 1 and 6), each into an accumulator of its own: one thread gets a
// tcgen05.mma out about every 50 clocks, and an M128 N16 K16 MMA that reads its M operand from shared memory
// keeps the tensor pipe busy for about 39 (measured: 54.8 clocks per MMA with one issuing thread, 2 x 1024 MMAs
// in 78.4 clocks per pair with two).  The k-blocks of a stage alternate between the two; the epilogue adds the
// two accumulators (always in the same order).
constexpr int kSkinnyThreads = 224;
template <int NT> struct SkinnyCfg {                       // NT: token box (UMMA N) = 16, 32 or 64
    // one k-block of W (`rows` weight rows of 128 bytes) and of the tokens
    static constexpr int block_bytes(int rows) { return rows * BK * 2 + NT * BK * 2; }
    static constexpr int kPartialBytes = NT * BM * 4;
    // k-blocks per TMA instruction at most: four at 16 tokens (three stages of 72 KB); at 32 and 64 tokens a k-block is
    // 20 / 24 KB and groups of four leave room for two stages only: up to three (in practice two, which divide the
    // k-blocks evenly: five / four stages) measured 1.5 % faster per step; 128 tokens: a k-block is 32 KB, two per stage
    static constexpr int kMaxGroup = NT <= 16 ? 4 : (NT <= 64 ? 3 : 2);
    static constexpr int kMaxStages = 12;
    static constexpr int max_stages(int group, int rows) {
        const int fit = (kSmemLimit - 2048 - kPartialBytes) / (group * block_bytes(rows));
        return fit > kMaxStages ? kMaxStages : fit;
    }
    static constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;      // two accumulators, one per issuing thread
    // a CTA takes only as many stages as it has work for, so that CTAs of the next kernel fit beside it
    static constexpr int smem_bytes(int stages, int group, int rows) { return stages * group * block_bytes(rows) + kPartialBytes + 1024 + 1024; }
};

template <int NT>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_sm100_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                         const GemmParams p, const int ksplit, const int kStages, const int group, const int tile_rows) {
    // group > 0: the maps are the 3D k-block views and a stage holds `group` k-blocks; group == 0: 2D maps,
    // one k-block per stage.
    // tile_rows (a multiple of 8, at most 128): weight rows per CTA.  What bounds a product of few rows is how many
    // bytes the GPU has in flight, i.e. how many SMs stream: a matrix of 88 tiles of 128 rows leaves 60 SMs idle,
    // 141 tiles of 80 rows do not.  The MMA is M = 128 all the same: a tile's k-blocks lie tile_rows * 128 bytes
    // apart in shared memory, the rows beyond tile_rows that the tensor core reads belong to whatever follows
    // there, and the sums they produce (rows of the accumulator that no row of C corresponds to) are never read.
    using C = SkinnyCfg<NT>;
    const int g = group > 0 ? group : 1;
    const int w_block = tile_rows * BK * 2;                                 // one k-block of the tile
    const int w_bytes = g * w_block, x_bytes = g * NT * BK * 2;           // one stage of each operand
    const int x_region = kStages * x_bytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* w_tiles = smem;                                   // [kStages][g][128 x 64]
    uint8_t* x_tiles = smem + kStages * w_bytes;               // [kStages][g][NT x 64]
    float* partial = reinterpret_cast<float*>(x_tiles + x_region);          // [NT][BM]
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_tiles + x_region + C::kPartialBytes);
    uint64_t* full = bars;
    uint64_t* acc_full = bars + C::kMaxStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kMaxStages + 1);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // A stage is used once per CTA when the CTA has at most kStages groups; beyond that the producer
    // reuses stage s for group s + kStages once the MMA warp has committed it (signalled through `reuse`).
    uint64_t* reuse = bars + C::kMaxStages + 2;   // [kStages] MMA -> TMA

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int n0 = (blockIdx.x / ksplit) * tile_rows;
    const int num_kb = (p.K + BK - 1) / BK;
    // a CTA's last group may reach into the next CTA's k-blocks: those bytes are loaded and not multiplied
    const int kb_per = (num_kb + ksplit - 1) / ksplit;
    const int kb_begin = rank * kb_per, kb_end = min(kb_begin + kb_per, num_kb);
    const int my_kb = max(kb_end - kb_begin, 0);
    const int my_groups = (my_kb + g - 1) / g;

    // a group that sticks out over the end of K is filled with zeros there and counts in full
    const int stage_tx = w_bytes + x_bytes;
    auto load_w = [&](int i, int s) {
        if (group > 0) tma_load_3d(w_tiles + s * w_bytes, &tmap_w, &full[s], 0, n0, kb_begin + i * g);
        else tma_load_2d(w_tiles + s * w_bytes, &tmap_w, &full[s], (kb_begin + i) * BK, n0);
    };
    const int first = min(my_groups, kStages);           // the stages that are filled without waiting for a free one
    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&reuse[s], 2); }
        mbar_init(acc_full, 2);
        mbar_fence_init();
        // The weights depend on nothing that runs before this kernel: this thread, which is the one that copies, asks
        // for their first stages as soon as the barriers they report to exist, ahead of the CTA's other set-up and of
        // the dependency wait.
        for (int i = 0; i < first; ++i) {
            mbar_arrive_expect_tx(&full[i], stage_tx);
            load_w(i, i);
        }
        prefetch_tensormap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const bool two_acc = g >= 2 && my_kb >= 2;           // the second issuing thread has k-blocks of its own
    // An unsplit tile with few tokens and an fp32 result goes straight from tensor memory to C; every other case
    // passes through `partial` in shared memory, where a thread then holds four neighbouring features of a token
    // (vector stores, gate and up side by side) instead of one feature of every token.
    const bool direct = ksplit == 1 && p.epilogue <= EPI_ACCUM_F32 && p.M <= 16;
    forge::pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            auto load_x = [&](int i, int s) {
                if (group > 0) tma_load_3d(x_tiles + s * x_bytes, &tmap_x, &full[s], 0, 0, kb_begin + i * g);
                else tma_load_2d(x_tiles + s * x_bytes, &tmap_x, &full[s], (kb_begin + i) * BK, 0);
            };
            // (the weights of the first stages were asked for during the set-up)
            forge::pdl_wait();                    // the activations come from the previous kernel
            for (int i = 0; i < first; ++i) load_x(i, i);
            bool ok = true;
            for (int i = first; i < my_groups && ok; ++i) {
                const int s = i % kStages;
                if (!(ok = mbar_wait(&reuse[s], ((i / kStages) - 1) & 1, abort, p.status))) break;
                mbar_arrive_expect_tx(&full[s], stage_tx);
                load_w(i, s);
                load_x(i, s);
            }
        }
    } else if (warp == 1 || warp == 6) {
        if (lane == 0) {
            // issuer 0 (warp 1) takes k-blocks 0 and 2 of every group, issuer 1 (warp 6) k-blocks 1 and 3
            const int who = warp == 1 ? 0 : 1;
            const uint32_t d_tmem = tmem_base + who * NT;
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, NT);
            bool ok = true, fresh = true;
            for (int i = 0; i < my_groups && ok; ++i) {
                const int s = i % kStages;
                if (!(ok = mbar_wait(&full[s], (i / kStages) & 1, abort, p.status))) break;
                tc_fence_after_sync();
                const uint64_t w_desc = umma_desc_k_sw128(smem_u32(w_tiles + s * w_bytes));
                const uint64_t x_desc = umma_desc_k_sw128(smem_u32(x_tiles + s * x_bytes));
                const int here = min(g, my_kb - i * g);            // k-blocks of this group inside my range
#pragma unroll
                for (int jj = 0; jj < (C::kMaxGroup + 1) / 2; ++jj) {
                    const int j = 2 * jj + who;
                    if (j >= here) break;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(d_tmem, umma_desc_advance(w_desc, j * w_block + k * UMMA_K * 2),
                                  umma_desc_advance(x_desc, j * (NT * BK * 2) + k * UMMA_K * 2), idesc, !(fresh && k == 0));
                    fresh = false;
                }
                umma_commit(&reuse[s]);           // one of the two arrivals that free the stage
            }
            if (ok && my_kb > 0) umma_commit(acc_full);
        }
    } else {
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;
        forge::pdl_wait();                        // C and bias: written or still read by earlier kernels
        bool ok = true;
        if (my_kb > 0) ok = mbar_wait(acc_full, 0, abort, p.status);
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        // 16 tokens of this thread's row: the first issuer's accumulator plus, if it had work, the second's
        auto load_acc = [&](int c, uint32_t (&r)[16]) {
            tmem_ld_32x32b_x16(t_row + c, r);
            if (two_acc) {
                uint32_t r2[16];
                tmem_ld_32x32b_x16(t_row + NT + c, r2);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
            } else {
                tmem_ld_wait();
            }
        };
        if (direct) {
            // the whole reduction happened in this CTA: straight from tensor memory to C.  A thread holds
            // one weight row n for all tokens, so for each token a warp writes 32 consecutive columns.
            // rows of the accumulator beyond the tile's own are not rows of C
            const int n = n_local < tile_rows ? n0 + n_local : p.N;
            const float b = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            if (ok) {
#pragma unroll
                for (int c = 0; c < NT; c += 16) {
                    uint32_t r[16];
                    load_acc(c, r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int m = c + i;
                        if (m >= p.M) break;                       // uniform over the warp
                        const float v = __uint_as_float(r[i]) + b;
                        if (p.epilogue == EPI_SWIGLU_BF16) {
                            const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                            if ((lane & 1) == 0 && n + 1 < p.N)
                                reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * (p.N >> 1) + (n >> 1)] =
                                    __float2bfloat16_rn(silu(v) * other);
                        } else if (n < p.N) {
                            if (p.epilogue == EPI_STORE_BF16) {
                                reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
                            } else {
                                // the residual add is a reduction that the L2 performs: nothing is read back, so
                                // the kernel's last step is a store either way (one add per element: the order
                                // of CTAs does not matter)
                                float* dst = reinterpret_cast<float*>(p.C) + (size_t)m * p.N + n;
                                if (p.epilogue == EPI_ACCUM_F32) atomicAdd(dst, v);
                                else *dst = v;
                            }
                        }
                    }
                }
            }
        } else if (my_kb > 0 && ok) {
            // park this CTA's partial [token][row] in shared memory for the cluster-wide sum
#pragma unroll
            for (int c = 0; c < NT; c += 16) {
                uint32_t r[16];
                load_acc(c, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) partial[(c + i) * BM + n_local] = __uint_as_float(r[i]);
            }
        } else {
            for (int m = 0; m < NT; ++m) partial[m * BM + n_local] = 0.f;
        }
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();                       // every CTA's partial is in place and visible

    if (warp >= 2 && warp < 6 && !direct) {
        // this CTA owns a share of the tile's rows: add the partials in rank order, four
        // adjacent rows (16 bytes of each peer's shared memory) per thread
        // (the tile's groups of four rows are dealt out as evenly as the cluster's size allows)
        const int group0 = (int)rank * (tile_rows / 4) / ksplit, groups = ((int)rank + 1) * (tile_rows / 4) / ksplit - group0;
        const int t = threadIdx.x - 64;                    // 0..127
        const uint32_t partial_addr = smem_u32(partial);
        for (int idx = t; idx < p.M * groups; idx += 128) {
            const int m = idx / groups, nl = 4 * (group0 + idx % groups);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int q = 0; q < ksplit; ++q) {
                const float4 v = ld_dsmem_f32x4(partial_addr + (m * BM + nl) * 4, q);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            const int n = n0 + nl;
            float v[4] = {acc.x, acc.y, acc.z, acc.w};
            if (p.bias) {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (n + i < p.N) v[i] += p.bias[n + i];
            }
            if (p.epilogue == EPI_SWIGLU_BF16) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * (p.N >> 1) + (n >> 1);
                if (n + 1 < p.N) dst[0] = __float2bfloat16_rn(silu(v[0]) * v[1]);
                if (n + 3 < p.N) dst[1] = __float2bfloat16_rn(silu(v[2]) * v[3]);
            } else if (p.epilogue == EPI_STORE_BF16) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.N + n;
#pragma unroll
                for (int i = 0; i < 4; ++i) if (n + i < p.N) dst[i] = __float2bfloat16_rn(v[i]);
            } else {
                float* dst = reinterpret_cast<float*>(p.C) + (size_t)m * p.N + n;
                const bool accum = p.epilogue == EPI_ACCUM_F32;
                // (the residual add is a reduction that the L2 performs: nothing is read back)
                if (n + 3 < p.N && (p.N & 3) == 0) {
                    const float4 o = make_float4(v[0], v[1], v[2], v[3]);
                    if (accum) atomicAdd(reinterpret_cast<float4*>(dst), o);
                    else *reinterpret_cast<float4*>(dst) = o;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (n + i >= p.N) continue;
                        if (accum) atomicAdd(dst + i, v[i]);
                        else dst[i] = v[i];
                    }
                }
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                       // nobody leaves while a peer may still read its partial
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------
// Few rows, every SM busy: the same weight-major tiles, but the (row tile, k-block) units of work are dealt
// out evenly to one persistent CTA per SM ("stream-K").  A CTA walks its contiguous range of units, which
// may end in the middle of one row tile and continue into the next; each piece of a tile it computes is a
// FRAGMENT.  The fragment that holds a tile's last k-blocks owns the tile: it waits for the other
// fragments' partial sums (written to a workspace in global memory, announced by a flag), adds them in
// fragment order (so the sum never depends on timing), applies the epilogue and writes C.  The producers
// of those partials are CTAs with lower indices, which hold an SM since before the owner started, so the
// wait cannot starve; it is bounded all the same.
//   Because the units are equal, all SMs stream the same number of weight bytes whatever N is: this is what
// makes a [2048 x 2048] projection (16 row tiles) use 128+ SMs and a [11264 x 2048] one (88 tiles) use all.
template <int NT> struct StreamKCfg {
    static constexpr int kStageBytes = BM * BK * 2 + NT * BK * 2;
    static constexpr int kStages = (kSmemLimit - 2048) / kStageBytes > 12 ? 12 : (kSmemLimit - 2048) / kStageBytes;
    static constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;
    static constexpr int smem_bytes(int stages) { return stages * kStageBytes + 1024 + 1024; }
};

struct StreamKWork {
    float* partials;      // [tiles_n][max_parts][NT][128]
    int* flags;           // [tiles_n][max_parts], zero between launches
    int per_cta;          // units per CTA
    int max_parts;
};

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

constexpr int kStreamKThreads = 224;       // warps 0 and 6 load, 1 issues the MMAs, 2..5 are the epilogue
template <int NT>
__global__ void __launch_bounds__(kStreamKThreads, 1)
gemm_sm100_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                          const GemmParams p, const StreamKWork wk, const int kStages) {
    using C = StreamKCfg<NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes);
    uint64_t* full = bars;                          // [kStages]
    uint64_t* empty = bars + C::kStages;            // [kStages]
    uint64_t* acc_full = bars + 2 * C::kStages;     // [2]
    uint64_t* acc_empty = bars + 2 * C::kStages + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + BK - 1) / BK;
    const int tiles_n = (p.N + BM - 1) / BM;
    const int total = tiles_n * num_kb;
    const int u_begin = min((int)blockIdx.x * wk.per_cta, total), u_end = min(u_begin + wk.per_cta, total);
    // Fragments are worked on from the LAST tile of the range to the first.  The last one is the piece this
    // CTA may have to hand to its successor, the first one the piece for which it may need its predecessors:
    // handing on first and collecting last means the partial sums a CTA needs were written long before it
    // asks for them, so the owners' waits cost (almost) nothing and no CTA waits on a chain of others.
    const int tile_first = u_begin / num_kb, tile_last = u_end > u_begin ? (u_end - 1) / num_kb : tile_first - 1;
    // i-th unit in processing order
    auto unit_at = [&](int i) {
        int t = tile_last;
        for (;; --t) {
            const int lo = max(u_begin, t * num_kb), hi = min(u_end, (t + 1) * num_kb);
            if (i < hi - lo) return lo + i;
            i -= hi - lo;
        }
    };

    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
        mbar_fence_init();
        prefetch_tensormap(&tmap_w);
        prefetch_tensormap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    forge::pdl_launch_dependents();

    if (warp == 0 || warp == 6) {
        if (lane == 0) {
            // Two threads of different warps ask for the units in turn (warp 0 the even ones, warp 6 the odd ones):
            // one thread's copies of 16 KB are taken one after the other and bring an SM less than its share of
            // HBM when all SMs stream (measured on a [128256 x 4096] vocabulary, 8 rows: 188 us with one thread,
            // 161 us = 6.5 TB/s with two; no difference where the matrix is small).
            const int who = warp == 0 ? 0 : 1;
            // the weights do not depend on earlier kernels: the first ring of stages is requested before the wait
            const int n_units = u_end - u_begin;
            const int first = min(n_units, kStages);
            for (int i = who; i < first; i += 2) {
                const int u = unit_at(i);
                mbar_arrive_expect_tx(&full[i], C::kStageBytes);
                tma_load_2d(tiles + i * C::kStageBytes, &tmap_w, &full[i], (u % num_kb) * BK, (u / num_kb) * BM);
            }
            forge::pdl_wait();
            for (int i = who; i < first; i += 2)
                tma_load_2d(tiles + i * C::kStageBytes + BM * BK * 2, &tmap_x, &full[i], (unit_at(i) % num_kb) * BK, 0);
            bool ok = true;
            for (int i = first + ((first ^ who) & 1); i < n_units && ok; i += 2) {
                const int s = i % kStages, u = unit_at(i);
                if (!(ok = mbar_wait(&empty[s], ((i / kStages) - 1) & 1, abort, p.status))) break;
                mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                uint8_t* dst = tiles + s * C::kStageBytes;
                tma_load_2d(dst, &tmap_w, &full[s], (u % num_kb) * BK, (u / num_kb) * BM);
                tma_load_2d(dst + BM * BK * 2, &tmap_x, &full[s], (u % num_kb) * BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, NT);
            bool ok = true;
            int frag = 0, i = 0;
            for (int tile = tile_last; tile >= tile_first && ok; --tile, ++frag) {
                const int f_begin = max(u_begin, tile * num_kb), f_end = min(u_end, (tile + 1) * num_kb);
                const int a = frag & 1;
                if (!(ok = mbar_wait(&acc_empty[a], ((frag >> 1) & 1) ^ 1, abort, p.status))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + a * NT;
                for (int u = f_begin; u < f_end; ++u, ++i) {
                    const int s = i % kStages;
                    if (!(ok = mbar_wait(&full[s], (i / kStages) & 1, abort, p.status))) break;
                    tc_fence_after_sync();
                    const uint32_t w_addr = smem_u32(tiles + s * C::kStageBytes);
                    const uint64_t w_desc = umma_desc_k_sw128(w_addr), x_desc = umma_desc_k_sw128(w_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(d_tmem, umma_desc_advance(w_desc, k * UMMA_K * 2), umma_desc_advance(x_desc, k * UMMA_K * 2),
                                  idesc, k != 0 || u != f_begin);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[a]);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;
        const int et = threadIdx.x - 64;            // 0..127 among the epilogue threads
        forge::pdl_wait();
        bool ok = true;

        // Finishes a tile this CTA owns: adds the `part` earlier fragments' partial sums (if any) in fragment
        // order, applies the epilogue and writes C.  Returns false if the bounded wait ran out.
        auto finish_tile = [&](float (&acc)[NT], int tile, int part) -> bool {
            if (part > 0) {
                int* tile_flags = wk.flags + tile * wk.max_parts;
                if (et < part) {
                    const unsigned long long t0 = global_ns();
                    while (ld_acquire(&tile_flags[et]) == 0) {
                        if (*abort || global_ns() - t0 > kWaitLimitNs) {
                            *abort = 1;
                            if (p.status) atomicOr(p.status, 2);
                            break;
                        }
                    }
                }
                epilogue_bar();
                if (*abort) return false;
                for (int q = 0; q < part; ++q) {
                    const float* src = wk.partials + ((size_t)tile * wk.max_parts + q) * NT * BM;
#pragma unroll
                    for (int m = 0; m < NT; ++m)
                        if (m < p.M) acc[m] += __ldcg(src + m * BM + n_local);
                }
                epilogue_bar();
                if (et < part) tile_flags[et] = 0;
            }
            // a thread holds weight row n for all tokens; per token a warp writes 32 consecutive columns
            const int n = tile * BM + n_local;
            const float b = (p.bias && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll
            for (int m = 0; m < NT; ++m) {
                if (m >= p.M) break;
                const float v = acc[m] + b;
                if (p.epilogue == EPI_SWIGLU_BF16) {
                    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                    if ((lane & 1) == 0 && n + 1 < p.N)
                        reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * (p.N >> 1) + (n >> 1)] =
                            __float2bfloat16_rn(silu(v) * other);
                } else if (n < p.N) {
                    if (p.epilogue == EPI_STORE_BF16) {
                        reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
                    } else {
                        float* dst = reinterpret_cast<float*>(p.C) + (size_t)m * p.N + n;
                        *dst = p.epilogue == EPI_ACCUM_F32 ? *dst + v : v;
                    }
                }
            }
            return true;
        };

        int frag = 0;
        for (int tile = tile_last; tile >= tile_first && ok; --tile, ++frag) {
            const int f_begin = max(u_begin, tile * num_kb), f_end = min(u_end, (tile + 1) * num_kb);
            const int kb0 = f_begin - tile * num_kb, kb1 = f_end - tile * num_kb;
            const int a = frag & 1;
            if (!(ok = mbar_wait(&acc_full[a], (frag >> 1) & 1, abort, p.status))) break;
            tc_fence_after_sync();
            float acc[NT];
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * NT;
#pragma unroll
            for (int c = 0; c < NT; c += 16) {
                uint32_t r[16];
                tmem_ld_32x32b_x16(t_row + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[c + i] = __uint_as_float(r[i]);
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[a]);             // the MMA warp may reuse this accumulator now
            // which fragment of its tile is this?  The tile's first unit belongs to CTA c0.
            const int part = (int)blockIdx.x - (tile * num_kb) / wk.per_cta;
            if (kb1 < num_kb) {
                // not the owner: park the partial sum and announce it
                float* my_partial = wk.partials + ((size_t)tile * wk.max_parts + part) * NT * BM;
#pragma unroll
                for (int m = 0; m < NT; ++m)
                    if (m < p.M) my_partial[m * BM + n_local] = acc[m];
                __threadfence();
                epilogue_bar();
                if (et == 0) st_release(&wk.flags[tile * wk.max_parts + part], 1);
            } else {
                ok = finish_tile(acc, tile, kb0 > 0 ? part : 0);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

int g_num_sms = 0;

template <int BN>
int launch(const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, cudaStream_t stream) {
    using C = Cfg<BN>;
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "gemm_sm100: cannot set %d bytes of shared memory: %s",
                                                 C::kSmemBytes, cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < g_num_sms ? tiles : g_num_sms;
    // fp32 results of the wide tiles leave by TMA where a map of C can be made (16-byte aligned rows)
    GemmParams q = p;
    CUtensorMap tc = ta;
    const char* err = nullptr;
    q.tma_out = C::kOutBytes > 0 && (p.epilogue == EPI_STORE_F32 || p.epilogue == EPI_ACCUM_F32) && p.N % 4 == 0 &&
                (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && f32_tile_map(p.C, p.M, p.N, BM, &tc, &err);
    return forge::check_launch("gemm_sm100", forge::launch(gemm_sm100_kernel<BN>, dim3(grid), dim3(kThreads),
                                                             C::kSmemBytes, stream, 1, ta, tw, tc, q));
}

// How many pairs of CTAs of the two-CTA kernel run at once (one CTA per SM, clusters of 2: 74 on B200).
int resident_pairs() {
    static int cached = 0;
    if (cached == 0) {
        cudaFuncSetAttribute(gemm_sm100_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes);
        cudaFuncSetAttribute(gemm_sm100_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes);
        cudaFuncSetAttribute(gemm_sm100_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 64);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_sm100_pair_kernel<2>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = g_num_sms / 2;
        }
        cached = n;
    }
    return cached;
}

template <int PBN>
int launch_pair_width(const void* A, const void* W, const GemmParams& p, cudaStream_t stream) {
    using C = PairCfgT<PBN>;
    const int pairs = resident_pairs();                 // also sets the kernels' shared-memory limit
    const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + PBN - 1) / PBN);
    const int grid = 2 * (tiles < pairs ? tiles : pairs);
    const int num_kb = (p.K + BK - 1) / BK;
    const int group = p.K % BK != 0 ? 0 : (num_kb >= 2 ? 2 : 1);
    CUtensorMap ta, tw;
    const char* err = nullptr;
    if (group > 0) {
        if (!bf16_kblock_map(A, p.M, p.K, BM, group, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
        if (!bf16_kblock_map(W, p.N, p.K, PBN / 2, group, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
    } else {
        if (!bf16_tile_map(A, p.M, p.K, BM, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
        if (!bf16_tile_map(W, p.N, p.K, PBN / 2, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
    }
    // fp32 results leave by TMA where a map of C can be made (16-byte aligned rows)
    GemmParams q = p;
    CUtensorMap tc = ta;
    q.tma_out = (p.epilogue == EPI_STORE_F32 || p.epilogue == EPI_ACCUM_F32) && p.N % 4 == 0 &&
                (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && f32_tile_map(p.C, p.M, p.N, BM, &tc, &err);
    cudaError_t e;
    if constexpr (PBN == kPairBN) {
        if (group == 2) e = forge::launch(gemm_sm100_pair_kernel<2>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, 2, ta, tw, tc, q);
        else if (group == 1) e = forge::launch(gemm_sm100_pair_kernel<1>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, 2, ta, tw, tc, q);
        else e = forge::launch(gemm_sm100_pair_kernel<0>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, 2, ta, tw, tc, q);
    } else {
        // the narrower tiles exist for K in whole groups of two k-blocks only (the caller checks)
        if (group != 2) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: tiles of %d columns need K %% 64 == 0 and K >= 128, got %d", PBN, p.K);
        static forge::PerDeviceFlag configured_on;
        bool& configured = configured_on.current();
        if (!configured) {
            cudaError_t a = cudaFuncSetAttribute(gemm_sm100_pair_kernel<2, PBN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
            if (a != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "gemm_sm100: cannot set %d bytes of shared memory: %s",
                                                     C::kSmemBytes, cudaGetErrorString(a));
            configured = true;
        }
        e = forge::launch(gemm_sm100_pair_kernel<2, PBN>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, 2, ta, tw, tc, q);
    }
    return forge::check_launch("gemm_sm100 (two CTAs per tile)", e);
}

int launch_pair(const void* A, const void* W, const GemmParams& p, cudaStream_t stream) {
    return launch_pair_width<kPairBN>(A, W, p, stream);
}

// How many CTAs of the split-K kernel run at once in clusters of `ks` (one CTA per SM; both forms of the kernel take
// the same shared memory).
constexpr int kSplitKSmem = SplitKCfg<2>::kSmemBytes;
static_assert(SplitKCfg<1>::kSmemBytes == kSplitKSmem, "one occupancy figure serves both forms");
int splitk_resident_ctas(int ks) {
    static int cached[5] = {0};
    if (ks != 2 && ks != 4) return 0;
    if (cached[ks] == 0) {
        cudaFuncSetAttribute(gemm_sm100_splitk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitKSmem);
        cudaFuncSetAttribute(gemm_sm100_splitk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitKSmem);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ks * 32);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSplitKSmem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = ks;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_sm100_splitk_kernel<2>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = (g_num_sms - (ks > 2 ? g_num_sms / 8 : 0)) / ks;      // a guess on the safe side
        }
        cached[ks] = n * ks;
    }
    return cached[ks];
}

int launch_splitk(const void* A, const void* W, const GemmParams& p, int ksplit, cudaStream_t stream) {
    splitk_resident_ctas(2);                            // also sets the kernels' shared-memory limit
    CUtensorMap ta, tw;
    const char* err = nullptr;
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + kSplitBN - 1) / kSplitBN);
    if (p.K % BK == 0) {                                // whole k-blocks: two of them per instruction
        if (!bf16_kblock_map(A, p.M, p.K, BM, 2, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
        if (!bf16_kblock_map(W, p.N, p.K, kSplitBN, 2, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
        return forge::check_launch("gemm_sm100 (K cut across a cluster)",
                                   forge::launch(gemm_sm100_splitk_kernel<2>, dim3(tiles * ksplit), dim3(kThreads),
                                                 kSplitKSmem, stream, ksplit, ta, tw, p, ksplit));
    }
    if (!bf16_tile_map(A, p.M, p.K, BM, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
    if (!bf16_tile_map(W, p.N, p.K, kSplitBN, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
    return forge::check_launch("gemm_sm100 (K cut across a cluster)",
                               forge::launch(gemm_sm100_splitk_kernel<1>, dim3(tiles * ksplit), dim3(kThreads),
                                             kSplitKSmem, stream, ksplit, ta, tw, p, ksplit));
}

// k-blocks per TMA instruction for a CTA that has kb_per of them; 0 = K is no multiple of 64 (2D maps).  The group
// that loads the fewest k-blocks beyond the CTA's own (its last group is whole all the same), the larger one of equals;
// at least two per instruction where there are two (one 16 KB box per instruction is bound by the instruction rate).
int few_rows_group(int K, int kb_per, int max_group) {
    if (K % BK != 0) return 0;
    if (kb_per <= max_group) return kb_per < 1 ? 1 : kb_per;
    int best = max_group, best_waste = (kb_per + max_group - 1) / max_group * max_group - kb_per;
    for (int g = max_group - 1; g >= 2; --g) {
        const int waste = (kb_per + g - 1) / g * g - kb_per;
        if (waste < best_waste) { best = g; best_waste = waste; }
    }
    return best;
}

template <int NT>
int launch_skinny(const void* W, const void* A, const GemmParams& p, int ksplit, int tile_rows, cudaStream_t stream) {
    using C = SkinnyCfg<NT>;
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_skinny_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "gemm_sm100: cannot set %d bytes of shared memory: %s",
                                                 kSmemLimit, cudaGetErrorString(e));
        configured = true;
    }
    const int tiles_n = (p.N + tile_rows - 1) / tile_rows;
    const int num_kb = (p.K + BK - 1) / BK, kb_per = (num_kb + ksplit - 1) / ksplit;
    const int group = few_rows_group(p.K, kb_per, C::kMaxGroup), g = group > 0 ? group : 1;
    const int groups_per = (kb_per + g - 1) / g;
    const int stages = groups_per < C::max_stages(g, tile_rows) ? groups_per : C::max_stages(g, tile_rows);
    CUtensorMap tw, tx;
    const char* err = nullptr;
    if (group > 0) {
        if (!bf16_kblock_map(W, p.N, p.K, tile_rows, group, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
        if (!bf16_kblock_map(A, p.M, p.K, NT, group, &tx, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
    } else {
        if (!bf16_tile_map(W, p.N, p.K, tile_rows, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
        if (!bf16_tile_map(A, p.M, p.K, NT, &tx, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
    }
    return forge::check_launch("gemm_sm100 (few rows)",
                               forge::launch(gemm_sm100_skinny_kernel<NT>, dim3(tiles_n * ksplit), dim3(kSkinnyThreads),
                                             C::smem_bytes(stages, g, tile_rows), stream, ksplit, tw, tx, p, ksplit, stages, group, tile_rows));
}

// workspace for the stream-K partial sums and flags, per device, handed over once by the caller
struct Workspace { void* ptr = nullptr; long long bytes = 0; };
Workspace g_workspace[64];
constexpr long long kFlagBytes = 256 * 1024;      // flags first (zeroed by the caller), partials after

// Whether the current device's workspace holds the evenly dealt kernel's partial sums for this product.
bool streamk_fits(int nt, int N, int K) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !g_workspace[dev].ptr) return false;
    const int tiles_n = (N + BM - 1) / BM, num_kb = (K + BK - 1) / BK;
    const int total = tiles_n * num_kb;
    int grid = total < g_num_sms ? total : g_num_sms;
    const int per_cta = (total + grid - 1) / grid;
    const int max_parts = (num_kb + per_cta - 1) / per_cta + 1;
    return g_workspace[dev].bytes >= kFlagBytes + (long long)tiles_n * max_parts * nt * BM * 4 &&
           (long long)tiles_n * max_parts * 4 <= kFlagBytes;
}

template <int NT>
int launch_streamk(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
    using C = StreamKCfg<NT>;
    static forge::PerDeviceFlag configured_on;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_streamk_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::smem_bytes(C::kStages));
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "gemm_sm100: cannot set %d bytes of shared memory: %s",
                                                 C::smem_bytes(C::kStages), cudaGetErrorString(e));
        configured = true;
    }
    int dev = 0;
    cudaGetDevice(&dev);
    const int tiles_n = (p.N + BM - 1) / BM, num_kb = (p.K + BK - 1) / BK;
    const int total = tiles_n * num_kb;
    int grid = total < g_num_sms ? total : g_num_sms;
    const int per_cta = (total + grid - 1) / grid;
    grid = (total + per_cta - 1) / per_cta;
    const int max_parts = (num_kb + per_cta - 1) / per_cta + 1;
    const long long need = kFlagBytes + (long long)tiles_n * max_parts * NT * BM * 4;
    if (dev < 0 || dev >= 64 || !g_workspace[dev].ptr || g_workspace[dev].bytes < need ||
        (long long)tiles_n * max_parts * 4 > kFlagBytes)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: the stream-K workspace of device %d holds %lld bytes, %lld needed "
                           "(call forge_gemm_sm100_set_workspace)", dev, dev >= 0 && dev < 64 ? g_workspace[dev].bytes : 0LL, need);
    StreamKWork wk{reinterpret_cast<float*>(static_cast<char*>(g_workspace[dev].ptr) + kFlagBytes),
                   static_cast<int*>(g_workspace[dev].ptr), per_cta, max_parts};
    const int stages = per_cta < C::kStages ? per_cta : C::kStages;
    return forge::check_launch("gemm_sm100 (few rows, stream-K)",
                               forge::launch(gemm_sm100_streamk_kernel<NT>, dim3(grid), dim3(kStreamKThreads),
                                             C::smem_bytes(stages), stream, 1, tw, tx, p, wk, stages));
}

// How many CTAs of the few-rows kernel run at once when launched in clusters of `ks` with all the shared
// memory an SM has (one CTA per SM): fewer than there are SMs, because a cluster lives inside one GPC
// (B200: 148, 148, 132 and 120 for clusters of 1, 2, 4 and 8).
int max_resident_ctas(int ks) {
    static int cached[9] = {0};
    if (ks < 1 || ks > 8) return 0;
    if (cached[ks] == 0) {
        cudaFuncSetAttribute(gemm_sm100_skinny_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ks * 64);
        cfg.blockDim = dim3(kSkinnyThreads);
        cfg.dynamicSmemBytes = kSmemLimit;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = ks;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_sm100_skinny_kernel<16>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = (g_num_sms - g_num_sms / 8 * (ks > 2 ? (ks > 4 ? 2 : 1) : 0)) / ks;      // a guess on the safe side
        }
        cached[ks] = n * ks;
    }
    return cached[ks];
}

}  // namespace

// Hands the library a zero-initialised device buffer (>= 256 KiB of flags + room for partial sums) that the
// stream-K kernel of the current device may use from now on.  The buffer must outlive all later calls.
extern "C" int forge_gemm_sm100_set_workspace(void* ptr, long long bytes) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return forge::fail(FORGE_ERR_ARG, "set_workspace: no current device");
    if (bytes < kFlagBytes + 1024 * 1024) return forge::fail(FORGE_ERR_ARG, "set_workspace: %lld bytes is too small", bytes);
    g_workspace[dev].ptr = ptr;
    g_workspace[dev].bytes = bytes;
    return FORGE_OK;
}

// A [M,K] bf16, W [N,K] bf16 (both row-major, K % 8 == 0, 16-byte aligned), bias fp32 [N] or null.
// epilogue: 0 C fp32 = ..., 1 C fp32 += ..., 2 C bf16 = ..., 3 C bf16 [M,N/2] = swiglu (N even).
// tile_n: 0 = choose; 16, 32, 64, 128, 160, 192, 224, 256 = token-major tiles of that width; 512 (M > 128) = a pair
// of CTAs on a [256 x 256] tile (cta_group::2); 1002, 1004 (M > 128, fp32 results) = tiles of 128 x 128 with K cut across
// a cluster of 2 or 4 CTAs; -1 .. -8 (M <= 128 only) =
// the few-rows kernel with K cut across a cluster of that many CTAs; -100 (M <= 64 only) = the few-rows kernel
// that deals units of work out evenly to persistent CTAs (the default once a workspace has been set).  status: device int, bit 1 raised if a wait ran out.
extern "C" int forge_gemm_sm100(const void* A, const void* W, const float* bias, void* C, int* status, int M, int N,
                                int K, int epilogue, int tile_n, void* reserved, cudaStream_t stream) {
    (void)reserved;
    if (M < 0 || N <= 0 || K <= 0) return forge::fail(FORGE_ERR_ARG, "gemm_sm100: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return FORGE_OK;
    if (K % 8 != 0) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: K=%d is not a multiple of 8 (TMA row stride)", K);
    if (epilogue < 0 || epilogue > 3) return forge::fail(FORGE_ERR_ARG, "gemm_sm100: unknown epilogue %d", epilogue);
    if (epilogue == EPI_SWIGLU_BF16 && (N & 1)) return forge::fail(FORGE_ERR_ARG, "gemm_sm100: swiglu epilogue needs even N, got %d", N);
    if (g_num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    const char* err = nullptr;
    if (M <= 128 && tile_n <= 0) {
        // few rows: weights are the MMA's M operand, K is cut across a cluster (tile_n < 0: -tile_n CTAs).  Up to
        // 128 tokens: with one row tile the token-major kernel would reload all tokens for every narrow column
        // tile (measured at 128 rows, [2048 x 5632]: 25.8 us against this kernel's 14).
        const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        const int tiles_n = (N + BM - 1) / BM, num_kb = (K + BK - 1) / BK;
        int dev = 0;
        cudaGetDevice(&dev);
        const bool have_ws = dev >= 0 && dev < 64 && g_workspace[dev].ptr != nullptr;
        // More row tiles than SMs (a vocabulary): deal the (row tile, k-block) units out evenly over the SMs.
        // Otherwise one wave of clusters, see below; the partial sums of stream-K cross global memory, which
        // costs more than an uneven last wave unless there are many tiles (measured at 88 tiles: 13.2 against
        // 11.0 us).
        // (up to 32 rows always where a workspace was set; 33 to 64 rows where the partial sums of 64 rows fit it:
        // [28672 x 4096] at 64 rows 62 -> 58 us)
        if ((tile_n == 0 && have_ws && nt <= 64 && tiles_n > g_num_sms && (nt <= 32 || streamk_fits(nt, N, K))) || tile_n == -100) {
            CUtensorMap tw, tx;
            if (!bf16_tile_map(W, N, K, BM, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
            if (!bf16_tile_map(A, M, K, nt, &tx, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
            GemmParams p{C, bias, M, N, K, epilogue, status};
            switch (nt) {
                case 16: return launch_streamk<16>(tw, tx, p, stream);
                case 32: return launch_streamk<32>(tw, tx, p, stream);
                case 64: return launch_streamk<64>(tw, tx, p, stream);
                default: return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: the evenly dealt kernel takes at most 64 rows, got %d", M);
            }
        }
        // The CTAs' shape: weight rows per tile (128, or fewer so that more SMs stream) and how many CTAs of a
        // cluster cut K between them.  tile_n = -(100 * rows + cluster) names both (tests and measurements),
        // -1 .. -8 the cluster with tiles of 128 rows.
        int ksplit = 1, tile_rows = BM;
        if (tile_n < 0) {
            ksplit = (-tile_n) % 100;
            if (-tile_n >= 100) tile_rows = (-tile_n) / 100;
            if (ksplit < 1 || ksplit > 8)
                return forge::fail(FORGE_ERR_ARG, "gemm_sm100: cluster size must be 1 to 8, got %d", ksplit);
            // The MMA reads 128 rows from a tile's base whatever the tile holds: (128 - rows) * 128 bytes beyond the
            // last k-block of the last stage, which must stay inside the CTA's shared memory.  Behind the weight
            // stages lie the tokens' stages and the partial sums (at least 8 KB): 64 rows or more are safe.
            if (tile_rows < 64 || tile_rows > BM || tile_rows % 16 != 0)
                return forge::fail(FORGE_ERR_ARG, "gemm_sm100: a tile's weight rows must be 64, 80, 96, 112 or 128, got %d", tile_rows);
        } else {
            // The widest cluster whose CTAs all run at once (a second wave doubles the time) and still have a
            // group of four k-blocks each.
            // (clusters of 3, 5, 6 and 7 work too but measured no faster than the next power of two below them:
            // [2560 x 2048] 4.5 us with 4 CTAs, 5.2 with 6; [2048 x 5632] 7.7 and 7.4; 7 fit too few at once)
            for (int ks = 2; ks <= 8; ks *= 2)
                if (tiles_n * ks <= max_resident_ctas(ks) && num_kb / ks >= 4) ksplit = ks;
            // More CTAs through tiles of fewer than 128 weight rows (the MMA rows that nobody reads are free here).
            // Up to 32 tokens this LOSES inside a decode step although each product alone gains: a product that
            // leaves SMs idle leaves them to the next product's CTAs, which start early and request their first
            // weight stages while this one runs; measured at 8 tokens, all four projections on 128 to 141 SMs:
            // 0.83 -> 0.95 ms per step.  At 33 to 64 tokens a product lasts long enough for the gain to stay:
            // gate/up 18.2 -> 15.3 us, 47.8 -> 49.1 thousand tokens a second at batch 64.
            if (nt == 64) {
                long best = (long)tiles_n * ksplit;
                for (int rows = BM - 16; rows >= 64; rows -= 16) {
                    const int tiles = (N + rows - 1) / rows;
                    for (int ks = 1; ks <= 8; ks *= 2) {
                        if (ks > 1 && num_kb / ks < 4) continue;
                        const long ctas = (long)tiles * ks;
                        if (ctas > max_resident_ctas(ks) || ctas <= best) continue;
                        best = ctas; ksplit = ks; tile_rows = rows;
                    }
                }
            }
        }
        // 65..128 tokens with an unsplit tile per CTA (many row tiles, e.g. gate/up): the token-major kernel with
        // 128-wide tiles is the faster one there (22 against 28-33 us at [11264 x 2048])
        const bool token_major_instead = nt == 128 && tile_n == 0 && ksplit == 1;
        GemmParams p{C, bias, M, N, K, epilogue, status};
        if (!token_major_instead) switch (nt) {
            case 16: return launch_skinny<16>(W, A, p, ksplit, tile_rows, stream);
            case 32: return launch_skinny<32>(W, A, p, ksplit, tile_rows, stream);
            case 64: return launch_skinny<64>(W, A, p, ksplit, tile_rows, stream);
            default: return launch_skinny<128>(W, A, p, ksplit, tile_rows, stream);
        }
    }
    // Some hundred rows onto a narrow matrix with an fp32 result (o and down projections of a short prompt): tiles of
    // 128 x 128 with K cut across 2 or 4 CTAs while that fills no more than the SMs that run at once.  tile_n 1002 and
    // 1004 name it (tests and measurements).
    if ((M > BM || tile_n > 1000) && (epilogue == EPI_STORE_F32 || epilogue == EPI_ACCUM_F32) && (tile_n == 0 || tile_n == 1002 || tile_n == 1004)) {
        const long tiles = (long)((M + BM - 1) / BM) * ((N + kSplitBN - 1) / kSplitBN);
        const int num_kb = (K + BK - 1) / BK;
        int ks = 0;
        if (tile_n > 1000) {
            ks = tile_n - 1000;
        } else {
            for (int c : {2, 4})
                if (tiles * c <= splitk_resident_ctas(c) && num_kb / c >= 8) ks = c;
        }
        if (ks > 0) {
            GemmParams p{C, bias, M, N, K, epilogue, status};
            return launch_splitk(A, W, p, ks, stream);
        }
    }
    int bn = tile_n;
    if (bn == 0) {
        // few rows (decode): narrow tiles so that many SMs stream W; many rows: the widest tile whose tile
        // count wastes the least of the last wave
        if (M <= BM) {
            // 65..128 rows: one row tile, so the column tiles alone must spread over the SMs; the narrowest width
            // that leaves at most ~0.6 tiles per SM (measured at 96 and 128 rows: 32 for N = 2048 and 2560, 128 for
            // N = 11264 beat 16 and 64 by 10-40 %)
            bn = 256;
            for (int cand : {16, 32, 64, 128}) {
                if ((N + cand - 1) / cand <= (g_num_sms * 6) / 10) { bn = cand; break; }
            }
        } else {
            // A k-step (16 of K) of a [128 x BN] tile moves 2 * (4 KB + BN * 32 B) through shared memory (TMA writes
            // it, the tensor core reads it) at 128 B per clock against BN / 2 clocks of arithmetic: 64 + BN / 2 clocks,
            // so wide tiles are cheaper per column.  Two CTAs on a [256 x 256] tile stage half the W bytes per SM and
            // run at the arithmetic's 128 clocks in their main loop; set-up, cluster hand-shakes and the two-SM
            // scheduling make that about 150 in a whole kernel (fitted to measurements at 512, 2048 and 4096 rows).
            // The epilogue of a CTA's last tile is not hidden behind a next tile: about 36 clocks per column.
            const long tm = (M + BM - 1) / BM, ksteps = (K + UMMA_K - 1) / UMMA_K;
            long best = -1;
            for (int cand : {256, 224, 192, 160, 128}) {
                const long tiles = tm * ((N + cand - 1) / cand);
                const long cost = ((tiles + g_num_sms - 1) / g_num_sms) * ksteps * (64 + cand / 2) + 36L * cand;
                if (best < 0 || cost < best) { best = cost; bn = cand; }
            }
            const long pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + kPairBN - 1) / kPairBN), pairs = resident_pairs();
            if (((pair_tiles + pairs - 1) / pairs) * ksteps * 150 + 36L * kPairBN < best) bn = 512;
        }
    }
    if (bn == 512 || bn == 1192 || bn == 1128) {
        if (M <= BM) return forge::fail(FORGE_ERR_ARG, "gemm_sm100: the two-CTA tile is for more than %d rows, got %d", BM, M);
        GemmParams p{C, bias, M, N, K, epilogue, status};
        if (bn == 512) return launch_pair(A, W, p, stream);
        if (K % BK != 0 || K < 2 * BK)
            return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: two-CTA tiles of %d columns need K %% 64 == 0 and K >= 128, got %d", bn - 1000, K);
        return bn == 1192 ? launch_pair_width<192>(A, W, p, stream) : launch_pair_width<128>(A, W, p, stream);
    }
    CUtensorMap ta, tw;
    if (!bf16_tile_map(A, M, K, BM, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: A: %s", err);
    if (!bf16_tile_map(W, N, K, bn, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100: W: %s", err);
    GemmParams p{C, bias, M, N, K, epilogue, status};
    switch (bn) {
        case 256: return launch<256>(ta, tw, p, stream);
        case 224: return launch<224>(ta, tw, p, stream);
        case 192: return launch<192>(ta, tw, p, stream);
        case 160: return launch<160>(ta, tw, p, stream);
        case 128: return launch<128>(ta, tw, p, stream);
        case 64: return launch<64>(ta, tw, p, stream);
        case 32: return launch<32>(ta, tw, p, stream);
        case 16: return launch<16>(ta, tw, p, stream);
        default: return forge::fail(FORGE_ERR_ARG, "gemm_sm100: tile_n must be 16, 32, 64, 128, 160, 192, 224, 256, or 512 / 1192 / 1128 (two CTAs on 256 x 256 / 192 / 128), got %d", bn);
    }
}

// The fused projection of a prompt step: x [M, K] . [Wq; Wk; Wv]^T (+ bias), whose epilogue rotates q and k by the rows'
// angles (rope_table [head_dim/2, M, 2] of (cos, sin); null: no rotation), writes q [M, NH*head_dim] in bf16 and puts k
// and v into the paged cache at slot_mapping (null or negative: not written).  Head sizes 64 and 128; for more than 128
// rows (fewer go through forge_gemm_sm100 and the separate rotary kernel).
extern "C" int forge_gemm_sm100_qkv_rope(const void* A, const void* W, const float* bias, void* q_out, void* kv_cache,
                                         const float* rope_table, const int32_t* slot_mapping, int* status, int M, int K,
                                         int NH, int NKV, int head_dim, int page_size, int force_tile, cudaStream_t stream) {
    if (head_dim != 64 && head_dim != 128) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100_qkv_rope: head_dim %d (64 or 128)", head_dim);
    if (M <= BM) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100_qkv_rope: for more than %d rows, got %d", BM, M);
    if (K <= 0 || K % 8 != 0 || NH <= 0 || NKV <= 0 || page_size <= 0)
        return forge::fail(FORGE_ERR_ARG, "gemm_sm100_qkv_rope: bad sizes K=%d NH=%d NKV=%d page=%d", K, NH, NKV, page_size);
    if (g_num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    const int N = (NH + 2 * NKV) * head_dim;
    // Tiles hold whole heads.  One CTA per tile of 128 or 256 columns, or a pair of CTAs on [256 x 128, 192 or 256]:
    // whichever needs the fewest clocks for its rounds of tiles.  Clocks per k-step of a tile, measured over prompts of
    // 512 to 4,096 rows: a single CTA is bound by shared-memory traffic at about 64 + width / 2 (133 and 188), a pair
    // takes 123, 128 and 174 for 128, 192 and 256 columns (about 0.68 per column with a floor of 123).
    // `force_tile` (tests and measurements): 0 = choose, 128 / 256 = one CTA, 1128 / 1192 / 1256 = a pair.
    const long tm = (M + BM - 1) / BM, ksteps = (K + UMMA_K - 1) / UMMA_K;
    const long tm2 = (M + 2 * BM - 1) / (2 * BM), pairs = resident_pairs();
    const bool pair_ok = K % BK == 0 && K >= 2 * BK;
    int choice = 128;
    long best = -1;
    for (int cand : {256, 128, 1256, 1192, 1128}) {
        const bool pair = cand > 1000;
        const int width = pair ? cand - 1000 : cand;
        if (pair && (!pair_ok || width % head_dim != 0)) continue;
        if (force_tile != 0 && cand != force_tile) continue;
        const long tiles = (pair ? tm2 : tm) * ((N + width - 1) / width);
        const long waves = pair ? (tiles + pairs - 1) / pairs : (tiles + g_num_sms - 1) / g_num_sms;
        const long per_kstep = pair ? (17L * width / 25 > 123 ? 17L * width / 25 : 123) : 64 + width / 2;
        const long cost = waves * ksteps * per_kstep + 36L * width;
        if (best < 0 || cost < best) { best = cost; choice = cand; }
    }
    if (best < 0) return forge::fail(FORGE_ERR_ARG, "gemm_sm100_qkv_rope: tile %d is not available for these sizes", force_tile);
    GemmParams p{q_out, bias, M, N, K, EPI_QKV_ROPE, status, 0, rope_table, slot_mapping, static_cast<__nv_bfloat16*>(kv_cache),
                 NH, NKV, head_dim, page_size};
    if (choice == 1256) return launch_pair_width<256>(A, W, p, stream);
    if (choice == 1192) return launch_pair_width<192>(A, W, p, stream);
    if (choice == 1128) return launch_pair_width<128>(A, W, p, stream);
    const char* err = nullptr;
    CUtensorMap ta, tw;
    if (!bf16_tile_map(A, M, K, BM, &ta, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100_qkv_rope: A: %s", err);
    if (!bf16_tile_map(W, N, K, choice, &tw, &err)) return forge::fail(FORGE_ERR_UNSUPPORTED, "gemm_sm100_qkv_rope: W: %s", err);
    return choice == 256 ? launch<256>(ta, tw, p, stream) : launch<128>(ta, tw, p, stream);
}

// (checks build) the bounds that this library's projection tests slots against
FORGE_DEFINE_CHECKS_ENTRY(gemm_sm100)

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
