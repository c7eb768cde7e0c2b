// All layers of a decode step (one new token for each of up to 16 requests) in ONE persistent kernel.
//
// A decode step of a dense decoder is a stream of weights through the SMs: every matrix is read once and
// multiplied with a handful of token rows.  Launched as one kernel per operation (norm, qkv, attention, o,
// norm, gate/up, down: seven a layer), every link of that chain pays a hand-over of about two microseconds
// during which no weight moves, which at small batches is most of the time.  Here one CTA per SM stays
// resident for all layers:
//
//  * warp 0 is the weight streamer.  The order in which this CTA needs weight tiles is known before the
//    step starts, so one thread walks that list for the whole step and keeps a ring of 32 KB stages full by
//    TMA (two [128 x 64] k-blocks of a matrix per instruction).  It never waits for data, only for a free
//    stage: weights for the next operation, and the next layer, arrive while the current one is computed.
//  * warp 1 issues the tcgen05 MMAs: the weight tile is the M operand (128 output features), the tokens are
//    the N side (16), the accumulator lives in tensor memory.
//  * warps 2-9 (256 threads) prepare the token operand and finish the products.  Activations live in global
//    memory in fp32 (they are a few hundred KB and stay in L2); the workers read the slice they need, apply
//    what stands between two products (norm weight, SwiGLU), round to bfloat16 and write the 128-byte-swizzled
//    tile the MMA reads; the loads of the next units are in flight while the current ones are converted.  After
//    a tile's last MMA they add its accumulator into the result in global memory with `red.global.add.f32` (the
//    L2 adds; nothing is read back).  They also run the attention.
//
// A matrix is dealt to the CTAs in units of (128 output features) x (128 of K), the same number of units to
// every CTA whatever the matrix's shape, so the partial sums of an output element come from several CTAs and
// meet in L2.  What follows a product is applied by the consumer of its result:
//     qkv_acc  += (x * w_norm1) . Wqkv^T           ssq1 += sum x^2
//     attention reads qkv_acc / rms + bias, rotates, writes the cache, attends      -> parts of the result
//     x        += merge(parts) . Wo^T
//     gu_acc   += (x * w_norm2) . Wgu^T             ssq2 += sum x^2
//     x        += (silu(g / rms) * (u / rms)) . Wd^T
// (RMSNorm is linear up to the division by the row's rms, which commutes with the product.)
// Between these five phases all CTAs meet at a barrier in global memory (an arrival counter that every CTA
// increments and polls); the weight streamer does not take part, so the barrier costs latency but no
// bandwidth.
//
// Attention: the keys of a (request, kv head) are dealt to up to 4 CTAs (tiles of 32 keys round the CTAs, then
// round a CTA's 4 warps), so that with few requests most SMs have a share and a warp has one or two tiles.  The
// tiles of earlier positions do not depend on this layer's projections: they are requested before the barrier
// that ends the qkv product, so their trip from HBM is over when q arrives.  Each CTA leaves its un-normalised
// partial result in global memory; the o-projection merges the parts (in part order) while it builds its token
// operand.  Rotary angles come from a table that the kernel fills once at its start.
//
// Every wait (mbarrier, grid barrier) has a time limit; on expiry the CTA raises a status bit and a flag that
// makes all other CTAs leave too.  The sums over K are made in an order that depends on timing (atomic adds),
// so results differ from run to run in the last bits of fp32; the bfloat16 path makes no promise beyond rounding.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "mma_sync.cuh"
#include "sm100.cuh"

#ifndef FORGE_ATT_HD
#define FORGE_ATT_HD 64
#endif

namespace {

using namespace sm100;
using namespace mma_sync;

constexpr int HD = FORGE_ATT_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head size: a multiple of 16 up to 128");
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int kPair = 2;                               // k-blocks per unit and per TMA instruction
constexpr int kStageW = kPair * BM * BK * 2;           // 32 KB of weights per stage
constexpr int kStages = 4;
constexpr int kThreads = 320, kWorkers = 256;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxTokens = 16;                         // tokens of a step: the N side of every MMA
constexpr int kSsqStride = 64;                          // ssq: [2][kSsqStride]
constexpr int kMaxSplit = 4;                            // CTAs that share the keys of one (request, kv head)

// attention inside the kernel: 4 warps (2 for head sizes above 64) take tiles of 32 keys in turn
constexpr int DKV = 32;
constexpr int LD = HD + 8;                              // padded row length in shared memory (bf16 elements)
constexpr int CPR = HD / 8;                             // 16-byte chunks per row
constexpr int kAttWarps = HD <= 64 ? 4 : 2;
constexpr int kAttBytes = (16 + kAttWarps * 4 * DKV) * LD * 2;
static_assert((size_t)kAttWarps * 16 * (HD + 2) * 4 <= (size_t)kAttWarps * 4 * DKV * LD * 2, "merge area fits the tile buffers");

enum { OP_NORMW = 0, OP_MERGE = 1, OP_SWIGLU = 2 };
constexpr int kAccs = 4;                                // accumulators in tensor memory: tiles whose sums wait for their epilogue

struct alignas(64) LayerDesc {
    CUtensorMap w_qkv, w_o, w_gu, w_down;              // k-block views {64, rows, K/64}, boxes {64, 128, 2}
    const float* norm1;                                // [H]
    const float* norm2;                                // [H]
    const float* qkv_bias;                             // [(NH + 2 NKV) * HD] or null
    __nv_bfloat16* kv;                                 // this layer's cache [pages, 2, NKV, page_size, HD]
};

struct Params {
    const LayerDesc* layers;
    int num_layers;
    float* resid;                 // [B, H] fp32, in and out: the residual stream
    float* qkv_acc;               // [B, QKV] fp32 scratch
    float* gu_acc;                // [B, 2I] fp32 scratch (gate and up interleaved)
    float* ssq;                   // [2][64] sums of squares of the rows before each norm (first 16 of each used)
    float2* rope_tab;             // [B, HD/2] (cos, sin) of the step's positions
    float* part_o;                // [B*NKV, kMaxSplit, 16, HD] un-normalised attention outputs of the parts of the keys
    float* part_ml;               // [B*NKV, kMaxSplit, 16, 2] their (maximum, sum of weights)
    const int32_t* block_table;   // [B, max_pages]
    const int32_t* positions;     // [B]
    const int32_t* slot_mapping;  // [B]
    unsigned int* barrier;        // [0] arrivals, [1] abort flag, [2] CTAs that are through; all zero before the first launch
    int* status;
    int B, H, I, NH, NKV, QKV, page_size, max_pages, window, rotary;
    float theta, scale_log2, eps;
    unsigned long long wait_limit_ns;
    int prefetch_units;            // how many units ahead of its ring loads the weight streamer asks L2 for
    unsigned long long* timeline;  // null, or [CTAs][barriers][2]: when each CTA reached and left each barrier (ns)
};

struct PhaseInfo {
    const CUtensorMap* map;
    int n_out, K, kp, tiles, op;
    float* out;
    int ldo;
    const float* normw;
    float* ssq;
};

__device__ __forceinline__ PhaseInfo phase_info(const Params& p, const LayerDesc* L, int ph) {
    PhaseInfo f;
    f.normw = nullptr;
    f.ssq = nullptr;
    if (ph == 0) {
        f.map = &L->w_qkv; f.n_out = p.QKV; f.K = p.H; f.op = OP_NORMW; f.out = p.qkv_acc; f.ldo = p.QKV;
        f.normw = L->norm1; f.ssq = p.ssq;
    } else if (ph == 1) {
        f.map = &L->w_o; f.n_out = p.H; f.K = p.NH * HD; f.op = OP_MERGE; f.out = p.resid; f.ldo = p.H;
    } else if (ph == 2) {
        f.map = &L->w_gu; f.n_out = 2 * p.I; f.K = p.H; f.op = OP_NORMW; f.out = p.gu_acc; f.ldo = 2 * p.I;
        f.normw = L->norm2; f.ssq = p.ssq + kSsqStride;
    } else {
        f.map = &L->w_down; f.n_out = p.H; f.K = p.I; f.op = OP_SWIGLU; f.out = p.resid; f.ldo = p.H;
    }
    f.kp = (f.K + kPair * BK - 1) / (kPair * BK);
    f.tiles = (f.n_out + BM - 1) / BM;
    return f;
}

// units [u0, u1) of this CTA: the same number (give or take one) for every CTA
__device__ __forceinline__ void unit_range(const PhaseInfo& f, int& u0, int& u1) {
    const long long U = (long long)f.tiles * f.kp;
    u0 = (int)(U * blockIdx.x / gridDim.x);
    u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
}

// Walks the units of this CTA in the order of the step: layers, in each the four products, in each the CTA's share.
struct UnitWalk {
    int layer, ph, u, u1;
    PhaseInfo f;
    bool done;
};
__device__ __forceinline__ void walk_settle(const Params& p, UnitWalk& w) {
    // moves on to the next product (or layer) until one has a unit for this CTA
    while (!w.done && w.u >= w.u1) {
        if (++w.ph == 4) { w.ph = 0; ++w.layer; }
        if (w.layer >= p.num_layers) { w.done = true; break; }
        w.f = phase_info(p, p.layers + w.layer, w.ph);
        unit_range(w.f, w.u, w.u1);
    }
}
__device__ __forceinline__ UnitWalk walk_begin(const Params& p) {
    UnitWalk w;
    w.layer = 0; w.ph = -1; w.u = 0; w.u1 = 0; w.done = p.num_layers <= 0;
    walk_settle(p, w);
    return w;
}
__device__ __forceinline__ void walk_next(const Params& p, UnitWalk& w) {
    ++w.u;
    walk_settle(p, w);
}
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs' workers meet: arrival number `target` (a running total over the barriers of the step) must be
// reached.  Called by the 256 workers of every CTA.  Returns false if the wait ran out or another CTA gave up.
__device__ __forceinline__ bool grid_barrier(const Params& p, unsigned int target, volatile int* abort, int tid) {
    workers_sync();
    if (tid == 0 && !*abort) {
        unsigned long long* stamp = nullptr;
        if (p.timeline) {
            const unsigned int nb = target / gridDim.x - 1, per_cta = 1 + 5 * p.num_layers;
            stamp = p.timeline + ((size_t)blockIdx.x * per_cta + nb) * 8;
            stamp[0] = global_ns();
        }
        __threadfence();
        const unsigned int mine = atomicAdd(p.barrier, 1u) + 1u;     // the CTA that brings the count to `target` need not poll
        const unsigned long long t0 = global_ns();
        while (mine < target && ld_acquire_u32(p.barrier) < target) {
            if (ld_acquire_u32(p.barrier + 1) != 0u) { *abort = 1; break; }
            if (global_ns() - t0 > p.wait_limit_ns) {
                *abort = 1;
                atomicExch(p.barrier + 1, 1u);
                if (p.status) atomicOr(p.status, 2 | (1 << 20));
                break;
            }
        }
        __threadfence();
        if (stamp) stamp[1] = global_ns();
    }
    workers_sync();
    return *abort == 0;
}

// g / (1 + e^-g) with the special-function unit's exponential and division (relative error of a few fp32 ulp; the
// result is rounded to bfloat16 right after)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 o;
    o.x = pack_bf16(v[0], v[1]);
    o.y = pack_bf16(v[2], v[3]);
    o.z = pack_bf16(v[4], v[5]);
    o.w = pack_bf16(v[6], v[7]);
    return o;
}

// The token operands of up to UG consecutive units (k-pairs pair0, pair0 + 1, ...) of one weight tile: rows =
// tokens (NT of them, those beyond B are zero), 128 of K each, every unit as two 128-byte-swizzled [NT x 64] bf16
// tiles in the stage of the ring that its turn names.  A thread makes 16-byte chunks (8 elements).  A unit's
// operand is one trip to L2 away and a CTA has dozens of units a layer, so the work is cut in two: load_group only
// issues a group's loads (into registers), store_group converts and stores them; the caller issues the loads of
// the next group before it converts the current one.
template <int NT, int UG> struct RawGroup { float4 v[UG][NT * 16 / kWorkers][4]; };

template <int NT, int UG, int OP>
__device__ __forceinline__ void load_group(const Params& p, const PhaseInfo& f, int pair0, int n_units, RawGroup<NT, UG>& raw, int tid) {
    constexpr int CH = NT * 16 / kWorkers;                 // chunks per thread and unit
#pragma unroll
    for (int j = 0; j < UG; ++j) {
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            const int idx = tid + ci * kWorkers;
            const int row = idx >> 4, chunk = idx & 15;
            const int k = (pair0 + j) * kPair * BK + chunk * 8;
            const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
            raw.v[j][ci][0] = raw.v[j][ci][1] = raw.v[j][ci][2] = raw.v[j][ci][3] = zero;
            if (j < n_units && row < p.B && k < f.K) {
                if (OP == OP_NORMW) {
                    const float4* src = reinterpret_cast<const float4*>(p.resid + (size_t)row * p.H + k);
                    const float4* wv = reinterpret_cast<const float4*>(f.normw + k);
                    raw.v[j][ci][0] = __ldcg(src); raw.v[j][ci][1] = __ldcg(src + 1);
                    raw.v[j][ci][2] = __ldg(wv); raw.v[j][ci][3] = __ldg(wv + 1);
                } else {
                    const float4* src = reinterpret_cast<const float4*>(p.gu_acc + (size_t)row * 2 * p.I + 2 * (size_t)k);
                    raw.v[j][ci][0] = __ldcg(src); raw.v[j][ci][1] = __ldcg(src + 1);
                    raw.v[j][ci][2] = __ldcg(src + 2); raw.v[j][ci][3] = __ldcg(src + 3);
                }
            }
        }
    }
}

// rinv: per chunk row of this thread, 1 / rms of the row (SwiGLU only)
template <int NT, int UG, int OP>
__device__ __forceinline__ void store_group(const Params& p, const PhaseInfo& f, int n_units, const RawGroup<NT, UG>& raw,
                                            const float (&rinv)[NT * 16 / kWorkers], uint8_t* x_ring, uint32_t it,
                                            uint64_t* act_full, bool do_ssq, int tid) {
    constexpr int CH = NT * 16 / kWorkers;
    constexpr int kXStage = kPair * NT * 128;
    const int lane = tid & 31;
#pragma unroll
    for (int j = 0; j < UG; ++j) {
        if (j >= n_units) break;
        uint8_t* xs = x_ring + ((it + j) % kStages) * kXStage;
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            const int idx = tid + ci * kWorkers;
            const int row = idx >> 4, chunk = idx & 15;
            const int kb = chunk >> 3, c = chunk & 7;
            const float4 a = raw.v[j][ci][0], b = raw.v[j][ci][1], w0 = raw.v[j][ci][2], w1 = raw.v[j][ci][3];
            uint4 packed;
            float sq = 0.f;
            if (OP == OP_NORMW) {
                sq = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
                const float v[8] = {a.x * w0.x, a.y * w0.y, a.z * w0.z, a.w * w0.w, b.x * w1.x, b.y * w1.y, b.z * w1.z, b.w * w1.w};
                packed = pack8(v);
            } else {
                const float r = rinv[ci];
                const float v[8] = {silu_f(a.x * r) * (a.y * r), silu_f(a.z * r) * (a.w * r), silu_f(b.x * r) * (b.y * r),
                                    silu_f(b.z * r) * (b.w * r), silu_f(w0.x * r) * (w0.y * r), silu_f(w0.z * r) * (w0.w * r),
                                    silu_f(w1.x * r) * (w1.y * r), silu_f(w1.z * r) * (w1.w * r)};
                packed = pack8(v);
            }
            *reinterpret_cast<uint4*>(xs + kb * (NT * 128) + row * 128 + ((c ^ (row & 7)) << 4)) = packed;
            if (OP == OP_NORMW && do_ssq) {
                // the 16 chunks of a row sit in 16 neighbouring lanes
                sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                if ((lane & 15) == 0 && row < p.B) atomicAdd(f.ssq + row, sq);
            }
        }
        fence_proxy_async();
        mbar_arrive(&act_full[(it + j) % kStages]);
    }
}

// The token operand of the o-projection is the attention's result, which exists as up to kMaxSplit un-normalised
// parts per (request, kv head), each with the maximum and the sum of its weights: the parts are merged here, on their
// way into the operand (so the attention needs no second round among its CTAs).  Two units at a time, all their loads
// in flight together.
template <int NT>
__device__ __forceinline__ bool convert_segment_merge(const Params& p, const PhaseInfo& f, int u, int seg_end, uint8_t* x_ring, uint32_t& it,
                                                      uint64_t* empty, uint64_t* act_full, int S, volatile int* abort, int tid) {
    static_assert(NT * 16 == kWorkers, "one chunk per worker and unit");
    constexpr int kXStage = kPair * NT * 128;
    const int row = tid >> 4, chunk = tid & 15;
    const int kb = chunk >> 3, c = chunk & 7;
    const int G = p.NH / p.NKV;
    while (u < seg_end) {
        const int n = min(2, seg_end - u);
        float4 o[2][kMaxSplit][2];
        float2 ml[2][kMaxSplit];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int k = ((u + j) % f.kp) * kPair * BK + chunk * 8;
            const int h = k / HD, d = k % HD;
            const size_t part0 = ((size_t)(row * p.NKV + h / G) * kMaxSplit) * 16 + (h % G);
            const bool live = j < n && row < p.B && k < f.K;
#pragma unroll
            for (int z = 0; z < kMaxSplit; ++z) {
                o[j][z][0] = o[j][z][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                ml[j][z] = make_float2(-INFINITY, 0.f);
                if (live && z < S) {
                    const size_t r = part0 + (size_t)z * 16;
                    ml[j][z] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + r * 2));
                    const float4* src = reinterpret_cast<const float4*>(p.part_o + r * HD + d);
                    o[j][z][0] = __ldcg(src);
                    o[j][z][1] = __ldcg(src + 1);
                }
            }
        }
        for (int j = 0; j < n; ++j) {
            const uint32_t t = it + j;
            if (t >= (uint32_t)kStages && !mbar_wait(&empty[t % kStages], ((t / kStages) - 1) & 1, abort, p.status, 4)) return false;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (j >= n) break;
            float M = -INFINITY;
#pragma unroll
            for (int z = 0; z < kMaxSplit; ++z) M = fmaxf(M, ml[j][z].x);
            float L = 0.f, v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int z = 0; z < kMaxSplit; ++z) {
                const float wt = ml[j][z].x == -INFINITY ? 0.f : exp2f(ml[j][z].x - M);
                L += wt * ml[j][z].y;
                v[0] += wt * o[j][z][0].x; v[1] += wt * o[j][z][0].y; v[2] += wt * o[j][z][0].z; v[3] += wt * o[j][z][0].w;
                v[4] += wt * o[j][z][1].x; v[5] += wt * o[j][z][1].y; v[6] += wt * o[j][z][1].z; v[7] += wt * o[j][z][1].w;
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= inv;
            uint8_t* xs = x_ring + ((it + j) % kStages) * kXStage;
            *reinterpret_cast<uint4*>(xs + kb * (NT * 128) + row * 128 + ((c ^ (row & 7)) << 4)) = pack8(v);
            fence_proxy_async();
            mbar_arrive(&act_full[(it + j) % kStages]);
        }
        it += n;
        u += n;
    }
    return true;
}

// The token operands of the units [u, seg_end) of one weight tile, in groups of UG, the next group's loads in flight
// while the current one is converted.  Returns false if a wait ran out.
template <int NT, int UG, int OP>
__device__ __forceinline__ bool convert_segment(const Params& p, const PhaseInfo& f, int u, int seg_end, uint8_t* x_ring, uint32_t& it,
                                                uint64_t* empty, uint64_t* act_full, bool do_ssq, volatile int* abort, int tid) {
    constexpr int CH = NT * 16 / kWorkers;
    float rinv[CH];
#pragma unroll
    for (int ci = 0; ci < CH; ++ci) {
        const int row = (tid + ci * kWorkers) >> 4;
        rinv[ci] = 1.f;
        if (OP == OP_SWIGLU && row < p.B) rinv[ci] = 1.0f / sqrtf(__ldcg(p.ssq + kSsqStride + row) / (float)p.H + p.eps);
    }
    auto wait_stages = [&](int n) {
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            const uint32_t t = it + j;
            if (t >= (uint32_t)kStages) ok = mbar_wait(&empty[t % kStages], ((t / kStages) - 1) & 1, abort, p.status, 4);
        }
        return ok;
    };
    RawGroup<NT, UG> ra, rb;
    int pair = u % f.kp;
    load_group<NT, UG, OP>(p, f, pair, min(UG, seg_end - u), ra, tid);
    while (u < seg_end) {
        const int na = min(UG, seg_end - u), nb = min(UG, seg_end - u - na);
        if (nb > 0) load_group<NT, UG, OP>(p, f, pair + na, nb, rb, tid);
        if (!wait_stages(na)) return false;
        store_group<NT, UG, OP>(p, f, na, ra, rinv, x_ring, it, act_full, do_ssq, tid);
        it += na; u += na; pair += na;
        if (nb == 0) break;
        const int nc = min(UG, seg_end - u - nb);
        if (nc > 0) load_group<NT, UG, OP>(p, f, pair + nb, nc, ra, tid);
        if (!wait_stages(nb)) return false;
        store_group<NT, UG, OP>(p, f, nb, rb, rinv, x_ring, it, act_full, do_ssq, tid);
        it += nb; u += nb; pair += nb;
    }
    return true;
}

// this CTA's share of `n` floats at `ptr` becomes zero (n a multiple of 4, ptr 16-byte aligned)
__device__ __forceinline__ void zero_slice(float* ptr, long long n, int tid) {
    const long long n4 = n / 4;
    const long long a = n4 * blockIdx.x / gridDim.x, b = n4 * (blockIdx.x + 1) / gridDim.x;
    float4* q = reinterpret_cast<float4*>(ptr);
    for (long long i = a + tid; i < b; i += kWorkers) q[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Attention of a decode step.  Unit v of a layer is (request s, kv head kvh, part z of S): the keys of (s, kvh) are
// dealt in tiles of 32, tile i to part i % S and there to warp (i / S) % kAttWarps.
struct AttUnit { int s, kvh, z, S; };

__device__ __forceinline__ int att_split(const Params& p) {
    const int units = p.B * p.NKV;
    int S = (int)gridDim.x / units;
    return S < 1 ? 1 : (S > kMaxSplit ? kMaxSplit : S);
}
__device__ __forceinline__ AttUnit att_unit(const Params& p, int v, int S) {
    AttUnit a;
    a.S = S;
    a.z = v % S;
    a.kvh = (v / S) % p.NKV;
    a.s = v / (S * p.NKV);
    return a;
}

struct AttGeometry {
    const int32_t* table;
    int pos, kv_lo, kv_hi, t_begin, t_end;
};
__device__ __forceinline__ AttGeometry att_geometry(const Params& p, int s) {
    AttGeometry g;
    g.pos = p.positions[s];
    g.table = p.block_table + (size_t)s * p.max_pages;
    g.kv_hi = g.pos + 1;
    g.kv_lo = (p.window > 0 && g.pos - p.window + 1 > 0) ? g.pos - p.window + 1 : 0;
    g.t_begin = g.kv_lo / DKV;
    g.t_end = (g.kv_hi + DKV - 1) / DKV;
    return g;
}

// The row of the cache (page * 2 * NKV + kvh) * page_size + slot that holds key `lane` of tile t, or -1 outside
// [kv_lo, kv_hi).  The same in every layer (the layers of a group share the block table).
__device__ __forceinline__ int att_tile_row(const Params& p, const AttGeometry& g, int kvh, int t, int lane) {
    const int tk = t * DKV + lane;
    if (tk < g.kv_lo || tk >= g.kv_hi) return -1;
    return (g.table[tk / p.page_size] * 2 * p.NKV + kvh) * p.page_size + tk % p.page_size;
}

// keys and values of a tile into buffer `buf` of this warp; ridx: att_tile_row of this lane (rows of -1: zeros)
__device__ __forceinline__ void att_load_tile(const Params& p, const __nv_bfloat16* kv, __nv_bfloat16* my_k, int buf, int ridx, int lane) {
    __nv_bfloat16* kd = my_k + (size_t)buf * 2 * DKV * LD;
    const int v_rows = p.NKV * p.page_size;
#pragma unroll 4
    for (int c = lane; c < DKV * CPR; c += 32) {
        const int r_row = c / CPR, ch = c % CPR;
        const int r = __shfl_sync(0xffffffffu, ridx, r_row);
        __nv_bfloat16* dk = kd + r_row * LD + ch * 8;
        __nv_bfloat16* dv = dk + DKV * LD;
        if (r >= 0) {
            const __nv_bfloat16* src = kv + (size_t)r * HD + ch * 8;
            cp_async16(dk, src);
            cp_async16(dv, src + (size_t)v_rows * HD);
        } else {
            *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
        }
    }
}

// What a warp needs to ask for its first two tiles of the CTA's first unit before q exists: worked out once per
// step (it is the same for every layer).  n: how many of them hold only earlier positions (the tile with the new
// token has to wait for this layer's key).
struct AttPrefetch { int n; int ridx[2]; };
__device__ __forceinline__ AttPrefetch att_prefetch_plan(const Params& p, const AttUnit& a, int tid) {
    AttPrefetch pf;
    pf.n = 0;
    pf.ridx[0] = pf.ridx[1] = -1;
    const int warp = tid >> 5, lane = tid & 31;
    if (warp < kAttWarps) {
        const AttGeometry g = att_geometry(p, a.s);
        for (; pf.n < 2; ++pf.n) {
            const int t = g.t_begin + a.z + a.S * (warp + kAttWarps * pf.n);
            if (t >= g.t_end - 1) break;
            pf.ridx[pf.n] = att_tile_row(p, g, a.kvh, t, lane);
        }
    }
    return pf;
}
__device__ __forceinline__ int attention_prefetch(const Params& p, const LayerDesc* L, const AttPrefetch& pf, uint8_t* scratch, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    if (warp < kAttWarps) {
        __nv_bfloat16* my_k = reinterpret_cast<__nv_bfloat16*>(scratch) + 16 * LD + (size_t)warp * 4 * DKV * LD;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (i < pf.n) {
                att_load_tile(p, L->kv, my_k, i, pf.ridx[i], lane);
                cp_async_commit();
            }
        }
    }
    return pf.n;
}

// The unit's share of the attention, by the workers (the first kAttWarps warps of them compute; all take part in
// the barriers): the new token's q (G heads) and k are taken from qkv_acc (divided by the row's rms, plus bias),
// rotated, k and v go into the cache (by the part that owns the last tile), and the G heads attend over the part's
// keys.  The part leaves its un-normalised result with its maximum and sum; the o-projection's operand is made of
// the parts (convert_segment_merge).
__device__ __forceinline__ void attention_unit(const Params& p, const LayerDesc* L, const AttUnit& a, uint8_t* scratch,
                                               int issued, int tid, unsigned long long* trace = nullptr) {
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(scratch);          // [16][LD]  (G heads, zero-padded)
    __nv_bfloat16* kvs = qs + 16 * LD;                                      // [kAttWarps][2 buffers][K | V][DKV][LD]
    const int warp = tid >> 5, lane = tid & 31;
    const int s = a.s, kvh = a.kvh, S = a.S;
    const int G = p.NH / p.NKV;
    const int half = HD / 2;
    const AttGeometry g = att_geometry(p, s);
    const int pos = g.pos, t_begin = g.t_begin, t_end = g.t_end;
    const float* row = p.qkv_acc + (size_t)s * p.QKV;
    const float rms = 1.0f / sqrtf(__ldcg(p.ssq + s) / (float)p.H + p.eps);
    const int slot = p.slot_mapping[s];
    __nv_bfloat16* kv = L->kv;
    __nv_bfloat16* page_base = kv + ((size_t)(slot / p.page_size) * 2 * p.NKV + kvh) * p.page_size * HD + (size_t)(slot % p.page_size) * HD;
    const float* bias = L->qkv_bias;
    __nv_bfloat16* my_k = kvs + (size_t)warp * 4 * DKV * LD;               // [buffer][K | V]
    const bool writes_kv = a.z == (t_end - 1 - t_begin) % S;               // the part that owns the tile with the new token
    const int t_first = t_begin + a.z + S * warp, t_step = S * kAttWarps;  // this warp's tiles

    // 1. rotate q (G heads) and k (one head), copy v; q to shared memory, k and v to the cache
    for (int i = tid; i < 16 * CPR; i += kWorkers)
        if (i / CPR >= G) *reinterpret_cast<uint4*>(qs + (i / CPR) * LD + (i % CPR) * 8) = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < (G + 2) * half; i += kWorkers) {
        const int h = i / half, d = i % half;                              // h < G: q head; G: k; G + 1: v
        if (h >= G && !writes_kv) continue;
        const int src_head = h < G ? kvh * G + h : (h == G ? p.NH + kvh : p.NH + p.NKV + kvh);
        float x0 = __ldcg(row + src_head * HD + d) * rms, x1 = __ldcg(row + src_head * HD + d + half) * rms;
        if (bias) { x0 += bias[src_head * HD + d]; x1 += bias[src_head * HD + d + half]; }
        if (p.rotary && h <= G) {
            const float2 cs = __ldcg(p.rope_tab + (size_t)s * half + d);
            const float y0 = x0 * cs.x - x1 * cs.y, y1 = x0 * cs.y + x1 * cs.x;
            x0 = y0;
            x1 = y1;
        }
        if (h < G) {
            qs[h * LD + d] = __float2bfloat16_rn(x0);
            qs[h * LD + d + half] = __float2bfloat16_rn(x1);
        } else {
            __nv_bfloat16* dst = page_base + (h == G ? 0 : (size_t)p.NKV * p.page_size * HD);
            dst[d] = __float2bfloat16_rn(x0);
            dst[d + half] = __float2bfloat16_rn(x1);
        }
    }
    __threadfence_block();        // the new key and value are read back below by whichever warp gets their tile
    workers_sync();
    if (trace && tid == 0) trace[2] = global_ns();

    // 2. every computing warp walks its share of the key tiles
    const bool valid_a = (lane >> 2) < G, valid_b = (lane >> 2) + 8 < G;
    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    if (warp < kAttWarps) {
        int n_done = 0;
        for (int t = t_first; t < t_end; t += t_step, ++n_done) {
            const int buf = n_done & 1;
            for (; issued < n_done + 2 && t_first + issued * t_step < t_end; ++issued) {
                att_load_tile(p, kv, my_k, issued & 1, att_tile_row(p, g, kvh, t_first + issued * t_step, lane), lane);
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
                uint32_t af[4];
                ldmatrix_x4(af, qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int nb = 0; nb < DKV / 16; ++nb) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kb + (nb * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sc[2 * nb], af, b[0], b[1]);
                    mma_bf16(sc[2 * nb + 1], af, b[2], b[3]);
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
    }

    // 3. merge the warps' partial results in shared memory (the tile buffers are free now), in warp order
    workers_sync();
    if (trace && tid == 0) trace[3] = global_ns();
    float* mo = reinterpret_cast<float*>(kvs);                             // [kAttWarps][16][HD]
    float* ml = mo + kAttWarps * 16 * HD;                                  // [kAttWarps][16][2]
    if (warp < kAttWarps) {
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
    workers_sync();
    const size_t unit = (size_t)s * p.NKV + kvh;
    float* my_po = p.part_o + (unit * kMaxSplit + a.z) * 16 * HD;
    float* my_pml = p.part_ml + (unit * kMaxSplit + a.z) * 32;
    for (int i = tid; i < G * HD; i += kWorkers) {
        const int r = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttWarps; ++w) M = fmaxf(M, ml[(w * 16 + r) * 2]);
        float Lsum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kAttWarps; ++w) {
            const float mw = ml[(w * 16 + r) * 2];
            const float wt = mw == -INFINITY ? 0.f : exp2f(mw - M);
            Lsum += wt * ml[(w * 16 + r) * 2 + 1];
            acc += wt * mo[((size_t)w * 16 + r) * HD + d];
        }
        my_po[r * HD + d] = acc;
        if (d == 0) { my_pml[r * 2] = M; my_pml[r * 2 + 1] = Lsum; }
    }
    workers_sync();               // the scratch is free for the next unit
    if (trace && tid == 0) trace[6] = global_ns();
}

template <int NT>
struct Cfg {
    static constexpr int kXStage = kPair * NT * 128;                       // two [NT x 64] bf16 tiles
    static constexpr int kAttScratch = (kAttBytes + 1023) / 1024 * 1024;   // apart from the ring: filled during the qkv product
    static constexpr int kTmemCols = kAccs * NT < 32 ? 32 : kAccs * NT;
    static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "tensor memory columns: a power of two");
    static constexpr int kSmemBytes = 1024 + kStages * kStageW + kStages * kXStage + kAttScratch + 512;
    static_assert(kSmemBytes <= kSmemLimit, "shared memory");
};

template <int NT>
__global__ void __launch_bounds__(kThreads, 1)
decode_layers_kernel(const Params p) {
    using C = Cfg<NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* w_ring = smem;                                    // [kStages][2][128 x 64] bf16
    uint8_t* x_ring = smem + kStages * kStageW;                // [kStages][2][NT x 64] bf16
    uint8_t* att_scratch = x_ring + kStages * C::kXStage;      // q, key and value tiles, the warps' partial results
    uint64_t* bars = reinterpret_cast<uint64_t*>(att_scratch + C::kAttScratch);
    uint64_t* full = bars;                                     // TMA -> MMA
    uint64_t* empty = bars + kStages;                          // MMA -> TMA and workers
    uint64_t* act_full = bars + 2 * kStages;                   // workers -> MMA
    uint64_t* acc_full = bars + 3 * kStages;                   // [kAccs] MMA -> workers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + kAccs);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        *abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&act_full[s], kWorkers); }
        for (int a = 0; a < kAccs; ++a) mbar_init(&acc_full[a], 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- the weight streamer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (UnitWalk ld = walk_begin(p); !ld.done; walk_next(p, ld), ++it) {
                const int s = it % kStages;
                if (it >= (uint32_t)kStages && !(ok = mbar_wait(&empty[s], ((it / kStages) - 1) & 1, abort, p.status, 1))) break;
                mbar_arrive_expect_tx(&full[s], kStageW);
                tma_load_3d(w_ring + s * kStageW, ld.f.map, &full[s], 0, (ld.u / ld.f.kp) * BM, (ld.u % ld.f.kp) * kPair);
            }
            // the copies asked for last must have landed before the CTA's shared memory goes (after a normal run
            // they have: the MMAs that read them are done; after an abort this waits for them, with a limit)
            const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0;
            for (uint32_t j = first; j < it; ++j) {
                const unsigned long long t0 = global_ns();
                while (!mbar_test_wait(&full[j % kStages], (j / kStages) & 1) && global_ns() - t0 < 20000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- the MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, NT);
            uint32_t it = 0, seg = 0;
            bool ok = true;
            for (UnitWalk w = walk_begin(p); !w.done && ok;) {
                // a segment: this CTA's units of one weight tile; its sums gather in accumulator seg % kAccs
                const int tile = w.u / w.f.kp, layer = w.layer, ph = w.ph;
                const uint32_t d_tmem = tmem_base + (seg % kAccs) * NT;
                bool fresh = true;
                while (!w.done && w.layer == layer && w.ph == ph && w.u / w.f.kp == tile) {
                    const int s = it % kStages;
                    const uint32_t par = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&full[s], par, abort, p.status, 2))) break;
                    if (!(ok = mbar_wait(&act_full[s], par, abort, p.status, 3))) break;
                    tc_fence_after_sync();
                    const uint64_t w_desc = umma_desc_k_sw128(smem_u32(w_ring + s * kStageW));
                    const uint64_t x_desc = umma_desc_k_sw128(smem_u32(x_ring + s * C::kXStage));
#pragma unroll
                    for (int j = 0; j < kPair; ++j) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            umma_bf16(d_tmem, umma_desc_advance(w_desc, j * (BM * BK * 2) + k * UMMA_K * 2),
                                      umma_desc_advance(x_desc, j * (NT * 128) + k * UMMA_K * 2), idesc, !(fresh && j == 0 && k == 0));
                        }
                    }
                    fresh = false;
                    umma_commit(&empty[s]);
                    walk_next(p, w);
                    ++it;
                }
                if (ok) umma_commit(&acc_full[seg % kAccs]);
                ++seg;
            }
        }
    } else {
        // ---------------------------------------------------------------- the workers
        const int tid = threadIdx.x - 64;
        const int quarter = warp & 3, col_half = (warp - 2) >> 2;   // two warps share a quarter of the lanes and split the tokens
        constexpr int UG = NT <= 16 ? 2 : 1;                        // units whose operands are fetched together
        const int S = att_split(p), att_units = p.B * p.NKV * S;
        const int half = HD / 2;
        forge::pdl_wait();                                   // the residual stream comes from the kernel before
        uint32_t it = 0, seg = 0, nbar = 0;
        int att_issued = 0;
        bool ok = true;
        // (profiling) slot k of the record of the barrier that will end the current phase
        auto mark = [&](int k) {
            if (p.timeline && tid == 0) p.timeline[((size_t)blockIdx.x * (1 + 5 * p.num_layers) + nbar) * 8 + k] = global_ns();
        };
        // before the first layer: the first product adds into qkv_acc and ssq1; the step's rotary angles
        zero_slice(p.qkv_acc, (long long)p.B * p.QKV, tid);
        if (blockIdx.x == 0 && tid < kSsqStride) p.ssq[tid] = 0.f;
        if (p.rotary) {
            for (int i = blockIdx.x * kWorkers + tid; i < p.B * half; i += gridDim.x * kWorkers) {
                const int d = i % half;
                const float freq = 1.0f / powf(p.theta, (2.0f * (float)d) / (float)HD);
                float sn, cs;
                sincosf((float)p.positions[i / half] * freq, &sn, &cs);
                p.rope_tab[i] = make_float2(cs, sn);
            }
        }
        ok = grid_barrier(p, ++nbar * gridDim.x, abort, tid);
        if (tid == 0) forge::pdl_launch_dependents();        // every CTA is resident: the next kernel may be set up
        const AttPrefetch att_pf = (int)blockIdx.x < att_units ? att_prefetch_plan(p, att_unit(p, blockIdx.x, S), tid) : AttPrefetch{0, {-1, -1}};
        for (int layer = 0; layer < p.num_layers && ok; ++layer) {
            const LayerDesc* L = p.layers + layer;
            for (int ph = 0; ph < 4 && ok; ++ph) {
                const PhaseInfo f = phase_info(p, L, ph);
                int u0, u1;
                unit_range(f, u0, u1);
                for (int u = u0; u < u1 && ok;) {
                    // up to kAccs tiles: first the token operands of all their units (so that no MMA waits for an
                    // epilogue), then the tiles' sums
                    int tiles[kAccs], n_tiles = 0;
                    const uint32_t seg0 = seg;
                    while (u < u1 && n_tiles < kAccs && ok) {
                        const int tile = u / f.kp;
                        const int seg_end = min(u1, (tile + 1) * f.kp);
                        const bool do_ssq = f.ssq != nullptr && tile == 0;
                        if (f.op == OP_NORMW) ok = convert_segment<NT, UG, OP_NORMW>(p, f, u, seg_end, x_ring, it, empty, act_full, do_ssq, abort, tid);
                        else if (f.op == OP_MERGE) ok = convert_segment_merge<NT>(p, f, u, seg_end, x_ring, it, empty, act_full, S, abort, tid);
                        else ok = convert_segment<NT, UG, OP_SWIGLU>(p, f, u, seg_end, x_ring, it, empty, act_full, false, abort, tid);
                        tiles[n_tiles++] = tile;
                        u = seg_end;
                    }
                    if (!ok) break;
                    mark(2);
                    for (int i = 0; i < n_tiles; ++i, ++seg) {
                        // a tile's (partial) sums: one output feature per thread, tokens along the columns
                        if (!(ok = mbar_wait(&acc_full[seg % kAccs], (seg / kAccs) & 1, abort, p.status, 5))) break;
                        if (i == 0) mark(3);
                        tc_fence_after_sync();
                        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (seg % kAccs) * NT;
                        const int n = tiles[i] * BM + quarter * 32 + lane;
#pragma unroll
                        for (int c = 16 * col_half; c < NT; c += 32) {
                            if (c >= p.B) break;                 // uniform over the warp
                            uint32_t r[16];
                            tmem_ld_32x32b_x16(t_row + c, r);
                            tmem_ld_wait();
                            if (n < f.n_out) {
#pragma unroll
                                for (int e = 0; e < 16; ++e)
                                    if (c + e < p.B) atomicAdd(f.out + (size_t)(c + e) * f.ldo + n, __uint_as_float(r[e]));
                            }
                        }
                        tc_fence_before_sync();
                    }
                    if (!ok) seg = seg0 + n_tiles;
                    mark(4);
                }
                if (!ok) break;
                if (ph == 0) {
                    // the keys of earlier positions do not wait for this layer's q: they travel during the barrier
                    att_issued = attention_prefetch(p, L, att_pf, att_scratch, tid);
                } else if (ph == 3) {
                    // nobody reads qkv_acc and ssq1 any more in this layer: clear them for the next one
                    zero_slice(p.qkv_acc, (long long)p.B * p.QKV, tid);
                    if (blockIdx.x == 0 && tid < kSsqStride) p.ssq[tid] = 0.f;
                }
                if (!(ok = grid_barrier(p, ++nbar * gridDim.x, abort, tid))) break;
                if (ph == 0) {
                    for (int v = blockIdx.x; v < att_units; v += gridDim.x) {
                        attention_unit(p, L, att_unit(p, v, S), att_scratch, att_issued, tid,
                                       p.timeline ? p.timeline + ((size_t)blockIdx.x * (1 + 5 * p.num_layers) + nbar) * 8 : nullptr);
                        att_issued = 0;
                    }
                    zero_slice(p.gu_acc, (long long)p.B * 2 * p.I, tid);
                    if (blockIdx.x == 0 && tid < kSsqStride) p.ssq[kSsqStride + tid] = 0.f;
                    if (!(ok = grid_barrier(p, ++nbar * gridDim.x, abort, tid))) break;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
    // the CTA that is through last (every CTA has left the last barrier by then) clears the counters for the
    // next launch; after an abort they stay as they are, for the host to see and to clear
    if (threadIdx.x == 64 && !*abort) {
        if (atomicAdd(p.barrier + 2, 1u) == gridDim.x - 1) {
            p.barrier[0] = 0u;
            p.barrier[2] = 0u;
            __threadfence();
        }
    }
}

// One CTA, one barrier that is one arrival short: the wait runs out and the status bit is raised.
__global__ void __launch_bounds__(kWorkers) barrier_probe_kernel(const Params p) {
    __shared__ int abort_flag;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    grid_barrier(p, 2u, &abort_flag, threadIdx.x);
}

template <int NT>
int launch_layers(const Params& p, cudaStream_t stream) {
    using C = Cfg<NT>;
    static forge::PerDeviceFlag configured_on;
    static int sms[forge::PerDeviceFlag::kMax + 1] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= forge::PerDeviceFlag::kMax) dev = forge::PerDeviceFlag::kMax;
    bool& configured = configured_on.current();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "decode_layers: cannot set %d bytes of shared memory: %s", C::kSmemBytes, cudaGetErrorString(e));
        int per_sm = 0, n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<NT>, kThreads, C::kSmemBytes);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev == forge::PerDeviceFlag::kMax ? 0 : dev);
        if (e != cudaSuccess || per_sm < 1 || n < 1)
            return forge::fail(FORGE_ERR_LAUNCH, "decode_layers: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
        sms[dev] = n;       // one CTA per SM: all of them are resident at once, which the grid barrier needs
        configured = true;
    }
    return forge::check_launch("decode_layers", forge::launch(decode_layers_kernel<NT>, dim3(sms[dev]), dim3(kThreads), C::kSmemBytes, stream, 1, p));
}

}  // namespace

extern "C" int forge_decode_layers_desc_bytes() { return (int)sizeof(LayerDesc); }
extern "C" int forge_decode_layers_head_dim() { return HD; }
extern "C" int forge_decode_layers_max_tokens() { return kMaxTokens; }

// Why these sizes cannot run here, or null.  (The caller falls back to one kernel per operation.)
static const char* unsupported(int B, int H, int I, int NH, int NKV, int head_dim) {
    if (head_dim != HD) return "built for another head size";
    if (B < 1 || B > kMaxTokens) return "more than 16 tokens";
    if (NH <= 0 || NKV <= 0 || NH % NKV != 0 || NH / NKV > 16) return "more than 16 query heads per kv head";
    if (H % 64 != 0 || I % 64 != 0 || (NH * HD) % 64 != 0) return "a reduction size that is not a multiple of 64";
    return nullptr;
}

extern "C" int forge_decode_layers_supports(int B, int H, int I, int NH, int NKV, int head_dim) {
    return unsupported(B, H, I, NH, NKV, head_dim) == nullptr ? 1 : 0;
}

// Writes the description of one layer (tensor maps of its four matrices, pointers) to descs[layer] on the device.
// Matrices are bf16 row-major [out, in]: wqkv [(NH+2NKV)*HD, H], wo [H, NH*HD], wgu [2I, H] (gate and up rows
// interleaved), wdown [H, I]; norms fp32 [H]; bias fp32 or null; kv the layer's cache.  Synchronous; call at load time.
extern "C" int forge_decode_layers_describe(void* descs, int layer, const void* wqkv, const void* wo, const void* wgu,
                                            const void* wdown, const float* norm1, const float* norm2, const float* bias,
                                            void* kv, int H, int I, int NH, int NKV, int head_dim) {
    const char* why = unsupported(1, H, I, NH, NKV, head_dim);
    if (why) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_layers: %s", why);
    LayerDesc d;
    const char* err = "";
    const int QKV = (NH + 2 * NKV) * HD;
    if (!sm100::bf16_kblock_map(wqkv, QKV, H, BM, kPair, &d.w_qkv, &err) || !sm100::bf16_kblock_map(wo, H, NH * HD, BM, kPair, &d.w_o, &err) ||
        !sm100::bf16_kblock_map(wgu, 2 * I, H, BM, kPair, &d.w_gu, &err) || !sm100::bf16_kblock_map(wdown, H, I, BM, kPair, &d.w_down, &err))
        return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_layers: %s", err);
    d.norm1 = norm1;
    d.norm2 = norm2;
    d.qkv_bias = bias;
    d.kv = static_cast<__nv_bfloat16*>(kv);
    cudaError_t e = cudaMemcpy(static_cast<uint8_t*>(descs) + (size_t)layer * sizeof(LayerDesc), &d, sizeof(LayerDesc), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return forge::fail(FORGE_ERR_LAUNCH, "decode_layers: %s", cudaGetErrorString(e));
    return FORGE_OK;
}

// Runs `num_layers` layers on the residual stream resid [B, H] (fp32, in place).  Scratch, all the caller's:
// qkv_acc fp32 [B, (NH+2NKV)*HD], gu_acc fp32 [B, 2I], ssq fp32 [128], rope_tab fp32 [B, HD], part_o fp32
// [B*NKV, 4, 16, HD], part_ml fp32 [B*NKV, 4, 16, 2] and barrier uint32 [4] (zero before the first call; the kernel
// leaves it zero unless a wait ran out).
// Calls on one device must not overlap (they would share the scratch).  prefetch_units: non-zero: weights are asked
// into L2 two or three products before they are needed (a layer's matrices should fit the L2).  timeline: null, or uint64 [CTAs (one per SM)]
// [1 + 5 * num_layers barriers][2] that receives the time (ns) at which each CTA reached and left each barrier.
extern "C" int forge_decode_layers(const void* descs, int num_layers, float* resid, float* qkv_acc, float* gu_acc, float* ssq,
                                   void* rope_tab, float* part_o, float* part_ml,
                                   const int32_t* block_table, const int32_t* positions,
                                   const int32_t* slot_mapping, unsigned int* barrier, int* status, int B, int H, int I, int NH,
                                   int NKV, int head_dim, int page_size, int max_pages, int window, int rotary, float theta,
                                   float scale, float eps, int prefetch_units, unsigned long long* timeline, cudaStream_t stream) {
    const char* why = unsupported(B, H, I, NH, NKV, head_dim);
    if (why) return forge::fail(FORGE_ERR_UNSUPPORTED, "decode_layers: %s", why);
    if (num_layers < 0 || page_size <= 0 || max_pages <= 0) return forge::fail(FORGE_ERR_ARG, "decode_layers: bad sizes");
    if (num_layers == 0) return FORGE_OK;
    Params p{static_cast<const LayerDesc*>(descs), num_layers, resid, qkv_acc, gu_acc, ssq,
             static_cast<float2*>(rope_tab), part_o, part_ml, block_table, positions, slot_mapping, barrier, status, B, H, I, NH, NKV, (NH + 2 * NKV) * HD, page_size, max_pages,
             window, rotary, theta, scale * 1.4426950408889634f, eps, sm100::kWaitLimitNs, prefetch_units < 0 ? 0 : prefetch_units, timeline};
    return launch_layers<16>(p, stream);
}

// For the test of the bounded wait: one CTA arrives at a barrier that expects two; the wait must run out after
// limit_ns, raise bit 1 (and bit 20) of *status and the abort word barrier[1], and the kernel must return.
extern "C" int forge_decode_layers_barrier_probe(unsigned int* barrier, int* status, unsigned long long limit_ns, cudaStream_t stream) {
    Params p{};
    p.barrier = barrier;
    p.status = status;
    p.wait_limit_ns = limit_ns;
    barrier_probe_kernel<<<1, kWorkers, 0, stream>>>(p);
    return forge::check_launch("barrier_probe");
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
