// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tile loads,
// TMEM allocation, tcgen05 MMA / commit / load, and the UMMA shared-memory and instruction descriptors.
//
// Every wait here has a time limit.  A wait that runs out raises `abort` (a flag in shared memory that
// all loops of the CTA poll) and bit 1 of the kernel's status word in global memory; the CTA then drains
// its copies in flight, frees its TMEM and returns, so a logic error shows up as an error code on the
// host instead of a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

#ifndef FORGE_WAIT_LIMIT_NS
#define FORGE_WAIT_LIMIT_NS 2000000000ull   // 2 s
#endif
constexpr unsigned long long kWaitLimitNs = FORGE_WAIT_LIMIT_NS;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase of `parity` to complete.  Returns false (after raising the flags) if another part
// of the CTA has aborted or the time limit passes.
// `where` (0..26) tags the wait: on expiry bit 4 + where of the status word is raised too, which tells
// a post-mortem which barrier was never completed.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait with an upper limit (ns) on how long the hardware may keep the thread suspended; it still wakes
// the thread as soon as the phase completes.
__device__ __forceinline__ bool mbar_try_wait_for(uint64_t* bar, uint32_t parity, uint32_t suspend_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_ns)
        : "memory");
    return ok != 0;
}
template <bool kProbeFirst = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* status, int where = 0) {
    // Suspending waits: the hardware wakes the thread the moment the phase completes (a polling loop with
    // sleeps in it notices a completed phase late, and in a short pipeline that delay is a bubble); the
    // suspend limit bounds how long an abort or the time limit can go unnoticed.
    // where most waits find their phase complete already, a plain probe first is cheaper than a suspending wait
    if (kProbeFirst && mbar_test_wait(bar, parity)) return true;
    if (mbar_try_wait_for(bar, parity, 1000)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (mbar_try_wait_for(bar, parity, 4000)) return true;
        if (*abort) return false;
        if (global_ns() - t0 > kWaitLimitNs) {
            *abort = 1;
            if (status) atomicOr(status, 2 | (1 << (4 + where)));
            return false;
        }
    }
}

// ----------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2D tile store shared -> global (the box is clipped at the tensor's edges), and the same as an fp32 add into
// global memory, done by the L2; both join the thread's current bulk group.  c0 * element size must be a
// multiple of 16 bytes, and neither coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of the thread's bulk groups still READ their shared memory / are still in flight
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// 2D tile load global -> shared; c0 is the innermost (contiguous) coordinate in elements, c1 the row.
// c0 * element size must be a multiple of 16 bytes.  Out-of-range parts of the box are filled with zeros
// and still count toward the barrier's byte total.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// 3D tile load: c0 innermost (elements), then c1, c2.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Makes shared-memory writes of this thread (generic proxy) visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- TMEM
// Whole-warp operations (.sync.aligned).  ncols: power of two, 32..512.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------- MMA
// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes (64 elements) wide
// and were written by TMA with 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset),
// the leading byte offset is unused for swizzled K-major layouts (set to 1), descriptor version 1
// (Blackwell), layout type 2 = SWIZZLE_128B.  The tile base must be 1024-byte aligned; stepping along K
// by 16 elements adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);   // start address, bits [0,14)
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (>>4), bits [16,30)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset (>>4), bits [32,46)
    d |= static_cast<uint64_t>(1) << 46;                      // version, bits [46,48)
    d |= static_cast<uint64_t>(2) << 61;                      // layout type, bits [61,64)
    return d;
}
// The descriptor of the same kind of tile `bytes` further on in shared memory (a multiple of 16; the start
// address field holds address >> 4 and shared memory ends below 2^18, so the sum never leaves the field).  One
// thread issues every MMA of a CTA and, being alone in its warp, runs an instruction every few cycles: building
// a descriptor from scratch for each MMA costs more than a small MMA takes, adding to a base does not.
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) {
    const uint32_t lo = static_cast<uint32_t>(desc) + (bytes >> 4);
    return (desc & 0xffffffff00000000ull) | lo;
}
// Descriptor of an MN-major bf16 tile: rows are K indices, each row holds 64 contiguous MN elements (128
// bytes), written by TMA with 128-byte swizzle.  8-row groups along K are 1024 bytes apart (stride byte
// offset); the leading byte offset is the distance between 64-element blocks along MN (`mn_block_bytes`,
// unused when the operand is 64 wide).  Stepping along K by 16 rows adds 2048 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_block_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>((mn_block_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor of kind::f16: D fp32 (bits [4,6) = 1), A and B bf16 (bits [7,10) and [10,13) = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at bits [17,23), M >> 4 at bits [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}
// As above with B MN-major (bit 16).
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32_bmn(int m, int n) {
    return umma_idesc_bf16_f32(m, n) | (1u << 16);
}
// D[tmem] (+)= A[smem] . B[smem]^T ; issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The barrier gets one arrival when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace sm100

// ------------------------------------------------------------------------- host: tensor maps for TMA
#include <cudaTypedefs.h>

#include <map>
#include <mutex>
#include <tuple>

namespace sm100 {

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

// Map of a row-major bf16 matrix [rows, cols] (cols contiguous) read in boxes of [box_rows, 64 columns]
// with 128-byte swizzle.  Needs a 16-byte aligned base and cols % 8 == 0.  Maps are cached by
// (pointer, shape, box): weights keep theirs for the life of the process.
inline bool bf16_tile_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out, const char** err) {
    using Key = std::tuple<const void*, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{ptr, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    auto fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols % 8) != 0) {
        *err = "TMA needs a 16-byte aligned base and a row of a multiple of 8 bf16";
        return false;
    }
    CUtensorMap m;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed"; return false; }
    if (cache.size() > 4096) cache.clear();   // activation buffers come and go; weights re-enter on next use
    cache.emplace(key, m);
    *out = m;
    return true;
}

// Map of a row-major fp32 matrix [rows, cols] written in boxes of [box_rows, 32 columns] (128 bytes a row) with
// 128-byte swizzle.  Needs a 16-byte aligned base and cols % 4 == 0.
inline bool f32_tile_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out, const char** err) {
    using Key = std::tuple<const void*, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{ptr, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    auto fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols % 4) != 0) {
        *err = "TMA needs a 16-byte aligned base and a row of a multiple of 4 floats";
        return false;
    }
    CUtensorMap m;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 4};
    const cuuint32_t box[2] = {32u, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed"; return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// Map of the same row-major bf16 matrix [rows, cols], cols % 64 == 0, seen as {64 columns, rows, cols / 64
// k-blocks}: a box {64, box_rows, group} brings `group` consecutive k-blocks of `box_rows` rows with ONE
// instruction and lands as `group` 128-byte-swizzled [box_rows x 64] tiles one after the other.  Coordinates
// are (0, row, k-block).  Rows and k-blocks out of range are filled with zeros.
inline bool bf16_kblock_map(const void* ptr, int rows, int cols, int box_rows, int group, CUtensorMap* out, const char** err) {
    using Key = std::tuple<const void*, int, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{ptr, rows, cols, box_rows, group};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    auto fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols % 64) != 0 || group < 1 || group > 256 || box_rows > 256) {
        *err = "the k-block view needs a 16-byte aligned base, a row of a multiple of 64 bf16 and boxes of at most 256";
        return false;
    }
    CUtensorMap m;
    const cuuint64_t dims[3] = {64u, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 64)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, 128u};
    const cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(group)};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed (k-block view)"; return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// Map of q [tokens, heads, 64 * blocks] bf16 read in boxes of [box_tokens, box_heads, 64]: a tile of query
// rows ordered (token, head of one kv group), 128 bytes each, 128-byte swizzle.
inline bool bf16_q_map(const void* ptr, int tokens, int heads, int head_dim, int box_tokens, int box_heads,
                       CUtensorMap* out, const char** err) {
    using Key = std::tuple<const void*, int, int, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{ptr, tokens, heads, head_dim, box_tokens, box_heads};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    auto fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || head_dim % 64 != 0) { *err = "q map needs a 16-byte aligned base and head_dim % 64 == 0"; return false; }
    CUtensorMap m;
    const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)heads * head_dim * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled (q) failed"; return false; }
    if (cache.size() > 1024) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

}  // namespace sm100
