// Index checks for the kernels that follow block tables and slot mappings, for a build made with -DFORGE_CHECKS=1.
//
// A page id taken from a block table, a slot taken from a slot mapping and a token index are the three numbers
// with which a kernel leaves the memory it was given if the host's bookkeeping is wrong.  In a checks build every
// such number is tested before it is used: a bad one raises bit 4 of the step's status word, records what it was,
// and the access is skipped (the kernel goes on with zeros), so a bookkeeping error shows as an error code on the
// host with the offending index instead of as a memory fault.  An ordinary build compiles the tests away.
//
// The predicates are plain functions of integers, compiled for host and device alike, so that they are tested on
// the CPU (with bad pages and slots that no GPU is ever given).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FORGE_HD __host__ __device__ __forceinline__
#else
#define FORGE_HD inline
#endif

namespace forge {

// a page id that may be dereferenced: inside the pool (released pages are -1 and never reach this test)
FORGE_HD bool page_in_pool(long long page, long long num_pages) { return page >= 0 && page < num_pages; }
// a slot (page * page_size + offset) that may be written
FORGE_HD bool slot_in_pool(long long slot, long long num_pages, long long page_size) {
    return page_size > 0 && slot >= 0 && slot < num_pages * page_size;
}
// a row of the step's flat token list
FORGE_HD bool token_in_step(long long t, long long num_tokens) { return t >= 0 && t < num_tokens; }

struct CheckBounds {
    int num_pages, page_size, num_tokens;
    int* status;            // the step's status word; bit 4 (16): an index was out of range
    int* first_bad;         // [3]: kind (1 page, 2 slot, 3 token), the value, the limit; written by the first offender
};

}  // namespace forge

#if defined(__CUDACC__)
#if FORGE_CHECKS
namespace forge {
static __device__ CheckBounds g_check_bounds;   // one per source file, set by its forge_checks_configure_<name> before a step

__device__ __forceinline__ void check_failed(int kind, long long value, long long limit) {
    const CheckBounds& b = g_check_bounds;
    if (b.status && (atomicOr(b.status, 16) & 16) == 0 && b.first_bad) {
        b.first_bad[0] = kind;
        b.first_bad[1] = (int)value;
        b.first_bad[2] = (int)limit;
    }
}
__device__ __forceinline__ bool check_page(long long page) {
    if (page_in_pool(page, g_check_bounds.num_pages)) return true;
    check_failed(1, page, g_check_bounds.num_pages);
    return false;
}
__device__ __forceinline__ bool check_slot(long long slot) {
    if (slot_in_pool(slot, g_check_bounds.num_pages, g_check_bounds.page_size)) return true;
    check_failed(2, slot, (long long)g_check_bounds.num_pages * g_check_bounds.page_size);
    return false;
}
__device__ __forceinline__ bool check_token(long long t) {
    if (token_in_step(t, g_check_bounds.num_tokens)) return true;
    check_failed(3, t, g_check_bounds.num_tokens);
    return false;
}
}  // namespace forge
#define FORGE_PAGE_OK(page) (forge::check_page(page))
#define FORGE_SLOT_OK(slot) (forge::check_slot(slot))
#define FORGE_TOKEN_OK(t) (forge::check_token(t))
// every source file that includes this header exports its own configure entry (the bounds live in that file)
#define FORGE_DEFINE_CHECKS_ENTRY(name)                                                                              \
    extern "C" int forge_checks_configure_##name(int num_pages, int page_size, int num_tokens, int* status, int* first_bad, \
                                                 cudaStream_t stream) {                                               \
        forge::CheckBounds b{num_pages, page_size, num_tokens, status, first_bad};                                   \
        cudaError_t e = cudaMemcpyToSymbolAsync(forge::g_check_bounds, &b, sizeof(b), 0, cudaMemcpyHostToDevice, stream); \
        return e == cudaSuccess ? 0 : forge::fail(FORGE_ERR_LAUNCH, "checks_configure: %s", cudaGetErrorString(e));   \
    }
#else
#define FORGE_PAGE_OK(page) (true)
#define FORGE_SLOT_OK(slot) (true)
#define FORGE_TOKEN_OK(t) (true)
#define FORGE_DEFINE_CHECKS_ENTRY(name)                                                                              \
    extern "C" int forge_checks_configure_##name(int, int, int, int*, int*, cudaStream_t) {                          \
        return forge::fail(FORGE_ERR_UNSUPPORTED, "this library was built without FORGE_CHECKS");                   \
    }
#endif
#endif
