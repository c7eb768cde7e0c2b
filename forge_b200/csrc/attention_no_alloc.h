// forge_paged_attention_mma_static: the sliced-keys attention without any allocation by anyone.
//
// This entry point has no counterpart in the reference (Cyxuan0311/Forge allocates a fresh device buffer
// for every operator output).  It exists for callers that are not allowed to allocate device memory at
// the moment they need attention: code running inside a CUDA stream capture, a real-time loop that must
// not take the allocator's lock, a host process that was handed device pointers by another runtime and
// owns no allocator at all.  forge_paged_attention_mma() asks such a caller for two scratch buffers that
// hold the per-slice partial results; here that scratch is a fixed array inside the library itself.
//
// What the caller should know:
//  * The scratch is a file-scope device array of FORGE_ATT_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU
//    on which the library is used keeps that array until the process exits.
//  * A call with num_splits > 1 needs  tiles * NKV * num_splits * R * (head_dim + 2)  floats, R = 16 if
//    max_rows <= 16 else 64.  If that exceeds the array the call is refused with FORGE_ERR_UNSUPPORTED and a
//    message; nothing runs.  A call with num_splits == 1 uses no scratch and is never refused for its size.
//  * The first call on each device that needs the scratch looks up the array's address on that device, and
//    the first call of either kind on each device sets the kernels' shared-memory limit there (both are kept
//    per device).  Make those first calls outside of any stream capture, with the device current that the
//    pointers belong to.  Later calls only launch kernels.
//  * All calls share the one array, and it keeps what the last call left in it.  Nothing in it has to start
//    at zero: every slice writes its whole partial result before the merge reads it.  But two calls that
//    overlap on the GPU (different streams, or graphs replayed concurrently) race on it; serialise them.
//  * Inputs and outputs are the caller's, exactly as for forge_paged_attention_mma(); no cudaMalloc,
//    cudaFree or other allocating routine is called here.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FORGE_ATT_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int forge_paged_attention_mma_static(const void* q, const void* kv, void* out, const int32_t* block_table,
                                     const int32_t* tile_req, const int32_t* tile_row0, const int32_t* q_start,
                                     const int32_t* ctx_before, int num_tiles, int max_rows, int NH, int NKV,
                                     int head_dim, int page_size, int max_pages, int window, int num_splits,
                                     float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
