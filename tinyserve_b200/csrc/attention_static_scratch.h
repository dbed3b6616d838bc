// Paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in priyammaz/tinyserve; it is an addition of this
// library.  Some hosts of a kernel library may not call cudaMalloc at all: code that runs
// inside a region where the allocator is frozen (a memory pool that was sized once and handed
// over, a real-time loop that must not take the driver's allocation lock, a plug-in that is
// given buffers for its inputs and outputs and nothing else).  The split-KV form of paged
// attention needs scratch beyond its inputs and outputs (the partial outputs of every key
// range and their softmax statistics).  ts_paged_attention takes that scratch from the caller;
// ts_paged_attention_static_scratch takes it from a fixed array that is part of the library
// image, so that the caller passes inputs and outputs only.
//
// Limits and rules:
//  * The array holds TS_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on which a process
//    loads this library keeps that much memory until the process ends.  A call with more
//    than one key range needs num_tokens * H * num_splits * (head size + 2) floats; a larger
//    call is refused with an error message and nothing is launched.  A call with num_splits
//    == 1 keeps nothing in the array and is never refused for its size.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and keeps it.  Make that first call before any stream capture begins.
//  * The function calls no cudaMalloc, cudaFree or other allocating routine.
//  * All calls share the one array, and it keeps what the last call left.  For every query
//    row that belongs to a request the kernels write each element before they read it, so
//    nothing has to start at zero and nothing is cleared.  (Rows of q past cu_q[num_requests],
//    padding, are combined from stale values; only their own output rows are affected, as with
//    ts_paged_attention and uninitialised caller scratch.)  Two calls that overlap on the GPU
//    (different streams, or graphs replayed side by side) race on the array: order them.
//
// Arguments are those of ts_paged_attention without part_o and part_ml.  Returns 0, or 1 with
// the message in ts_last_error().
#pragma once

#include <cuda_runtime.h>

#define TS_STATIC_SCRATCH_FLOATS (1 << 20)

extern "C" int ts_paged_attention_static_scratch(
    int dtype, const void* q, void* out, const void* k_cache, const void* v_cache,
    const int* block_table, const int* cu_q, const int* kv_lens, int num_tokens, int num_requests,
    int max_q_len, int H, int Hkv, int page_size, int max_blocks, float scale, int window,
    int num_splits, cudaStream_t stream);
