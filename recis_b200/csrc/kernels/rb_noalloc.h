// Allocation-free entry point of the id dedup + owner bucketing step.
//
// This function has no counterpart in the reference project; it exists for callers of this library that are not allowed to
// allocate device memory at the moment they need the operation:
//   * code running inside a region where cudaMalloc is off limits (a stream being captured into a CUDA graph, a real-time
//     serving loop with a no-allocation rule on its latency path),
//   * plain C / C++ hosts that link the shared object directly and have no tensor framework (and therefore no caching
//     allocator) to borrow scratch buffers from.
// The regular entry point (rb_dedup_partition in rb_kernels.h) takes its scratch (hash-set keys, hash-set positions and one
// slot index per id) from the caller. Here the scratch is a fixed array compiled into the library: every GPU that loads the
// library carries it (about 7.3 MB) until the process exits.
//
// Contract
//   * All pointers are device pointers owned by the caller: ids [n] in; counts [world], offsets [world + 1],
//     unique_ids [n], reverse [n] out. Results are the same as rb_dedup_partition's: unique ids bucketed by owner rank (the
//     order inside a bucket is not specified), reverse[i] = position of ids[i] in unique_ids, offsets[world] = unique count.
//   * n may be at most RB_NOALLOC_MAX_IDS; a larger n is rejected with return code 2 and a message in `err`.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine; it enqueues two memsets and two kernels
//     on `stream` and returns without synchronising.
//   * The first call on a device looks up the device address of the built-in scratch array (cudaGetSymbolAddress, with that
//     device current). Make that first call outside of any stream capture; later calls only reuse the cached address.
//     The cache is keyed by the device ordinal and assumes that the device's primary context lives as long as the process:
//     after a cudaDeviceReset the cached address is stale and this entry point must not be used again in that process.
//   * Every call uses the same scratch array, which still holds the previous call's contents on entry; the function resets
//     what has to start empty. Two calls that can overlap on the GPU (different streams, or different host threads without
//     ordering between their streams) race on that array: keep calls on one stream or order them with events.
// Return value: 0 on success; 1 bad arguments, 2 n above the limit, 3 no usable current device, 4 symbol lookup failed,
// 5 a memset could not be enqueued, 6 a kernel launch failed. `err` (optional, `err_len` bytes) receives a human-readable message on failure.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#define RB_NOALLOC_MAX_IDS (1 << 18)   /* 262144 ids per call */

#ifdef __cplusplus
extern "C" {
#endif

int rb_dedup_partition_noalloc(const int64_t* ids, int64_t n, int world, int32_t* counts, int32_t* offsets, int64_t* unique_ids,
                               int32_t* reverse, cudaStream_t stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
