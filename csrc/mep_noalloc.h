// Allocation-free planning entry point.
//
// This entry point has no counterpart in the reference library. It exists for hosts that
// are not allowed to allocate device memory at the moment they need a plan: code running
// inside a memory-pool callback or under a framework that forbids allocator re-entry,
// real-time loops that must not risk the implicit device synchronisation cudaMalloc/cudaFree
// perform, and processes whose memory budget was fixed at start-up. The regular planner takes
// its work space (histograms, per-expert tables, barrier words, duplicate-group staging) from
// tensors the Buffer allocated; here the same planning kernel runs on work space carved out of
// a fixed array that lives inside the library image.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Hard limits of the built-in work space (requests beyond them are rejected, nothing runs).
#define MEP_NOALLOC_MAX_ENTRIES 65536   // S * K
#define MEP_NOALLOC_MAX_EXPERTS 1024    // E
// Size of the built-in work space. Every GPU that loads this library holds this much device
// memory from load until the process exits, whether or not the entry point is ever called.
#define MEP_NOALLOC_SCRATCH_BYTES (1280 * 1024)

// Plan the dispatch of one rank that owns all E experts (an EP group of size 1): computes the
// slot of every (token, k) entry in expert-grouped order and the padded group boundaries --
// the same five outputs Buffer.dispatch's planner produces for R = 1.
//
//   topk              [S*K] int32, expert id of every entry (device memory, input)
//   tokens_per_expert [E]   int32, histogram of topk          (device memory, input)
//   dst               [S*K] int32 out: slot of entry i; later entries of the same token are
//                                      encoded as -(slot) - 1 (duplicates on the same rank)
//   cu_seqlens        [2*E] int32 out: padded end row of each group (second half repeats the
//                                      last boundary: a single rank has no prefetch slots)
//   zero_fill_ranges  [2*E, 2] int32 out: (first padding row, padding rows) per group
//   experts_to_copy   [E]   int32 out: all -1
//   remote_stats      [2]   int32 out: zeros
//
// Rules
//  * Calls nothing that allocates: no cudaMalloc/cudaFree, no library allocator. The launch is
//    asynchronous on `stream`; outputs are valid once the stream reaches that point.
//  * The FIRST call on each device resolves the device address of the work space (one
//    cudaGetSymbolAddress with that device current).
//  * A call on a stream that is being captured is rejected (returns -1, nothing is recorded):
//    the rank context travels to the device in an asynchronous copy from the caller's stack,
//    which a captured graph would replay from a dead frame. Call it on a stream that executes
//    its work directly.
//  * All calls on a device share the one work space, which keeps the previous call's contents;
//    the entry point clears the words that must start at zero itself. Two calls whose kernels
//    can overlap on the GPU (different streams, no ordering) race on it: serialise them.
//  * Returns 0 on success, -1 on a rejected request or a CUDA error (text: mep_last_error()).
//    S*K > MEP_NOALLOC_MAX_ENTRIES, E > MEP_NOALLOC_MAX_EXPERTS, K > 32 or token_padding < 1
//    are rejected before anything is launched.
int mep_plan_single_rank_noalloc(const int32_t* topk, const int32_t* tokens_per_expert,
                                 int S, int K, int E, int token_padding,
                                 int32_t* dst, int32_t* cu_seqlens, int32_t* zero_fill_ranges,
                                 int32_t* experts_to_copy, int32_t* remote_stats, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
