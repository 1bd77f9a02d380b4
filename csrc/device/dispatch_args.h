// Argument block and tuning constants shared by the dispatch kernels (dispatch.cu: token-ordered
// sender with an exit barrier; dispatch_flagged.cu: slot-ordered sender with per-tile ready flags).
#pragma once
#include <stdint.h>
#include <cuda_bf16.h>
#include "../mep_types.h"

namespace mep {

struct DispatchArgs {
  const __nv_bfloat16* hidden;   // [S, H] local tokens
  const float* weights;          // [S, K] or null
  const int32_t* dst;            // [N] plan
  const int32_t* zero_fill;      // [2epn, 2] plan
  int32_t fresh;                 // non-zero: publish duplicate-table counts to the peers. 1 / 2: the planner used
                                 // send_cnt half 0 / 1; 3: the half the fast planner's device-side epoch names
  int32_t entry_barrier;         // 1: cross-rank barrier before the first remote write
  int64_t srcinfo_off;           // 0, or byte offset (inside a rank's chunk) of the provenance table [NvS] int32: the
                                 // sender writes src_rank * S*K + s*K + k for each of a token's K slots and -1 for
                                 // padding rows, so that a GEMM epilogue can send a row straight back to its source
  // flagged dispatch only (see dispatch_flagged.cu)
  const int32_t* send_list;      // [N] plan: entries (s*K + k) whose row is sent, in send order
  const int32_t* send_meta;      // [4] plan: number of entries in send_list, end of the used part of the shard
                                 // (cu_seqlens[2epn-1]), two spare words
};
struct DispatchArgsPack { DispatchArgs a[MEP_MAX_VRANKS]; };

constexpr int kSendWarps = 6;                 // sender warps per CTA
constexpr int kDispThreads = (kSendWarps + 1) * 32;   // + one zero-fill warp
constexpr int kMaxStages = 8;
constexpr int kMetaTokens = 32;   // tokens per warp whose plan entries / weights are staged at once


}  // namespace mep
