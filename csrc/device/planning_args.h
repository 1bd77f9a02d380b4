// Argument block of the planning kernel and the kernel's declaration, shared by its launchers.
#pragma once
#include <stdint.h>
#include "../mep_types.h"

namespace mep {

struct PlanArgs {
  const int32_t* topk;        // [N]
  const int32_t* tpe;         // [E]
  int32_t* dst;               // [N]
  int32_t* cu_seqlens;        // [2epn]
  int32_t* experts_to_copy;   // [R, epn]
  int32_t* zero_fill;         // [2epn, 2]
  int32_t* remote_stats;      // [2]
  uint32_t epoch;             // non-zero selects the barrier-free fast path where the geometry allows it (the launch
                              // epoch itself is kept in device memory, see planning_fast_kernel)
  int32_t pad;
};
struct PlanArgsPack { PlanArgs a[MEP_MAX_VRANKS]; };

constexpr int kPlanThreads = 1024;
constexpr int kSmemECap = 8192;   // per-expert scratch lives in shared memory up to this E

__global__ void planning_kernel(MepCtxPack P, PlanArgsPack A);
__global__ void planning_fast_kernel(MepCtxPack P, PlanArgsPack A);

// The fast path keeps every lookup table in shared memory (one private copy per CTA).
constexpr int kFastMaxE = 2048;
constexpr int kFastMaxER = 8192;
constexpr int kFastTableE = 512;   // up to this E the stable ranking uses a [32 warps, E] table

}  // namespace mep
