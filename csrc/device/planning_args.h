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
};
struct PlanArgsPack { PlanArgs a[MEP_MAX_VRANKS]; };

constexpr int kPlanThreads = 1024;
constexpr int kSmemECap = 8192;   // per-expert scratch lives in shared memory up to this E

__global__ void planning_kernel(MepCtxPack P, PlanArgsPack A);

}  // namespace mep
