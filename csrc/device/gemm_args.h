// Argument block of the grouped GEMM kernels (shared by the 1-CTA and the 2-CTA launchers).
#pragma once
#include <stdint.h>

namespace mep {

enum GemmMode { GEMM_GATE_UP = 0, GEMM_DOWN = 1, GEMM_DGRAD = 2, GEMM_DGRAD_GU = 3, GEMM_WGRAD = 4 };

struct GemmArgs {
  const int32_t* cu_seqlens;   // [G] padded end row of each group
  int32_t G;
  int32_t N;                   // output columns (GATE_UP: width of act = out dim of each weight)
  int32_t K;                   // reduction length (DGRAD_GU: 2 * inner); unused for WGRAD
  int32_t M_w;                 // WGRAD: rows of one weight matrix
  int32_t b_group_rows;        // rows one group occupies in the flattened 2-D weight tensor(s)
  int32_t accumulate;          // WGRAD: 1 -> out += acc, 0 -> out = acc
  int32_t g_begin, g_end;      // only groups in [g_begin, g_end) are computed
  int32_t zero_empty_below;    // WGRAD without accumulate: empty groups g < this get zeros
  int32_t reserved0;
  void* out;                   // bf16 [rows, ldo]; WGRAD: fp32 [G, M_w, N]
  void* out2;                  // GATE_UP: optional bf16 [rows, 2N] pre-activations (gate | up)
  const float* row_scale;      // GATE_UP / DOWN: optional per-row factor [rows]
  int64_t ldo;
  int32_t* status;             // [4] error word: code, site, block, tile
  uint64_t budget_ns;
  uint32_t* sched;             // [2] zero-initialised ticket counter of the dynamic tile scheduler, or null for
                               // the static strided tile order
  // DOWN / DGRAD / DGRAD_GU, optional "push" epilogue: row r of the output is not stored to `out` but sent
  // to the rank it came from: push_info[r] = src_rank * push_rows + index (or < 0 for a padding row) and the
  // row lands at push_base + src_rank * push_stride + index * N * 2 (row `index` of that rank's [push_rows, N]
  // bf16 receive area inside the symmetric heap). push_wsrc[r], if given, goes to the float at
  // push_wbase + src_rank * push_stride + index * 4.
  const int32_t* push_info;
  unsigned char* push_base;
  unsigned char* push_wbase;
  const float* push_wsrc;
  uint64_t push_stride;
  // GATE_UP / DGRAD, optional: the rows of `a` are produced by a flagged dispatch that is still running.
  // tile_done[t] holds the flag epoch at which rows [128 t, 128 t + 128) became complete; the TMA producer waits
  // (bounded) for tile_done[t] >= *tile_epoch before it loads rows of tile t. The launch must leave the dispatch
  // kernel's SMs free (num_ctas <= SMs - its CTAs), since that kernel has to be resident meanwhile.
  const uint32_t* tile_done;
  const uint32_t* tile_epoch;
  int32_t* status_host;        // optional host-mapped copy of status[0]
  // optional: the weights of groups g >= group_first are still being written by a prefetch. group_flags[g -
  // group_first] holds the prefetch epoch at which that slot became complete; the TMA producer waits (bounded)
  // for it to reach *group_epoch before it loads weights of such a group.
  const uint32_t* group_flags;
  const uint32_t* group_epoch;
  int32_t push_rows;
  int32_t push_ranks;
  int32_t group_first;
  int32_t sched_ctas;          // dynamic order: CTAs over ALL launches that draw from `sched` (several launches of
                               // one GEMM may share a counter); 0 = just this launch
  // WGRAD (CTA-pair kernel), optional optimizer in the epilogue: for a group g with upd_mask[g] != 0 the
  // gradient tile is not written to `out`; the bf16 weights upd_w[g] (same [G, M_w, N] layout) are updated in
  // place instead, w -= upd_lr * dW, with the arithmetic of the stand-alone SGD kernel. Groups with
  // upd_mask[g] == 0 (e.g. experts whose gradient still has to be reduced across ranks) are written as usual.
  void* upd_w;
  const int32_t* upd_mask;
  float upd_lr;
  int32_t reserved1;
};

}  // namespace mep
