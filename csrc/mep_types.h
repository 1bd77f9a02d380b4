// Plain-C structs shared by the host launchers, the device kernels and the
// Python ctypes layer (moonep_b200/_native.py mirrors them field by field).
#pragma once
#include <stdint.h>

#define MEP_MAX_RANKS 128   // rank ids fit 7 bits (reference: moonep/constants.py:7)
#define MEP_MAX_VRANKS 8    // ranks one launch may host on a single GPU (emulation)
#define MEP_MAX_TOPK 32
#define MEP_BAR_ROWS 4      // independent cross-rank flag rows per Buffer
#define MEP_FLAG_ROWS 128   // rows per ready-flag tile (= the grouped GEMM's M tile)

// Slots of the optional per-Buffer counter block (MepRankCtx.counters, unsigned 64-bit each):
// accumulated by the kernels with relaxed atomics, read by Buffer.stats().
enum MepCounter {
  MEP_CNT_DISPATCHES = 0,       // dispatch launches
  MEP_CNT_ROWS_SENT = 1,        // token rows stored to any rank's shard
  MEP_CNT_ROWS_REMOTE = 2,      // ... of which to another rank
  MEP_CNT_PAD_ROWS = 3,         // padding rows cleared
  MEP_CNT_BARRIER_WAIT_NS = 4,  // time CTA 0 spent waiting in cross-rank barriers
  MEP_CNT_BARRIERS = 5,         // cross-rank barriers executed
  MEP_CNT_COMBINES = 6,         // combine launches
  MEP_CNT_ROWS_PULLED = 7,      // rows read by combine (local and remote)
  MEP_CNT_DUP_ROWS = 8,         // duplicate rows expanded by a flagged dispatch
  MEP_CNT_PEER_ROWS = 16,       // [16 + d]: rows sent to rank d (first 48 ranks)
  MEP_CNT_SLOTS = 64,
};

// Error codes written to MepStatus.code by device code; 0 means "no error".
enum MepError {
  MEP_OK = 0,
  MEP_ERR_GRID_SYNC_TIMEOUT = 1,   // a CTA of this rank never arrived
  MEP_ERR_PEER_TIMEOUT = 2,        // a peer rank never arrived at a cross-rank barrier
  MEP_ERR_BOUNDS = 3,              // checked build: computed index out of range
  MEP_ERR_FLAG_TIMEOUT = 4,        // a ready flag never reached its expected value
  MEP_ERR_MBAR_TIMEOUT = 5,        // an mbarrier phase never completed
};

enum MepKernelId {
  MEP_K_SYNC = 1, MEP_K_PLANNING = 2, MEP_K_DISPATCH = 3, MEP_K_EXPAND = 4,
  MEP_K_DUP_REDUCE = 5, MEP_K_COMBINE = 6, MEP_K_PREFETCH = 7, MEP_K_GRAD_REDUCE = 8,
  MEP_K_GEMM = 9, MEP_K_WAIT_PROBE = 10,
};

// First failure recorded by any kernel of a Buffer. Lives in device memory; the host
// copies it back lazily. All-zero == healthy.
typedef struct MepStatus {
  int32_t code;       // MepError
  int32_t kernel;     // MepKernelId
  int32_t site;       // which wait inside the kernel
  int32_t rank;
  int32_t peer;       // peer rank (cross-rank barrier) or CTA index (grid sync)
  uint32_t observed;
  uint32_t expected;
  int32_t reserved;
} MepStatus;

// Per-rank constant context. One instance per rank in device memory, written once
// when the Buffer is created.
typedef struct MepRankCtx {
  int32_t rank, R, S, H, K, E, epn, N, NvS, token_padding;
  int32_t vblock_entries, num_vblocks, num_sms, checked;
  // symmetric heap: rank r's chunk is heap_base + r * chunk_stride (all ranks mapped)
  char* heap_base;
  int64_t chunk_stride;
  int64_t off_hidden, off_weights, off_tpe, off_bar, off_dupcnt, off_dupgroups,
      off_duploffs, off_ready;
  int64_t dup_group_cap, dup_loff_cap;   // per-source capacity of the staging tables
  // local scratch (ordinary device memory)
  uint32_t* grid_bar;      // [2] software grid barrier words: [0] token kernels, [1] weight-pool kernels
  uint32_t* epoch;         // [MEP_BAR_ROWS] cross-rank barrier epochs
  int32_t* hist;           // [num_vblocks, E]
  int32_t* count;          // [E]   tokens per expert over the whole group
  int32_t* tpe_prefix;     // [E]   tokens of expert e on ranks < rank
  int32_t* remaining;      // [E]
  int32_t* alloc;          // [E, R]
  int32_t* alloc_cumsum;   // [E, R]
  int32_t* expert_off;     // [R, E]
  int32_t* etc_all;        // [R, epn] experts_to_copy of every rank
  int32_t* stats_all;      // [R, 2]
  unsigned long long* send_cnt;  // [R] (groups<<32 | loffs) emitted to each destination
  MepStatus* status;
  uint64_t wait_budget_ns;
  // optional device-timestamp ring (null = tracing off): word 0 = number of records written,
  // then 2 words per record: %globaltimer ns, (kernel << 48 | site << 32 | cta << 8 | warp)
  unsigned long long* trace;
  int64_t trace_cap;
  // NVSwitch multicast alias of one chunk (null = not available): a multimem store to
  // mc_base + off lands at offset off of EVERY rank's chunk
  char* mc_base;
  // fast planner: flag per 1024-entry block, set to the launch epoch once its histogram is published
  uint32_t* vb_flags;
  // host-visible copy of status.code (pinned host memory mapped into the device, or null): the
  // first failure is written to both, so the host can test for a failure without synchronising
  int32_t* status_host;
  // tile-ready flags (dispatch -> consumer GEMM), see dispatch_flagged_kernel. A tile is
  // MEP_FLAG_ROWS consecutive slots of a rank's shard.
  //   heap, off_ready:  uint32 [ntiles] arrivals; every flagged dispatch adds exactly one arrival per
  //                     slot of the tile (row landed / duplicate registered / padding cleared / unused)
  //   heap, off_rowsrc: int32 [NvS] slot a row's payload comes from (itself, the row it duplicates,
  //                     or -1 for a padding row)
  int64_t off_rowsrc;
  uint32_t* tile_done;     // local [ntiles]: flag epoch at which the tile became complete (all rows
                           // landed, duplicates expanded); consumers wait for tile_done[t] >= epoch
  uint32_t* flag_epoch;    // local: [0] flagged dispatches issued so far (advanced by flag_epoch_bump in
                           // stream order before the dispatch and its consumers), [1] expander ticket
  int32_t ntiles;          // ceil(NvS / MEP_FLAG_ROWS)
  int32_t reserved1;
  // per-op counters (null = off), see MepCounters
  unsigned long long* counters;
  // per-slot prefetch flags (prefetch -> consumer GEMM), see prefetch_kernel
  //   heap, off_slotflag: uint32 [epn]: prefetch epoch at which slot b of this rank last became complete
  int64_t off_slotflag;
  uint32_t* slot_done;     // local [R * epn]: chunks of slot (d, b) this rank has finished copying (self-resetting)
  uint32_t* pf_epoch;      // local [1]: prefetch launches issued so far (advanced by pf_epoch_bump in stream order
                           // before the prefetch kernel and before every consumer of its slot flags)
} MepRankCtx;

typedef struct MepCtxPack { const MepRankCtx* ctx[MEP_MAX_VRANKS]; } MepCtxPack;
