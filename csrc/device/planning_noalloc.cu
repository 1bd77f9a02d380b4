// Allocation-free variant of the planner for a single rank; see ../mep_noalloc.h for the
// contract and for who needs it. The planning kernel itself is the regular one; what changes
// is where its work space comes from: a fixed array in this file instead of tensors owned by
// a Buffer.
#include "planning_args.h"
#include "../mep_noalloc.h"
#include "../host/launch.h"
#include <mutex>
#include <string.h>

// The work space. In host code this name is only a handle for the runtime (it is NOT a device
// address); the device address is looked up once per device below and only that pointer is
// handed to the kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MEP_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
constexpr int kCtas = 8;                 // CTAs of the cooperative launch
constexpr size_t kControlBytes = 4096;   // context + barrier words + status: cleared every call

std::mutex g_mu;
unsigned char* g_base[kMaxDevices] = {};

inline size_t up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Device address of the work space on the current device (resolved on first use).
int scratch_base(unsigned char** out) {
  int dev = 0;
  MEP_CUDA_CHECK(cudaGetDevice(&dev));
  MEP_REQUIRE(dev >= 0 && dev < kMaxDevices, "noalloc: device index %d not supported", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_base[dev]) {
    void* p = nullptr;
    MEP_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    MEP_REQUIRE(p != nullptr, "noalloc: work space has no device address");
    g_base[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_base[dev];
  return 0;
}

}  // namespace

extern "C" int mep_plan_single_rank_noalloc(const int32_t* topk, const int32_t* tokens_per_expert,
                                            int S, int K, int E, int token_padding,
                                            int32_t* dst, int32_t* cu_seqlens, int32_t* zero_fill_ranges,
                                            int32_t* experts_to_copy, int32_t* remote_stats, cudaStream_t stream) {
  MEP_REQUIRE(S > 0 && K > 0 && E > 0, "noalloc: S, K, E must be positive (got %d, %d, %d)", S, K, E);
  MEP_REQUIRE(K <= MEP_MAX_TOPK, "noalloc: K=%d exceeds %d", K, MEP_MAX_TOPK);
  MEP_REQUIRE(token_padding >= 1, "noalloc: token_padding must be >= 1");
  const long long N = (long long)S * K;
  MEP_REQUIRE(N <= MEP_NOALLOC_MAX_ENTRIES, "noalloc: S*K=%lld exceeds the built-in work space (max %d entries)",
              N, MEP_NOALLOC_MAX_ENTRIES);
  MEP_REQUIRE(E <= MEP_NOALLOC_MAX_EXPERTS, "noalloc: E=%d exceeds the built-in work space (max %d experts)",
              E, MEP_NOALLOC_MAX_EXPERTS);
  MEP_REQUIRE(topk && tokens_per_expert && dst && cu_seqlens && zero_fill_ranges && experts_to_copy && remote_stats,
              "noalloc: null input or output pointer");
  const long long nvs_ll = up((size_t)N + (size_t)(token_padding - 1) * 2 * E, token_padding);
  MEP_REQUIRE(nvs_ll < (1ll << 24), "noalloc: padded slot count %lld exceeds 2^24", nvs_ll);
  // The rank context below is copied from this stack frame with an asynchronous copy: a stream
  // capture would record the frame's address and replay the copy after the frame is gone.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  MEP_CUDA_CHECK(cudaStreamIsCapturing(stream, &cap));
  MEP_REQUIRE(cap == cudaStreamCaptureStatusNone, "noalloc: the stream is being captured; this entry point only runs on a "
              "stream that executes its work directly");

  unsigned char* base = nullptr;
  if (scratch_base(&base)) return -1;

  // ---- carve the work space
  const int vb = (1024 / K) * K;
  const int nvb = (int)((N + vb - 1) / vb);
  size_t off = 0;
  auto take = [&](size_t bytes) { off = up(off, 256); size_t o = off; off += bytes; return o; };
  const size_t o_ctx = take(sizeof(MepRankCtx));
  const size_t o_status = take(sizeof(MepStatus));
  const size_t o_gridbar = take(16), o_epoch = take(16), o_sendcnt = take(8);
  const size_t o_bar = take((size_t)MEP_BAR_ROWS * MEP_MAX_RANKS * 4);
  const size_t o_dupcnt = take(8);
  MEP_REQUIRE(off <= kControlBytes, "noalloc: internal layout error");
  off = kControlBytes;
  const size_t o_hist = take((size_t)nvb * E * 4);
  const size_t o_count = take((size_t)E * 4), o_prefix = take((size_t)E * 4), o_remaining = take((size_t)E * 4);
  const size_t o_alloc = take((size_t)E * 4), o_cumsum = take((size_t)E * 4), o_expoff = take((size_t)E * 4);
  const size_t o_etc = take((size_t)E * 4), o_stats = take(8);
  const size_t o_tpe = take((size_t)E * 4);
  const size_t gcap = (size_t)N / 2 + 1, lcap = (size_t)N;
  const size_t o_dupgroups = take(gcap * 3 * 4), o_duploffs = take(lcap * 4);
  MEP_REQUIRE(off <= (size_t)MEP_NOALLOC_SCRATCH_BYTES, "noalloc: request needs %zu bytes of work space, %d available",
              off, MEP_NOALLOC_SCRATCH_BYTES);

  // ---- context of the single rank; the "symmetric heap" is the work space itself
  MepRankCtx c;
  memset(&c, 0, sizeof c);
  c.rank = 0; c.R = 1; c.S = S; c.H = 8; c.K = K; c.E = E; c.epn = E; c.N = (int)N; c.NvS = (int)nvs_ll;
  c.token_padding = token_padding; c.vblock_entries = vb; c.num_vblocks = nvb; c.num_sms = kCtas;
  c.heap_base = (char*)base; c.chunk_stride = MEP_NOALLOC_SCRATCH_BYTES;
  c.off_tpe = (int64_t)o_tpe; c.off_bar = (int64_t)o_bar; c.off_dupcnt = (int64_t)o_dupcnt;
  c.off_dupgroups = (int64_t)o_dupgroups; c.off_duploffs = (int64_t)o_duploffs;
  c.dup_group_cap = (int64_t)gcap; c.dup_loff_cap = (int64_t)lcap;
  c.grid_bar = (uint32_t*)(base + o_gridbar); c.epoch = (uint32_t*)(base + o_epoch);
  c.hist = (int32_t*)(base + o_hist); c.count = (int32_t*)(base + o_count);
  c.tpe_prefix = (int32_t*)(base + o_prefix); c.remaining = (int32_t*)(base + o_remaining);
  c.alloc = (int32_t*)(base + o_alloc); c.alloc_cumsum = (int32_t*)(base + o_cumsum);
  c.expert_off = (int32_t*)(base + o_expoff); c.etc_all = (int32_t*)(base + o_etc);
  c.stats_all = (int32_t*)(base + o_stats); c.send_cnt = (unsigned long long*)(base + o_sendcnt);
  c.status = (MepStatus*)(base + o_status);
  c.wait_budget_ns = 2000000000ull;

  // Barrier words, epochs and the status word must start at zero; everything else the kernel
  // initialises itself before reading it. The context is copied from pageable host memory,
  // which the runtime stages before returning, so `c` may live on this stack frame.
  MEP_CUDA_CHECK(cudaMemsetAsync(base, 0, kControlBytes, stream));
  MEP_CUDA_CHECK(cudaMemcpyAsync(base + o_ctx, &c, sizeof c, cudaMemcpyHostToDevice, stream));

  MepCtxPack P = {};
  P.ctx[0] = (const MepRankCtx*)(base + o_ctx);
  mep::PlanArgsPack A = {};
  A.a[0] = mep::PlanArgs{topk, tokens_per_expert, dst, cu_seqlens, experts_to_copy, zero_fill_ranges, remote_stats, 0u, 0};
  const size_t smem = (E <= mep::kSmemECap ? (size_t)E : 1) * sizeof(int);
  return mep::launch_cooperative(mep::planning_kernel, dim3(kCtas, 1), dim3(mep::kPlanThreads), smem, stream, false, P, A);
}
