// prefetch_weight: owner-push of redundant experts' weights into the peers' prefetch slots.
//
// Counterpart of the reference's PrefetchKernel (moonep/prefetch.py:45-470): one launch
// copies up to six tensors (gate/up/down and optionally their block scales) of every local
// expert that the plan placed in some rank's slot (experts_to_copy[d, b] in this rank's id
// range) to pool[d, b]. Expert payloads are contiguous, so the copy is 1-D: 16 KB pieces are
// dealt round-robin to the copy warps of all CTAs; one thread per warp runs a ring of shared-memory
// slots, filling each with an untiled bulk copy from local memory and draining it with an untiled
// bulk store to the holder's slot (no multicast, no tensor map). Dtype-agnostic (bytes).
// Ends with a cross-rank barrier: on return every rank's slots are complete.
// Per-slot flags on top of that (the reference only has the trailing barrier, moonep/prefetch.py:467-470):
// the CTA that finishes the last share of a slot release-stores the launch's prefetch epoch into the
// holder's flag word for that slot, so a consumer on the holder (the grouped GEMM, group epn + b) can start
// on a prefetched expert as soon as that expert has landed instead of waiting for the whole launch.
#include "prims.cuh"
#include "../host/launch.h"

namespace mep {

struct CopyTensor {
  const char* local;          // [epn, expert_bytes]
  char* pool;                 // rank 0's slot 0; slot (d, b) = pool + d*rank_stride + b*expert_bytes
  int64_t expert_bytes;
  int64_t rank_stride;
};
struct PrefetchArgs {
  const int32_t* etc;         // plan.experts_to_copy [R, epn]
  int32_t ntensors;
  int32_t pad;
  CopyTensor t[6];
};
struct PrefetchArgsPack { PrefetchArgs a[MEP_MAX_VRANKS]; };

constexpr int kPfWarps = 6;                 // copy warps per CTA (two 16 KB slots each at the usual sizes)
constexpr int kCopyThreads = kPfWarps * 32;
constexpr int64_t kChunk = 16384;           // bytes per piece (one shared-memory slot)
constexpr int kPfMaxStages = 4;

__global__ void __launch_bounds__(kCopyThreads, 1) prefetch_kernel(MepCtxPack P, PrefetchArgsPack A, int stages, int list_bytes) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const PrefetchArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) unsigned char pf_smem[];
  int* s_list = reinterpret_cast<int*>(pf_smem);
  unsigned char* slots = pf_smem + list_bytes;
  __shared__ int s_n;
  __shared__ __align__(8) uint64_t s_bar[kPfWarps * kPfMaxStages];
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = c.R, epn = c.epn, lo = c.rank * epn;
  const uint32_t ep = c.pf_epoch ? *(volatile uint32_t*)c.pf_epoch : 0u;
  if (tid < kPfWarps * kPfMaxStages) mbar_init(&s_bar[tid], 1);
  fence_mbar_init();

  // Slot list in ascending (rank, slot) order. Every CTA must build the IDENTICAL list, because
  // work unit u is mapped to list entry u / chunks_per_slot on whichever warp owns u: one warp
  // compacts with ballots (no atomics, whose arrival order could differ between CTAs).
  if (tid < 32) {
    int n = 0;
    for (int i0 = 0; i0 < R * epn; i0 += 32) {
      const int i = i0 + tid;
      bool has = false;
      if (i < R * epn) { const int e = a.etc[i]; has = e >= lo && e < lo + epn && i / epn != c.rank; }
      const unsigned bal = __ballot_sync(0xffffffffu, has);
      if (has) s_list[n + __popc(bal & lanemask_lt())] = i;
      n += __popc(bal);
    }
    if (tid == 0) s_n = n;
  }
  __syncthreads();
  const int nslots = s_n;
  if (tid == 0) trace_mark(c, MEP_K_PREFETCH, 1);

  int64_t chunks_per_slot = 0;
  for (int t = 0; t < a.ntensors; ++t) chunks_per_slot += (a.t[t].expert_bytes + kChunk - 1) / kChunk;
  const int64_t total = (int64_t)nslots * chunks_per_slot;
  if (lane == 0) {
    // One thread per warp drives the warp's pipeline. Pieces of one slot are consecutive work units, so
    // the warp has finished its share of a slot when its next unit belongs to another one: only then it
    // waits for its stores to complete, makes them visible and adds its count to the slot's counter;
    // whoever completes the count publishes the slot's flag on the holder.
    unsigned char* ring = slots + (size_t)warp * stages * kChunk;
    uint64_t* bars = s_bar + warp * kPfMaxStages;
    const int64_t gw = (int64_t)blockIdx.x * kPfWarps + warp, nw = (int64_t)nb * kPfWarps;
    const int64_t n = gw < total ? (total - gw + nw - 1) / nw : 0;
    struct Piece { const char* src; char* dst; uint32_t len; int si; };
    auto piece = [&](int64_t j) {
      const int64_t u = gw + j * nw;
      const int si = (int)(u / chunks_per_slot);
      int64_t ck = u - (int64_t)si * chunks_per_slot;
      int t = 0;
      for (;; ++t) { const int64_t m = (a.t[t].expert_bytes + kChunk - 1) / kChunk; if (ck < m) break; ck -= m; }
      const CopyTensor& T = a.t[t];
      const int idx = s_list[si], d = idx / epn, b = idx - d * epn, le = a.etc[idx] - lo;
      const int64_t beg = ck * kChunk;
      const int64_t len = (T.expert_bytes - beg) < kChunk ? (T.expert_bytes - beg) : kChunk;
      return Piece{T.local + (int64_t)le * T.expert_bytes + beg, T.pool + (int64_t)d * T.rank_stride + (int64_t)b * T.expert_bytes + beg,
                   (uint32_t)len, si};
    };
    auto load = [&](int64_t j) {
      const Piece p = piece(j); const int st = (int)(j % stages);
      mbar_expect_tx(&bars[st], p.len);
      bulk_g2s(ring + (size_t)st * kChunk, p.src, p.len, &bars[st]);
    };
    int cur_si = -1, cur_cnt = 0;
    auto finish_slot = [&]() {
      if (cur_si < 0 || !c.slot_done) return;
      bulk_wait_all<0>(); fence_proxy_async();
      const int idx = s_list[cur_si], d = idx / epn, b = idx - d * epn;
      __threadfence_system();
      if (atomicAdd(c.slot_done + idx, (uint32_t)cur_cnt) + (uint32_t)cur_cnt == (uint32_t)chunks_per_slot) {
        c.slot_done[idx] = 0u;
        __threadfence();
        st_release_sys((uint32_t*)peer_ptr(c, d, c.off_slotflag) + b, ep);
      }
    };
    const int pre = stages - 1;
    for (int64_t i = 0; i < pre && i < n; ++i) load(i);
    for (int64_t j = 0; j < n; ++j) {
      const Piece p = piece(j);
      if (p.si != cur_si) { finish_slot(); cur_si = p.si; cur_cnt = 0; }
      ++cur_cnt;
      if (j + pre < n) { bulk_wait_read<0>(); load(j + pre); }       // that slot's previous store has left it
      const int st = (int)(j % stages);
      if (!mbar_wait_bounded(&bars[st], (uint32_t)(j / stages) & 1u, c.wait_budget_ns)) {
        report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_PREFETCH, 20, (int)j, 0, 0); break;
      }
      bulk_s2g(p.dst, ring + (size_t)st * kChunk, p.len);
      bulk_commit();
    }
    finish_slot();
    bulk_wait_all<0>(); fence_proxy_async();
    trace_mark(c, MEP_K_PREFETCH, 2);
  }
  cross_rank_barrier(c, nb, kWeightLaneRow, MEP_K_PREFETCH, 10);
  if (tid == 0) trace_mark(c, MEP_K_PREFETCH, 3);
}

}  // namespace mep

// One thread: a prefetch is about to be issued (see MepRankCtx.pf_epoch).
namespace mep {
__global__ void pf_epoch_bump_kernel(MepCtxPack P) {
  const MepRankCtx* c = P.ctx[blockIdx.y];
  if (threadIdx.x == 0 && c->pf_epoch) c->pf_epoch[0] += 1u;
}
}  // namespace mep

extern "C" int mep_launch_pf_epoch_bump(int nv, const MepRankCtx* const* ctxs, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "pf_epoch_bump: nv=%d out of range", nv);
  MepCtxPack P = {};
  for (int i = 0; i < nv; ++i) P.ctx[i] = ctxs[i];
  return mep::launch_plain(mep::pf_epoch_bump_kernel, dim3(1, nv), dim3(32), 0, stream, P);
}

extern "C" int mep_launch_prefetch(int nv, const MepRankCtx* const* ctxs, const mep::PrefetchArgs* args,
                                   int num_sms, int R, int epn, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "prefetch: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::PrefetchArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  const size_t list_bytes = (((size_t)R * epn * sizeof(int)) + 127) & ~(size_t)127;
  MEP_REQUIRE(list_bytes <= 96 * 1024, "prefetch: R*epn=%d exceeds the slot-list capacity", R * epn);
  int stages = (int)((220 * 1024 - list_bytes) / ((size_t)mep::kPfWarps * mep::kChunk));
  if (stages > mep::kPfMaxStages) stages = mep::kPfMaxStages;
  const size_t smem = list_bytes + (size_t)mep::kPfWarps * stages * mep::kChunk;
  return mep::launch_cooperative(mep::prefetch_kernel, dim3(num_sms, nv), dim3(mep::kCopyThreads), smem,
                                 stream, false, P, A, stages, (int)list_bytes);
}

MEP_EXPORT_SIZEOF(PrefetchArgs, mep::PrefetchArgs)
