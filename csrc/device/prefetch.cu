// prefetch_weight: owner-push of redundant experts' weights into the peers' prefetch slots.
//
// Counterpart of the reference's PrefetchKernel (moonep/prefetch.py:45-470): one launch
// copies up to six tensors (gate/up/down and optionally their block scales) of every local
// expert that the plan placed in some rank's slot (experts_to_copy[d, b] in this rank's id
// range) to pool[d, b]. Expert payloads are contiguous, so the copy is 1-D: 64 KB chunks are
// dealt round-robin to the CTAs and moved with 16-byte local loads and 16-byte peer stores
// (eight per thread in flight) -- no TMA touches peer memory. Dtype-agnostic (bytes).
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

constexpr int kCopyThreads = 512;
constexpr int64_t kChunk = 65536;
constexpr int kVec = 8;               // 16-byte vectors per thread in flight

__global__ void __launch_bounds__(kCopyThreads, 1) prefetch_kernel(MepCtxPack P, PrefetchArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const PrefetchArgs& a = A.a[blockIdx.y];
  extern __shared__ int s_list[];
  __shared__ int s_n;
  const int nb = gridDim.x, tid = threadIdx.x, nt = blockDim.x;
  const int R = c.R, epn = c.epn, lo = c.rank * epn;
  const uint32_t ep = c.pf_epoch ? *(volatile uint32_t*)c.pf_epoch : 0u;

  // Slot list in ascending (rank, slot) order. Every CTA must build the IDENTICAL list, because
  // work unit u is mapped to list entry u / chunks_per_slot on whichever CTA owns u: one warp
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

  int64_t chunks_per_slot = 0;
  for (int t = 0; t < a.ntensors; ++t) chunks_per_slot += (a.t[t].expert_bytes + kChunk - 1) / kChunk;
  const int64_t total = (int64_t)nslots * chunks_per_slot;
  // Slot flags: chunks of one slot are consecutive work units, so a CTA finishes its share of slot `si`
  // when its next unit belongs to another slot. Only then -- once per slot and CTA, not per chunk, so the
  // stores of consecutive chunks stay in flight together -- it makes its stores visible, adds its chunk
  // count to the slot's counter, and whoever completes the count publishes the flag on the holder.
  int cur_si = -1, cur_cnt = 0;
  auto finish_slot = [&]() {
    if (cur_si < 0 || !c.slot_done) return;
    __syncthreads();
    if (tid == 0) {
      const int idx = s_list[cur_si], d = idx / epn, b = idx - d * epn;
      __threadfence_system();
      if (atomicAdd(c.slot_done + idx, (uint32_t)cur_cnt) + (uint32_t)cur_cnt == (uint32_t)chunks_per_slot) {
        c.slot_done[idx] = 0u;
        __threadfence();
        st_release_sys((uint32_t*)peer_ptr(c, d, c.off_slotflag) + b, ep);
      }
    }
  };
  for (int64_t u = blockIdx.x; u < total; u += nb) {
    const int si = (int)(u / chunks_per_slot);
    if (si != cur_si) { finish_slot(); cur_si = si; cur_cnt = 0; }
    ++cur_cnt;
    int64_t ck = u - (int64_t)si * chunks_per_slot;
    int t = 0;
    for (;; ++t) { const int64_t n = (a.t[t].expert_bytes + kChunk - 1) / kChunk; if (ck < n) break; ck -= n; }
    const CopyTensor& T = a.t[t];
    const int idx = s_list[si], d = idx / epn, b = idx - d * epn, le = a.etc[idx] - lo;
    const int64_t beg = ck * kChunk;
    const int64_t len = (T.expert_bytes - beg) < kChunk ? (T.expert_bytes - beg) : kChunk;
    const char* src = T.local + (int64_t)le * T.expert_bytes + beg;
    char* dstp = T.pool + (int64_t)d * T.rank_stride + (int64_t)b * T.expert_bytes + beg;
    const int nvec = (int)(len >> 4);
    for (int v0 = 0; v0 < nvec; v0 += kVec * nt) {
      int4 x[kVec];
#pragma unroll
      for (int j = 0; j < kVec; ++j) { const int v = v0 + j * nt + tid; if (v < nvec) x[j] = ld_nc_v4(src + (size_t)v * 16); }
#pragma unroll
      for (int j = 0; j < kVec; ++j) { const int v = v0 + j * nt + tid; if (v < nvec) st_na_v4(dstp + (size_t)v * 16, x[j]); }
    }
    for (int64_t i = ((int64_t)nvec << 4) + tid; i < len; i += nt) dstp[i] = src[i];   // ragged tail
  }
  finish_slot();
  cross_rank_barrier(c, nb, 1, MEP_K_PREFETCH, 10);
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
  const size_t smem = (size_t)R * epn * sizeof(int);
  MEP_REQUIRE(smem <= 160 * 1024, "prefetch: R*epn=%d exceeds the slot-list capacity", R * epn);
  return mep::launch_cooperative(mep::prefetch_kernel, dim3(num_sms, nv), dim3(mep::kCopyThreads), smem,
                                 stream, false, P, A);
}

MEP_EXPORT_SIZEOF(PrefetchArgs, mep::PrefetchArgs)
