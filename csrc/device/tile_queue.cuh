// Tile hand-out for the persistent grouped-GEMM kernels.
//
// Static order: every role of a CTA walks the strided sequence first, first + stride, ... on its
// own (`Strided`); nothing is shared.
// Dynamic order (the launch passes a ticket counter): one thread per CTA (per CTA pair: one
// thread of the leader CTA), the TMA producer, is the scheduler. It draws the next tile number
// from the global counter -- CTAs that start late or run beside another kernel simply draw fewer
// tiles -- and publishes it through a small ring in shared memory to the other roles of the CTA
// (MMA issuer, epilogue warps) and, in a pair, to the peer CTA's ring through distributed shared
// memory, so every role walks the same sequence. A negative number ends the sequence.
//
// Ticket counter protocol (two words: next ticket, finished schedulers): schedulers draw with
// atomicAdd; at CTA teardown every scheduler CTA counts itself and the last one puts both words
// back to zero, so back-to-back launches (and CUDA-graph replays) need no host-side reset, and a
// kernel that gave up on a bounded wait still leaves the counter clean.
#pragma once
#include "prims.cuh"

namespace mep {
namespace tq {

constexpr int kSlots = 8;

struct Strided {
  int cur, step, n;
  __device__ __forceinline__ int next() { const int t = cur; cur += step; return t < n ? t : -1; }
};

struct Ring {
  uint64_t full[kSlots];    // scheduler -> roles of THIS CTA: slot holds a tile number
  uint64_t empty[kSlots];   // roles of all CTAs -> scheduler (only the scheduler CTA's copy is used)
  int id[kSlots];
};

__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait whose acquire covers writes made by the other CTA of the cluster.
__device__ __forceinline__ bool wait_cluster_bounded(uint64_t* bar, uint32_t parity, uint64_t budget_ns) {
  if (try_wait_cluster(bar, parity)) return true;
#pragma unroll 1
  for (int i = 0; i < 4096; ++i) { __nanosleep(MEP_POLL_SLEEP_NS); if (try_wait_cluster(bar, parity)) return true; }
  const long long t0 = clock64(), lim = budget_cycles(budget_ns);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) { __nanosleep(MEP_POLL_SLEEP_NS); if (try_wait_cluster(bar, parity)) return true; }
    if (clock64() - t0 > lim) return false;
  }
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster(uint32_t cluster_addr, int v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}

// Called by one thread per CTA before the CTA-wide (and cluster-wide) start-up barrier.
// `consumers` = number of threads, over all CTAs served by one scheduler, that call Consumer::next.
__device__ __forceinline__ void init(Ring* r, int consumers) {
  for (int i = 0; i < kSlots; ++i) { mbar_init(&r->full[i], 1); mbar_init(&r->empty[i], consumers); }
}

// PAIR: the scheduler also feeds the ring of cluster CTA 1.
template <bool PAIR>
struct Scheduler {
  Ring* r; uint32_t* counter; int ntiles, n;
  uint32_t pending;                // ticket drawn one call ahead: its round trip to L2 hides behind a tile's loads
  uint32_t peer_full, peer_id;     // cluster addresses of the peer ring's full[0] / id[0]
  __device__ __forceinline__ void setup(Ring* ring, uint32_t* ctr, int ntiles_) {
    r = ring; counter = ctr; ntiles = ntiles_; n = 0;
    if (PAIR) { peer_full = map_to_cta(smem_u32(&ring->full[0]), 1); peer_id = map_to_cta(smem_u32(&ring->id[0]), 1); }
    pending = atomicAdd(counter, 1u);
  }
  // Next tile, or -1 at the end of the sequence; -2 if the ring never drained (bounded wait expired).
  __device__ __forceinline__ int next(uint64_t budget_ns) {
    const int slot = n % kSlots; const uint32_t ph = (uint32_t)(n / kSlots) & 1u;
    const bool ok = PAIR ? wait_cluster_bounded(&r->empty[slot], ph ^ 1u, budget_ns) : mbar_wait_bounded(&r->empty[slot], ph ^ 1u, budget_ns);
    if (!ok) return -2;
    int t = (int)pending;
    if (t < ntiles) pending = atomicAdd(counter, 1u); else t = -1;
    *(volatile int*)&r->id[slot] = t;
    if (PAIR) st_cluster(peer_id + 4u * slot, t);
    mbar_arrive(&r->full[slot]);
    if (PAIR) arrive_cluster(peer_full + 8u * slot);
    ++n;
    return t;
  }
};

// Teardown accounting of one scheduler CTA (call after every role of the CTA has left its loop).
__device__ __forceinline__ void scheduler_done(uint32_t* counter, int nschedulers) {
  if (!counter) return;
  __threadfence();
  if (atomicAdd(counter + 1, 1u) == (uint32_t)nschedulers - 1u) {
    counter[0] = 0u; counter[1] = 0u;
    __threadfence();
  }
}

// PAIR: `sched_rank` (0) owns the empty barriers; arrivals go through cluster addresses.
template <bool PAIR>
struct Consumer {
  Ring* r; int n; uint32_t sched_empty;
  __device__ __forceinline__ void setup(Ring* ring) {
    r = ring; n = 0;
    if (PAIR) sched_empty = map_to_cta(smem_u32(&ring->empty[0]), 0);
  }
  // Next tile (>= 0), -1 at the end, -2 if the bounded wait expired. One thread per role calls this.
  __device__ __forceinline__ int next(uint64_t budget_ns) {
    const int slot = n % kSlots; const uint32_t ph = (uint32_t)(n / kSlots) & 1u;
    const bool ok = PAIR ? wait_cluster_bounded(&r->full[slot], ph, budget_ns) : mbar_wait_bounded(&r->full[slot], ph, budget_ns);
    if (!ok) return -2;
    const int t = *(volatile int*)&r->id[slot];
    if (PAIR) arrive_cluster(sched_empty + 8u * slot);
    else mbar_arrive(&r->empty[slot]);
    ++n;
    return t;
  }
};

}  // namespace tq
}  // namespace mep
