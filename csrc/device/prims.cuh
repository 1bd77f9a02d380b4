// Device primitives: bounded waits, software grid barrier, cross-rank barrier,
// peer-memory addressing, bulk-copy and mbarrier wrappers.
//
// Behavioural counterpart of the reference's moonep/_common.py (grid_sync :249-271,
// cross_rank_barrier :274-346, bulk copies :414-459) with two deliberate differences:
//  * every wait is bounded by a time budget (nanoseconds, converted to SM cycles and measured
//    with clock64); on expiry the waiter records the site in MepStatus and the kernel returns
//    -- it never traps;
//  * cross-rank flags are monotone epochs (one slot per peer) instead of +/-1 counters,
//    so a barrier needs no reset and a late or repeated arrival cannot corrupt it.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../mep_types.h"

#ifndef MEP_POLL_SLEEP_NS
#define MEP_POLL_SLEEP_NS 40   // pause between two polls of an mbarrier (see mbar_wait_bounded)
#endif

namespace mep {

// ---------------------------------------------------------------- memory-model wrappers
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v; asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
// 16-byte load served by L2 (never by this SM's L1): for data another agent wrote during this kernel
__device__ __forceinline__ int4 ld_cg_v4(const void* p) {
  int4 v; asm volatile("ld.global.cg.v4.s32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_release_gpu(uint32_t* p, uint32_t v) {
  uint32_t old; asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory"); return old;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m; asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(m)); return m;
}
// 16-byte accesses that bypass L1 allocation (streaming payloads, peer memory)
__device__ __forceinline__ int4 ld_nc_v4(const void* p) {
  int4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v;
}
// peer data that other GPUs may have just written: weak load through L2, no L1 allocation
__device__ __forceinline__ int4 ld_peer_v4(const void* p) {
  int4 v; asm volatile("ld.global.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_v4(void* p, int4 v) {
  asm volatile("st.global.v4.s32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_na_v4(void* p, int4 v) {
  asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// Counterpart of the reference's pdl_wait_predecessor / pdl_trigger_dependents
// (moonep/_common.py:393-406). pdl_wait: returns once every kernel this launch depends on has
// completed and its writes are visible (a no-op for a launch without the attribute).
// pdl_trigger: this CTA has nothing left that a dependent launch must wait for before being
// SCHEDULED; the dependent still waits in pdl_wait for this grid to finish.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- NVSwitch multicast
// One store, delivered by the switch to the same offset of every rank's chunk.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, int4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc_addr), "f"(__int_as_float(v.x)), "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)), "f"(__int_as_float(v.w)) : "memory");
}
// Orders accesses made through the multicast alias against accesses through the ordinary mapping.
__device__ __forceinline__ void fence_proxy_alias() { asm volatile("fence.proxy.alias;" ::: "memory"); }

// ---------------------------------------------------------------- peer addressing
__device__ __forceinline__ char* peer_ptr(const MepRankCtx& c, int r, int64_t off) {
  return c.heap_base + (int64_t)r * c.chunk_stride + off;
}

// ---------------------------------------------------------------- status
__device__ __forceinline__ void report(const MepRankCtx& c, int code, int kernel, int site,
                                       int peer, uint32_t observed, uint32_t expected) {
  MepStatus* s = c.status;
  if (atomicCAS(&s->code, 0, code) == 0) {
    s->kernel = kernel; s->site = site; s->rank = c.rank; s->peer = peer;
    s->observed = observed; s->expected = expected;
    __threadfence();
    if (c.status_host) { *(volatile int32_t*)c.status_host = code; __threadfence_system(); }
  }
}
__device__ __forceinline__ void count(const MepRankCtx& c, int slot, unsigned long long v) {
  if (c.counters) atomicAdd(c.counters + slot, v);
}
__device__ __forceinline__ bool aborted(const MepRankCtx& c) {
  return *(volatile int32_t*)&c.status->code != 0;
}

// Wait budgets are given in nanoseconds but measured with the SM cycle counter (reading
// %globaltimer costs about a microsecond, far too slow for a polling loop): cycles = ns * 2.2
// over-estimates the budget at any clock the part can run at, which is the safe direction.
__device__ __forceinline__ long long budget_cycles(uint64_t ns) { return (long long)(ns * 22 / 10); }

// Spin helper: `cond()` is polled; after a first burst of polls the cycle counter and the abort
// word are checked every 64 polls. Returns false when the budget ran out or another waiter
// already failed.
template <class Cond>
__device__ __forceinline__ bool bounded_wait(const MepRankCtx& c, Cond cond) {
#pragma unroll 1
  for (int i = 0; i < 256; ++i) { if (cond()) return true; }
  const long long t0 = clock64(), lim = budget_cycles(c.wait_budget_ns);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) { if (cond()) return true; }
    if (aborted(c)) return false;
    if (clock64() - t0 > lim) return false;
    __nanosleep(20);
  }
}

// ---------------------------------------------------------------- tracing
// One record per call (call it from a single thread of the warp/CTA you want to stamp).
__device__ __forceinline__ void trace_mark(const MepRankCtx& c, int kernel, int site) {
  if (c.trace == nullptr) return;
  const unsigned long long i = atomicAdd(c.trace, 1ull);
  if ((int64_t)i < c.trace_cap) {
    c.trace[1 + 2 * i] = globaltimer_ns();
    c.trace[2 + 2 * i] = ((unsigned long long)kernel << 48) | ((unsigned long long)site << 32) |
                         ((unsigned long long)blockIdx.x << 8) | (unsigned long long)(threadIdx.x >> 5);
  }
}

// Same record format, but the first word carries a caller-supplied value (e.g. accumulated cycles).
__device__ __forceinline__ void trace_value(const MepRankCtx& c, int kernel, int site, unsigned long long value) {
  if (c.trace == nullptr) return;
  const unsigned long long i = atomicAdd(c.trace, 1ull);
  if ((int64_t)i < c.trace_cap) {
    c.trace[1 + 2 * i] = value;
    c.trace[2 + 2 * i] = ((unsigned long long)kernel << 48) | ((unsigned long long)site << 32) |
                         ((unsigned long long)blockIdx.x << 8) | (unsigned long long)(threadIdx.x >> 5);
  }
}

// ---------------------------------------------------------------- grid barrier
// All `nblocks` CTAs of one rank (blockIdx.x in [0, nblocks)) must call it; CTAs must be
// co-resident (cooperative launch). Self-resetting: CTA 0 adds 0x80000000-(n-1), the
// others add 1, so the top bit flips exactly when everyone has arrived.
// `sys` makes this CTA's earlier writes to peer memory visible system-wide first.
// The weight-pool kernels (prefetch, grad_reduce) use a barrier word and a cross-rank flag row of their own
// (kWeightLaneRow), so that one of them may run beside a token kernel (dispatch, combine) of the same Buffer
// on another stream; two kernels of the same lane must still be ordered by their streams.
constexpr int kWeightLaneRow = 3;
// The duplicate expansion / reduction kernels split every row into this many column parts, one warp each.
constexpr int kDupParts = 4;
// ... so their grids are whole multiples of it (block b works on part b % kDupParts).
inline int dup_grid(int num_blocks) { return (num_blocks + kDupParts - 1) / kDupParts * kDupParts; }
__device__ __forceinline__ int bar_lane(int kernel) { return (kernel == MEP_K_PREFETCH || kernel == MEP_K_GRAD_REDUCE) ? 1 : 0; }
__device__ __forceinline__ bool grid_sync(const MepRankCtx& c, int nblocks, int kernel, int site, bool sys = false) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sys) __threadfence_system(); else __threadfence();
    bool ok = true;
    if (nblocks > 1) {
      const uint32_t inc = (blockIdx.x == 0) ? (0x80000000u - (uint32_t)(nblocks - 1)) : 1u;
      uint32_t* word = c.grid_bar + bar_lane(kernel);
      const uint32_t old = atom_add_release_gpu(word, inc);
      uint32_t now = 0;
      ok = bounded_wait(c, [&] { now = ld_acquire_gpu(word); return ((now ^ old) & 0x80000000u) != 0; });
      if (!ok) report(c, MEP_ERR_GRID_SYNC_TIMEOUT, kernel, site, blockIdx.x, now, old);
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// ---------------------------------------------------------------- cross-rank barrier
// Executed by ONE CTA of the rank (all its threads). Flag row `row` of every rank holds
// one epoch word per peer; arrival = release-store of the new epoch into slot [my rank]
// of every peer; completion = every slot of my row has reached the epoch.
__device__ __forceinline__ bool cross_rank_arrive_wait(const MepRankCtx& c, int row, int kernel, int site) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  if (threadIdx.x == 0) { s_epoch = c.epoch[row] + 1; c.epoch[row] = s_epoch; s_fail = 0; }
  __syncthreads();
  const uint32_t ep = s_epoch;
  for (int p = threadIdx.x; p < c.R; p += blockDim.x) {
    uint32_t* slot = (uint32_t*)peer_ptr(c, p, c.off_bar) + row * MEP_MAX_RANKS + c.rank;
    st_release_sys(slot, ep);
  }
  for (int p = threadIdx.x; p < c.R; p += blockDim.x) {
    const uint32_t* slot = (const uint32_t*)peer_ptr(c, c.rank, c.off_bar) + row * MEP_MAX_RANKS + p;
    uint32_t seen = 0;
    bool ok = bounded_wait(c, [&] { seen = ld_acquire_sys(slot); return (int32_t)(seen - ep) >= 0; });
    if (!ok) { report(c, MEP_ERR_PEER_TIMEOUT, kernel, site, p, seen, ep); s_fail = 1; }
  }
  __syncthreads();
  return s_fail == 0;
}

// Full barrier for every CTA of the rank: local grid barrier (publishing peer writes),
// CTA 0 exchanges epochs with the peers, second grid barrier releases the rest.
__device__ __forceinline__ bool cross_rank_barrier(const MepRankCtx& c, int nblocks, int row, int kernel, int site) {
  if (!grid_sync(c, nblocks, kernel, site, true)) return false;
  if (blockIdx.x == 0) {
    if (c.R > 1) {
      const uint64_t t0 = (c.counters && threadIdx.x == 0) ? globaltimer_ns() : 0;
      cross_rank_arrive_wait(c, row, kernel, site + 1);
      if (c.counters && threadIdx.x == 0) { count(c, MEP_CNT_BARRIER_WAIT_NS, globaltimer_ns() - t0); count(c, MEP_CNT_BARRIERS, 1); }
    }
  }
  if (!grid_sync(c, nblocks, kernel, site + 2, false)) return false;
  return !aborted(c);
}

// ---------------------------------------------------------------- mbarrier + bulk copies (local TMA engine)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded mbarrier wait (budget in nanoseconds, see budget_cycles).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  // Back off between polls. Measured on the CTA-pair wgrad kernel (10 polling threads per CTA):
  // 1106 TFLOP/s with this 40 ns pause, 875 without it -- threads spinning on barriers keep the
  // shared-memory pipe busy and slow down every other barrier / copy instruction of the CTA.
#pragma unroll 1
  for (int i = 0; i < 4096; ++i) { __nanosleep(MEP_POLL_SLEEP_NS); if (mbar_try_wait(bar, parity)) return true; }
  const long long t0 = clock64(), lim = budget_cycles(budget_ns);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) { __nanosleep(MEP_POLL_SLEEP_NS); if (mbar_try_wait(bar, parity)) return true; }
    if (clock64() - t0 > lim) return false;
  }
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// 1-D bulk copy global -> this CTA's shared memory, completion counted on `bar`.
// The source may be local or peer memory (this form has no multicast). Size and both addresses multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 1-D bulk copy shared -> global (local or peer memory), tracked by bulk groups.
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :: "l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" :: "n"(N) : "memory"); }

// ---------------------------------------------------------------- warp helpers
__device__ __forceinline__ int warp_incl_scan(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += t; }
  return v;
}
__device__ __forceinline__ long long warp_max64(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { long long t = __shfl_xor_sync(0xffffffffu, v, o); v = t > v ? t : v; }
  return v;
}
// key for "largest value, lowest index wins ties"
__device__ __forceinline__ long long argmax_key(int value, int index) {
  return ((long long)value << 32) | (uint32_t)(0x7fffffff - index);
}
__device__ __forceinline__ int key_index(long long key) { return 0x7fffffff - (int)(uint32_t)(key & 0xffffffffu); }
__device__ __forceinline__ int key_value(long long key) { return (int)(key >> 32); }

}  // namespace mep
