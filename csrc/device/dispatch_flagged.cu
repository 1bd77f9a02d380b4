// Dispatch with per-tile ready flags: the consumer (the grouped GEMM that reads the shard) starts
// on a 128-row tile as soon as that tile is complete, instead of after the whole all-to-all.
//
// The reference ends its dispatch with a full cross-rank barrier before anything may read the
// shard (moonep/dispatch.py:687-692) and expands duplicate rows in a separate kernel afterwards
// (moonep/dispatch_epilogue.py:44-304). Here one kernel per rank does all of it, tile by tile:
//
//   sender warps    walk the plan's SEND LIST -- the rows to put on the wire, ordered by
//                   (destination tile, destination rank rotated by the own rank) -- so that every
//                   rank's shard fills up front to back at the same pace and no destination takes
//                   traffic from two senders at once. Per row: local bulk copy into shared memory,
//                   one bulk store to the destination slot, and for every slot of that token on that
//                   rank the 4-byte side tables (route weight, provenance, `rowsrc`). Once the bulk
//                   store has COMPLETED the warp adds one arrival to the destination tile's counter
//                   (red.release.sys); duplicate slots arrive right after their `rowsrc` entry.
//   zero-fill       padding rows of the local shard are cleared and arrive as well, unused slots
//                   behind the last group arrive without being written: every slot of every tile
//                   gets exactly one arrival per dispatch, so a tile is complete when its counter has
//                   reached (dispatches so far) x (rows of the tile) and no counter is ever reset.
//   expander warps  draw the local tiles in ascending order; when a tile's arrivals are complete they
//                   copy each duplicate row from the row it duplicates (same shard, a tile that is
//                   complete too) and publish tile_done[t] = epoch (st.release.gpu).
//
// A consumer polls tile_done[t] (ld.acquire.gpu, bounded) before it loads rows of tile t; it must
// leave `num_sms` SMs free so that this kernel is resident while the consumer waits. The kernel
// still ends with the cross-rank barrier, so its completion means what the plain dispatch's does.
//
// Which row goes on the wire: of a token's slots on one rank, the one with the LOWEST slot offset
// (not the lowest k as in plan.dst's sign encoding), so a duplicate always copies from an earlier
// slot and tiles complete in the order the consumer walks them.
#include "prims.cuh"
#include "dispatch_args.h"
#include "../host/launch.h"

namespace mep {

constexpr int kFSend = 5;                                          // sender warps per CTA (`stages` row slots each)
constexpr int kExpWarps = 2;                                       // expander warps per CTA (two row slots each)
constexpr int kFlagThreads = (kFSend + 1 + kExpWarps) * 32;        // senders + zero-fill warp + expanders
constexpr int kSigLag = 2;          // a unit's arrivals are signalled once at most this many newer units are pending
constexpr int kSigBatch = 8;        // units between two signalling rounds (one system-scope fence per round)
constexpr int kSigRing = 16;         // units whose slot lists are remembered until they are signalled (>= kSigLag + kSigBatch)

__device__ __forceinline__ uint32_t* ready_of(const MepRankCtx& c, int d) { return (uint32_t*)peer_ptr(c, d, c.off_ready); }
__device__ __forceinline__ int tile_rows(const MepRankCtx& c, int t) {
  const int r = c.NvS - t * MEP_FLAG_ROWS; return r < MEP_FLAG_ROWS ? r : MEP_FLAG_ROWS;
}
__device__ __forceinline__ void bar_expanders() { asm volatile("bar.sync 1, %0;" :: "n"(kExpWarps * 32) : "memory"); }
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_done() { asm volatile("cp.async.bulk.wait_group %0;" :: "n"(N) : "memory"); }

// ------------------------------------------------------------------ flag epoch
// One thread: a new flagged dispatch is about to be issued. Runs in stream order BEFORE the
// dispatch kernel and before every consumer of its flags, so both read the same epoch.
__global__ void flag_epoch_bump_kernel(MepCtxPack P) {
  const MepRankCtx* c = P.ctx[blockIdx.y];
  if (threadIdx.x == 0) { c->flag_epoch[0] += 1u; c->flag_epoch[1] = 0u; }
}

// ------------------------------------------------------------------ send list
// send_list = the entries whose row goes on the wire (per token and destination rank the slot with
// the lowest offset), counting-sorted by bucket = (slot >> shift) * R + (d - rank mod R). Three
// grid-wide steps on a bucket histogram in device memory: classify + count, exclusive scan (one
// CTA), place. The order inside a bucket is whatever the atomics give (all of a bucket's rows
// belong to one tile of one destination).
struct SendOrderArgs {
  const int32_t* dst; const int32_t* cu_seqlens; int32_t* send_list; int32_t* send_meta;
  int32_t* hist;      // [nbuckets] scratch, zero on entry
  int32_t* bucket;    // [N] scratch: bucket of a wire entry, -1 for every other entry
};
struct SendOrderArgsPack { SendOrderArgs a[MEP_MAX_VRANKS]; };

__global__ void __launch_bounds__(256) send_classify_kernel(MepCtxPack P, SendOrderArgsPack A, int shift, int nbuckets) {
  const MepRankCtx& c = *P.ctx[blockIdx.y];
  const SendOrderArgs& a = A.a[blockIdx.y];
  const int K = c.K, NvS = c.NvS, R = c.R, N = c.N;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) {
    const int s = i / K;
    const int dv = a.dst[i];
    const int raw = dv >= 0 ? dv : -dv - 1;
    const int d = raw / NvS, loff = raw - d * NvS;
    bool wire = d < R;
    if (!wire) report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 50, s, (uint32_t)raw, (uint32_t)(R * NvS));
    for (int k2 = 0; k2 < K && wire; ++k2) {
      const int dv2 = a.dst[(size_t)s * K + k2];
      const int raw2 = dv2 >= 0 ? dv2 : -dv2 - 1;
      if (raw2 / NvS == d && raw2 < raw) wire = false;     // same rank, lower slot
    }
    int b = -1;
    if (wire) {
      b = (loff >> shift) * R + (d - c.rank + R) % R;
      if (b >= nbuckets) b = nbuckets - 1;
      atomicAdd(a.hist + b, 1);
    }
    a.bucket[i] = b;
  }
}

__global__ void __launch_bounds__(1024, 1) send_scan_kernel(MepCtxPack P, SendOrderArgsPack A, int nbuckets) {
  const MepRankCtx& c = *P.ctx[blockIdx.y];
  const SendOrderArgs& a = A.a[blockIdx.y];
  __shared__ int s_part[32];
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  // exclusive scan of the bucket counts: each thread owns a contiguous run of buckets
  const int per = (nbuckets + nt - 1) / nt, b0 = tid * per, b1 = min(nbuckets, b0 + per);
  int sum = 0;
  for (int b = b0; b < b1; ++b) sum += a.hist[b];
  const int incl = warp_incl_scan(sum);
  if (lane == 31) s_part[warp] = incl;
  __syncthreads();
  if (warp == 0) { const int v = lane < nwarps ? s_part[lane] : 0; const int iv = warp_incl_scan(v); s_part[lane] = iv - v; }
  __syncthreads();
  int run = s_part[warp] + incl - sum;
  for (int b = b0; b < b1; ++b) { const int n = a.hist[b]; a.hist[b] = run; run += n; }
  if (tid == nt - 1) {
    a.send_meta[0] = run;
    a.send_meta[1] = a.cu_seqlens[2 * c.epn - 1];
    a.send_meta[2] = 0; a.send_meta[3] = 0;
  }
}

__global__ void __launch_bounds__(256) send_place_kernel(MepCtxPack P, SendOrderArgsPack A) {
  const MepRankCtx& c = *P.ctx[blockIdx.y];
  const SendOrderArgs& a = A.a[blockIdx.y];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < c.N; i += gridDim.x * blockDim.x) {
    const int b = a.bucket[i];
    if (b >= 0) a.send_list[atomicAdd(a.hist + b, 1)] = i;
  }
}

// ------------------------------------------------------------------ dispatch
// Shared memory: [kFSend x stages rows: sender rings][kExpWarps x 2 rows: two slots per expander warp]
// [padding-row tables]. Every data movement goes through the copy engine (bulk copies), so the
// bytes in flight per SM are the rows staged in shared memory, not registers.
__global__ void __launch_bounds__(kFlagThreads, 1)
dispatch_flagged_kernel(MepCtxPack P, DispatchArgsPack A, int stages) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const DispatchArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[kFSend * kMaxStages];
  __shared__ __align__(8) uint64_t s_xbar[kExpWarps * 2];
  __shared__ uint32_t s_sig[kFSend][kSigRing];               // (destination << 8 | slots stored) of a unit
  __shared__ int s_sloff[kFSend][kSigRing][MEP_MAX_TOPK];     // the slots a unit stored to
  __shared__ int s_znext, s_ztotal;
  __shared__ int s_xtile, s_xn, s_xfail;
  __shared__ int s_xlist[MEP_FLAG_ROWS];
  __shared__ int s_peer[MEP_MAX_RANKS];     // rows this CTA sent to each rank (counters only)
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = c.K, S = c.S, NvS = c.NvS;
  const uint32_t row_bytes = (uint32_t)c.H * 2u;
  const uint32_t ep = *(volatile uint32_t*)c.flag_epoch;
  const int cu_end = a.send_meta[1];

  if (tid == 0) { s_xfail = 0; s_xn = 0; }
  if (tid < MEP_MAX_RANKS) s_peer[tid] = 0;
  if (tid < kFSend * kMaxStages) mbar_init(&s_bar[tid], 1);
  if (tid < kExpWarps * 2) mbar_init(&s_xbar[tid], 1);
  fence_mbar_init();
  const int ngroups = 2 * c.epn;
  unsigned char* xslots = smem + (size_t)kFSend * stages * row_bytes;
  int* s_zpre = reinterpret_cast<int*>(xslots + (size_t)kExpWarps * 2 * row_bytes);
  int* s_zstart = s_zpre + ngroups + 1;
  for (int g = tid; g < ngroups; g += blockDim.x) { s_zstart[g] = a.zero_fill[2 * g]; s_zpre[g + 1] = a.zero_fill[2 * g + 1]; }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int g = 0; g < ngroups; ++g) { const int n = s_zpre[g + 1]; s_zpre[g] = run; run += n; }
    s_zpre[ngroups] = run; s_ztotal = run; s_znext = 0;
  }
  __syncthreads();

  uint32_t* const my_ready = ready_of(c, c.rank);
  // Clear the padding rows that fall to this CTA; each cleared row is one arrival for its tile.
  auto zero_fill_work = [&]() {
    char* hid = peer_ptr(c, c.rank, c.off_hidden);
    float* wts = (float*)peer_ptr(c, c.rank, c.off_weights);
    int* rsrc = (int*)peer_ptr(c, c.rank, c.off_rowsrc);
    const int vec_per_row = (int)(row_bytes >> 4);
    const int4 z = make_int4(0, 0, 0, 0);
    const int total = s_ztotal;
    int done = 0;
    for (;;) {
      int k = 0;
      if (lane == 0) k = atomicAdd(&s_znext, 1);
      k = __shfl_sync(0xffffffffu, k, 0);
      const long long rr = (long long)blockIdx.x + (long long)k * nb;
      if (rr >= total) break;
      int lo = 0, hi = ngroups - 1;                 // last g with s_zpre[g] <= rr
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (s_zpre[mid] <= (int)rr) lo = mid; else hi = mid - 1; }
      const int prow = s_zstart[lo] + ((int)rr - s_zpre[lo]);
      if ((unsigned)prow >= (unsigned)NvS) {
        if (lane == 0) report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 40, lo, (uint32_t)prow, (uint32_t)NvS);
        continue;
      }
      char* row = hid + (size_t)prow * row_bytes;
      for (int v = lane; v < vec_per_row; v += 32) st_v4(row + (size_t)v * 16, z);
      if (lane == 0) {
        if (a.weights) wts[prow] = 0.f;
        if (a.srcinfo_off) ((int*)peer_ptr(c, c.rank, (size_t)a.srcinfo_off))[prow] = -1;
        rsrc[prow] = -1;
      }
      __syncwarp();                                  // every lane's stores precede the releasing arrival
      if (lane == 0) red_release_sys_add(my_ready + prow / MEP_FLAG_ROWS, 1u);
      ++done;
    }
    if (lane == 0 && done) count(c, MEP_CNT_PAD_ROWS, (unsigned long long)done);
  };

  if (tid == 0) trace_mark(c, MEP_K_DISPATCH, 1);
  if (a.entry_barrier) { if (!cross_rank_barrier(c, nb, 1, MEP_K_DISPATCH, 10)) return; }

  if (a.fresh && blockIdx.x == 0) {
    for (int d = tid; d < c.R; d += blockDim.x) {
      const int half = a.fresh == 3 ? (int)(__ldcg(c.vb_flags + c.num_vblocks) & 1u) : a.fresh - 1;
      const unsigned long long v = c.send_cnt[(size_t)half * c.R + d];
      int* cnt = (int*)peer_ptr(c, d, c.off_dupcnt) + 2 * c.rank;
      cnt[0] = (int)(v >> 32); cnt[1] = (int)(v & 0xffffffffu);
    }
  }

  if (warp < kFSend) {
    // ---------------------------------------------------------------- senders
    unsigned char* ring = smem + (size_t)warp * stages * row_bytes;
    uint64_t* bars = s_bar + warp * kMaxStages;
    const int nunits = a.send_meta[0];
    const int gw = blockIdx.x * kFSend + warp, nw = nb * kFSend;
    const int n = gw < nunits ? (nunits - gw + nw - 1) / nw : 0;       // this warp's units: gw, gw + nw, ...
    const int D = stages >= 3 ? 1 : 0, pre = stages - 1 - D;
    // the warp's list entries live in two register chunks of 32 (lane j of chunk A = unit cbase + j)
    auto load_chunk = [&](int c0) { const int j = c0 + lane; return j < n ? a.send_list[gw + (size_t)j * nw] : -1; };
    int entA = load_chunk(0), entB = load_chunk(32), cbase = 0;
    auto entry_of = [&](int j) {                   // cbase <= j < cbase + 64, called by all lanes
      const int o = j - cbase;
      const int va = __shfl_sync(0xffffffffu, entA, o & 31), vb = __shfl_sync(0xffffffffu, entB, o & 31);
      return o < 32 ? va : vb;
    };
    for (int i = 0; i < pre; ++i) {
      const int e = entry_of(i);
      if (lane == 0 && e >= 0) {
        mbar_expect_tx(&bars[i], row_bytes);
        bulk_g2s(ring + (size_t)i * row_bytes, a.hidden + (size_t)min(e / K, S - 1) * c.H, row_bytes, &bars[i]);
      }
    }
    int nd = 0; float nwt = 0.f;                   // plan entry / weight of the NEXT unit, fetched one unit ahead
    {
      const int e0 = entry_of(0);
      if (e0 >= 0 && e0 < S * K && lane < K) { const size_t o = (size_t)(e0 / K) * K + lane; nd = a.dst[o]; nwt = a.weights ? a.weights[o] : 0.f; }
    }
    int sent = 0, sent_remote = 0;
    // lane 0: the stores of units [signalled, upto) have completed -- one arrival per slot the token owns
    // on the destination (the slot that got the row, and on a peer its duplicates, whose rowsrc entry was
    // written before the store was issued). One system-scope fence covers the whole round.
    int signalled = 0;
    auto signal_upto = [&](int upto) {
      if (upto <= signalled) return;
      fence_proxy_async();
      fence_acq_rel_sys();
      for (int j = signalled; j < upto; ++j) {
        const uint32_t v = s_sig[warp][j & (kSigRing - 1)];
        uint32_t* rdy = ready_of(c, (int)(v >> 8));
        for (int i = 0; i < (int)(v & 0xffu); ++i) red_relaxed_sys_add(rdy + s_sloff[warp][j & (kSigRing - 1)][i] / MEP_FLAG_ROWS, 1u);
      }
      signalled = upto;
    };
    int it = 0;
    for (; it < n; ++it) {
      if (it - cbase >= 32) { entA = entB; cbase += 32; entB = load_chunk(cbase + 32); }
      const int e = entry_of(it), e1 = entry_of(it + 1), eL = entry_of(it + pre);
      const int s = e / K, kp = e - s * K;
      const int st = it % stages;
      const uint32_t parity = (uint32_t)(it / stages) & 1u;
      const int dval = nd; const float w = nwt;
      if (e1 >= 0 && e1 < S * K && lane < K) { const size_t o = (size_t)(e1 / K) * K + lane; nd = a.dst[o]; nwt = a.weights ? a.weights[o] : 0.f; }
      bool ok = true;
      if (lane == 0) {
        if (eL >= 0) {
          if (D) bulk_wait_read<1>(); else bulk_wait_read<0>();
          const int ns = (it + pre) % stages;
          mbar_expect_tx(&bars[ns], row_bytes);
          bulk_g2s(ring + (size_t)ns * row_bytes, a.hidden + (size_t)min(eL / K, S - 1) * c.H, row_bytes, &bars[ns]);
        }
        ok = mbar_wait_bounded(&bars[st], parity, c.wait_budget_ns);
        if (!ok) report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_DISPATCH, 20, s, 0, 0);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      int d = -1, loff = 0;
      if (lane < K) { const int raw = dval >= 0 ? dval : -dval - 1; d = raw / NvS; loff = raw - d * NvS; }
      const int du = __shfl_sync(0xffffffffu, d, kp), lu = __shfl_sync(0xffffffffu, loff, kp);
      const bool good = du >= 0 && du < c.R && e < S * K;   // the send list only names valid entries; checked all the same
      const bool local = du == c.rank;
      const bool mine = good && lane < K && d == du;
      if (mine) {
        // side tables of every slot this token owns on that rank. On the own rank every slot gets the
        // row itself (a store costs no link bandwidth there); on a peer only slot `lu` does and the
        // other slots are duplicates that the peer expands from it.
        if (a.weights) ((float*)peer_ptr(c, du, c.off_weights))[loff] = w;
        if (a.srcinfo_off) ((int*)peer_ptr(c, du, (size_t)a.srcinfo_off))[loff] = c.rank * (S * K) + s * K + lane;
        ((int*)peer_ptr(c, du, c.off_rowsrc))[loff] = local ? loff : lu;
      }
      const unsigned owned = __ballot_sync(0xffffffffu, mine);
      const unsigned stores = __ballot_sync(0xffffffffu, mine && (local || loff == lu));
      __syncwarp();
      int nst = 0, nown = 0;
      for (unsigned m = owned; m; m &= m - 1) {
        const int k = __ffs(m) - 1;
        const int lk = __shfl_sync(0xffffffffu, loff, k);
        if (lane == 0) {
          if ((stores >> k) & 1u) {
            bulk_s2g(peer_ptr(c, du, c.off_hidden) + (size_t)lk * row_bytes, ring + (size_t)st * row_bytes, row_bytes);
            ++nst;
          }
          s_sloff[warp][it & (kSigRing - 1)][nown] = lk;
        }
        ++nown;
      }
      if (lane == 0) {
        if (good) {
          sent += nst; if (!local) sent_remote += nst;
          if (c.counters) atomicAdd(&s_peer[du], nst);
        } else {
          report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 41, s, (uint32_t)dval, (uint32_t)(c.R * NvS));
        }
        s_sig[warp][it & (kSigRing - 1)] = ((uint32_t)(good ? du : 0) << 8) | (uint32_t)nown;
        bulk_commit();                               // one bulk group per unit, empty for a dropped one
        if ((it % kSigBatch) == kSigBatch - 1 && it >= kSigLag) { bulk_wait_done<kSigLag>(); signal_upto(it + 1 - kSigLag); }
      }
    }
    if (lane == 0) {
      bulk_wait_done<0>();
      if (it == n) signal_upto(n);
      if (sent) { count(c, MEP_CNT_ROWS_SENT, (unsigned long long)sent); count(c, MEP_CNT_ROWS_REMOTE, (unsigned long long)sent_remote); }
      trace_mark(c, MEP_K_DISPATCH, 2);
    }
    zero_fill_work();
    if (lane == 0) trace_mark(c, MEP_K_DISPATCH, 3);
  } else if (warp == kFSend) {
    // ---------------------------------------------------------------- zero-fill warp
    if (blockIdx.x == 0) {
      // slots behind the last group take no data: they arrive unwritten, so that every tile's
      // counter advances by the same amount per dispatch
      for (int t = cu_end / MEP_FLAG_ROWS + lane; t < c.ntiles; t += 32) {
        const int lo = max(t * MEP_FLAG_ROWS, cu_end), hi = min((t + 1) * MEP_FLAG_ROWS, NvS);
        if (hi > lo) red_release_sys_add(my_ready + t, (uint32_t)(hi - lo));
      }
      if (lane == 0) count(c, MEP_CNT_DISPATCHES, 1);
    }
    zero_fill_work();
    if (lane == 0) trace_mark(c, MEP_K_DISPATCH, 4);
  } else {
    // ---------------------------------------------------------------- expanders
    const int xt = tid - (kFSend + 1) * 32, xw = xt >> 5;
    const int used_tiles = (cu_end + MEP_FLAG_ROWS - 1) / MEP_FLAG_ROWS;
    const int* rsrc = (const int*)peer_ptr(c, c.rank, c.off_rowsrc);
    char* hid = peer_ptr(c, c.rank, c.off_hidden);
    unsigned char* slot = xslots + (size_t)xw * 2 * row_bytes;      // this warp's two slots
    uint32_t xpar = 0;                                              // bit s = parity of slot s's mbarrier
    auto tile_complete = [&](int t, int site) {      // bounded wait for tile t's arrivals (any thread)
      const uint32_t target = ep * (uint32_t)tile_rows(c, t);
      uint32_t seen = 0;
      const bool ok = bounded_wait(c, [&] { seen = ld_acquire_sys(my_ready + t); return (int32_t)(seen - target) >= 0; });
      if (!ok) { report(c, MEP_ERR_FLAG_TIMEOUT, MEP_K_DISPATCH, site, t, seen, target); s_xfail = 1; }
      return ok;
    };
    int ndup = 0;
    for (;;) {
      if (xt == 0) { s_xtile = (int)atomicAdd(c.flag_epoch + 1, 1u); s_xn = 0; }
      bar_expanders();
      const int t = s_xtile;
      if (t >= used_tiles || s_xfail) break;
      if (xt == 0) tile_complete(t, 60);
      bar_expanders();
      if (s_xfail) break;
      for (int r = xt; r < MEP_FLAG_ROWS; r += kExpWarps * 32) {
        const int row = t * MEP_FLAG_ROWS + r;
        if (row < NvS) {
          const int src = __ldcg(rsrc + row);
          if (src >= 0 && src != row) {
            if (src >= NvS) report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 61, row, (uint32_t)src, (uint32_t)NvS);
            else {
              const int st = src / MEP_FLAG_ROWS;
              if (st == t || tile_complete(st, 62)) s_xlist[atomicAdd(&s_xn, 1)] = (src << 7) | r;
            }
          }
        }
      }
      bar_expanders();
      if (s_xfail) break;
      // duplicate rows of this tile: row of the same shard -> one of this warp's two slots -> duplicate
      // slot; the load of the next row is under way while this one is stored. Everything a copy reads
      // was acquired above.
      const int nd_ = s_xn;
      if (lane == 0) {
        const int nj = nd_ > xw ? (nd_ - xw + kExpWarps - 1) / kExpWarps : 0;
        auto issue_load = [&](int j) {
          const int v = s_xlist[xw + j * kExpWarps], sl = j & 1;
          mbar_expect_tx(&s_xbar[xw * 2 + sl], row_bytes);
          bulk_g2s(slot + (size_t)sl * row_bytes, hid + (size_t)(v >> 7) * row_bytes, row_bytes, &s_xbar[xw * 2 + sl]);
        };
        fence_proxy_async();
        if (nj > 0) issue_load(0);
        for (int j = 0; j < nj; ++j) {
          if (j + 1 < nj) { bulk_wait_read<0>(); issue_load(j + 1); }     // that slot's previous store has left it
          const int sl = j & 1;
          if (!mbar_wait_bounded(&s_xbar[xw * 2 + sl], (xpar >> sl) & 1u, c.wait_budget_ns)) {
            report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_DISPATCH, 63, t, 0, 0); s_xfail = 1; break;
          }
          xpar ^= 1u << sl;
          const int v = s_xlist[xw + j * kExpWarps];
          bulk_s2g(hid + (size_t)(t * MEP_FLAG_ROWS + (v & 127)) * row_bytes, slot + (size_t)sl * row_bytes, row_bytes);
          bulk_commit();
        }
        bulk_wait_done<0>(); fence_proxy_async();
      }
      if (xt == 0) ndup += nd_;
      bar_expanders();
      if (s_xfail) break;
      if (xt == 0) { __threadfence(); st_release_gpu(c.tile_done + t, ep); trace_mark(c, MEP_K_DISPATCH, 7); }
    }
    if (xt == 0) trace_mark(c, MEP_K_DISPATCH, 6);
    if (xt == 0 && ndup) count(c, MEP_CNT_DUP_ROWS, (unsigned long long)ndup);
  }
  cross_rank_barrier(c, nb, 1, MEP_K_DISPATCH, 30);
  if (c.counters && tid < c.R && tid < 48 && s_peer[tid]) count(c, MEP_CNT_PEER_ROWS + tid, (unsigned long long)s_peer[tid]);
  if (tid == 0) trace_mark(c, MEP_K_DISPATCH, 5);
}

// Bounded wait on a tile flag outside any collective: the test of the consumer-side timeout
// path (nothing ever completes the tile, the wait gives up and records a status).
__global__ void tile_wait_probe_kernel(MepCtxPack P, int tile) {
  const MepRankCtx c = *P.ctx[blockIdx.y];
  if (threadIdx.x == 0) {
    const uint32_t ep = *(volatile uint32_t*)c.flag_epoch;
    uint32_t seen = 0;
    const bool ok = bounded_wait(c, [&] { seen = ld_acquire_gpu(c.tile_done + tile); return (int32_t)(seen - ep) >= 0; });
    if (!ok) report(c, MEP_ERR_FLAG_TIMEOUT, MEP_K_WAIT_PROBE, 2, tile, seen, ep);
  }
}

}  // namespace mep

extern "C" int mep_launch_flag_epoch_bump(int nv, const MepRankCtx* const* ctxs, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "flag_epoch_bump: nv=%d out of range", nv);
  MepCtxPack P = {};
  for (int i = 0; i < nv; ++i) P.ctx[i] = ctxs[i];
  return mep::launch_plain(mep::flag_epoch_bump_kernel, dim3(1, nv), dim3(32), 0, stream, P);
}

// nbuckets for a geometry: one bucket per (flag tile, destination), coarser tiles beyond 40960 buckets.
extern "C" int mep_send_order_buckets(int NvS, int R, int* shift_out) {
  int shift = 7;
  while ((((long long)NvS >> shift) + 1) * R > 40960) ++shift;
  if (shift_out) *shift_out = shift;
  return (int)((((long long)NvS >> shift) + 1) * R);
}

extern "C" int mep_launch_send_order(int nv, const MepRankCtx* const* ctxs, const mep::SendOrderArgs* args,
                                     int N, int NvS, int R, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "send_order: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::SendOrderArgsPack A = {};
  int shift = 7;
  const int nbuckets = mep_send_order_buckets(NvS, R, &shift);
  for (int i = 0; i < nv; ++i) {
    P.ctx[i] = ctxs[i]; A.a[i] = args[i];
    MEP_REQUIRE(args[i].hist && args[i].bucket, "send_order: scratch missing");
    MEP_CUDA_CHECK(cudaMemsetAsync(args[i].hist, 0, (size_t)nbuckets * sizeof(int), stream));
  }
  const int blocks = (N + 255) / 256 < 128 ? (N + 255) / 256 : 128;
  if (mep::launch_plain(mep::send_classify_kernel, dim3(blocks, nv), dim3(256), 0, stream, P, A, shift, nbuckets)) return -1;
  if (mep::launch_plain(mep::send_scan_kernel, dim3(1, nv), dim3(1024), 0, stream, P, A, nbuckets)) return -1;
  return mep::launch_plain(mep::send_place_kernel, dim3(blocks, nv), dim3(256), 0, stream, P, A);
}

extern "C" int mep_launch_dispatch_flagged(int nv, const MepRankCtx* const* ctxs, const mep::DispatchArgs* args,
                                           int num_sms, int H, int epn, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "dispatch: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::DispatchArgsPack A = {};
  for (int i = 0; i < nv; ++i) {
    P.ctx[i] = ctxs[i]; A.a[i] = args[i];
    MEP_REQUIRE(args[i].send_list && args[i].send_meta, "dispatch: the plan carries no send list (it was not made by a flagged dispatch)");
  }
  const size_t row = (size_t)H * 2;
  const size_t tables = (size_t)(4 * epn + 2) * sizeof(int);
  const size_t budget = 212 * 1024;      // dynamic part; the kernel's static tables take another ~14 KB of the 227 KB
  MEP_REQUIRE(budget > tables + row * (2 * mep::kExpWarps + mep::kFSend),
              "dispatch: H=%d rows (%zu B) with epn=%d do not fit shared memory", H, row, epn);
  int stages = (int)((budget - tables - row * 2 * mep::kExpWarps) / (row * mep::kFSend));
  if (stages > mep::kMaxStages) stages = mep::kMaxStages;
  const size_t smem = row * (mep::kFSend * stages + 2 * mep::kExpWarps) + tables;
  return mep::launch_cooperative(mep::dispatch_flagged_kernel, dim3(num_sms, nv), dim3(mep::kFlagThreads), smem,
                                 stream, false, P, A, stages);
}

extern "C" int mep_launch_tile_wait_probe(const MepRankCtx* ctx, int tile, cudaStream_t stream) {
  MepCtxPack P = {}; P.ctx[0] = ctx;
  return mep::launch_plain(mep::tile_wait_probe_kernel, dim3(1, 1), dim3(32), 0, stream, P, tile);
}

MEP_EXPORT_SIZEOF(SendOrderArgs, mep::SendOrderArgs)
