// Dispatch: fused permute + expert all-to-all, and the local duplicate expansion.
//
// Counterpart of the reference's DispatchKernel (moonep/dispatch.py:50-692) and
// DispatchEpilogueKernel (moonep/dispatch_epilogue.py:44-304), redesigned:
//  * every warp of every CTA is an independent sender: it stages one token row in its own
//    shared-memory ring slot with a local bulk copy and fans it out with one bulk store per
//    distinct destination rank (entries with dst >= 0) while its lanes scatter the K route
//    weights -- instead of one producer lane and one consumer lane per CTA;
//  * duplicate groups were already emitted by the planner from the sender side, so there is
//    no builder pass here: `dup_finalize` only compacts the per-source staging regions into
//    the plan-owned tables after the exit barrier;
//  * a spare warp per CTA clears the padding rows of the local shard meanwhile.
// Exit: one cross-rank barrier publishes all remote writes.
#include "prims.cuh"
#include "dispatch_args.h"
#include "../host/launch.h"

namespace mep {

template <int N> __device__ __forceinline__ void wait_read_le() { bulk_wait_read<N>(); }
__device__ __forceinline__ void wait_read_dyn(int n) {
  switch (n) {
    case 0: bulk_wait_read<0>(); break; case 1: bulk_wait_read<1>(); break;
    case 2: bulk_wait_read<2>(); break; case 3: bulk_wait_read<3>(); break;
    case 4: bulk_wait_read<4>(); break; case 5: bulk_wait_read<5>(); break;
    case 6: bulk_wait_read<6>(); break; default: bulk_wait_read<7>(); break;
  }
}

__global__ void __launch_bounds__(kDispThreads, 1)
dispatch_kernel(MepCtxPack P, DispatchArgsPack A, int stages) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const DispatchArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[kSendWarps * kMaxStages];
  __shared__ int s_err;
  __shared__ int s_znext, s_ztotal;
  __shared__ int s_peer[MEP_MAX_RANKS];     // rows this CTA sent to each rank (counters only)
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = c.K, S = c.S, NvS = c.NvS;
  const uint32_t row_bytes = (uint32_t)c.H * 2u;

  if (tid == 0) s_err = 0;
  if (tid < MEP_MAX_RANKS) s_peer[tid] = 0;
  if (tid < kSendWarps * kMaxStages) mbar_init(&s_bar[tid], 1);
  fence_mbar_init();
  // padding-row table of the local shard: s_zstart[g] = first padding row of group g,
  // s_zpre[g] = number of padding rows in groups < g (so a flat row index maps to (g, j))
  const int ngroups = 2 * c.epn;
  int* s_zpre = reinterpret_cast<int*>(smem + (size_t)kSendWarps * stages * row_bytes);
  int* s_zstart = s_zpre + ngroups + 1;
  int* s_meta_all = s_zstart + ngroups;            // [warps][kMetaTokens][K] dst, then the same for weights
  for (int g = tid; g < ngroups; g += blockDim.x) { s_zstart[g] = a.zero_fill[2 * g]; s_zpre[g + 1] = a.zero_fill[2 * g + 1]; }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int g = 0; g < ngroups; ++g) { const int n = s_zpre[g + 1]; s_zpre[g] = run; run += n; }
    s_zpre[ngroups] = run; s_ztotal = run; s_znext = 0;
  }
  __syncthreads();

  // Zero the padding rows (and their weight slots) that fall to this CTA (flat index = CTA id
  // mod grid). Any warp may call it; rows are handed out through a shared counter, so the
  // dedicated warp starts at once and the sender warps join when their tokens are on the wire.
  auto zero_fill_work = [&]() {
    char* hid = peer_ptr(c, c.rank, c.off_hidden);
    float* wts = (float*)peer_ptr(c, c.rank, c.off_weights);
    const int vec_per_row = (int)(row_bytes >> 4);
    const int4 z = make_int4(0, 0, 0, 0);
    const int total = s_ztotal;
    for (;;) {
      int k = 0;
      if (lane == 0) k = atomicAdd(&s_znext, 1);
      k = __shfl_sync(0xffffffffu, k, 0);
      const long long rr = (long long)blockIdx.x + (long long)k * nb;
      if (rr >= total) break;
      int lo = 0, hi = ngroups - 1;                 // last g with s_zpre[g] <= rr
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (s_zpre[mid] <= (int)rr) lo = mid; else hi = mid - 1; }
      const int prow = s_zstart[lo] + ((int)rr - s_zpre[lo]);
      if ((unsigned)prow >= (unsigned)NvS) {      // a corrupt zero_fill_ranges table must not reach memory
        if (lane == 0) report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 40, lo, (uint32_t)prow, (uint32_t)NvS);
        continue;
      }
      char* row = hid + (size_t)prow * row_bytes;
      for (int v = lane; v < vec_per_row; v += 32) st_v4(row + (size_t)v * 16, z);
      if (lane == 0 && a.weights) wts[prow] = 0.f;
      if (lane == 0 && a.srcinfo_off) ((int*)peer_ptr(c, c.rank, (size_t)a.srcinfo_off))[prow] = -1;
    }
  };

  if (tid == 0) trace_mark(c, MEP_K_DISPATCH, 1);
  if (a.entry_barrier) { if (!cross_rank_barrier(c, nb, 1, MEP_K_DISPATCH, 10)) return; }

  if (a.fresh && blockIdx.x == 0) {
    // tell every destination how many groups / duplicate offsets this rank appended
    for (int d = tid; d < c.R; d += blockDim.x) {
      const int half = a.fresh == 3 ? (int)(__ldcg(c.vb_flags + c.num_vblocks) & 1u) : a.fresh - 1;
      const unsigned long long v = c.send_cnt[(size_t)half * c.R + d];
      int* cnt = (int*)peer_ptr(c, d, c.off_dupcnt) + 2 * c.rank;
      cnt[0] = (int)(v >> 32); cnt[1] = (int)(v & 0xffffffffu);
    }
  }

  if (warp < kSendWarps) {
    unsigned char* ring = smem + (size_t)warp * stages * row_bytes;
    uint64_t* bars = s_bar + warp * kMaxStages;
    const int first = blockIdx.x * kSendWarps + warp, stride = nb * kSendWarps;
    const int ntok = first < S ? (S - first + stride - 1) / stride : 0;
    // Software pipeline over this warp's tokens. Bulk-group g holds the stores of token g. At
    // iteration `it` the slot of token it-1-D is reloaded with token it+pre (pre = stages-1-D):
    // its stores only need to have finished READING shared memory, so at most the D most recent
    // groups may still be pending (D = 1 when the ring is deep enough to skip the newest group).
    const int D = stages >= 3 ? 1 : 0;
    const int pre = stages - 1 - D;
    if (lane == 0) {
      for (int i = 0; i < pre && i < ntok; ++i) {
        mbar_expect_tx(&bars[i], row_bytes);
        bulk_g2s(ring + (size_t)i * row_bytes, a.hidden + (size_t)(first + i * stride) * c.H, row_bytes, &bars[i]);
      }
    }
    int* m_dst = s_meta_all + (size_t)warp * 2 * kMetaTokens * K;
    float* m_w = reinterpret_cast<float*>(m_dst + kMetaTokens * K);
    for (int it = 0; it < ntok; ++it) {
      const int s = first + it * stride;
      const int st = it % stages;
      const uint32_t parity = (uint32_t)(it / stages) & 1u;
      if ((it % kMetaTokens) == 0) {       // stage the next chunk of plan entries (all loads in flight at once)
        const int cnt = (ntok - it < kMetaTokens ? ntok - it : kMetaTokens) * K;
        __syncwarp();
        for (int i = lane; i < cnt; i += 32) {
          const int tt = i / K, k = i - tt * K;
          const size_t e = (size_t)(first + (it + tt) * stride) * K + k;
          m_dst[i] = a.dst[e];
          m_w[i] = a.weights ? a.weights[e] : 0.f;
        }
        __syncwarp();
      }
      int dval = 0; float w = 0.f;
      if (lane < K) { dval = m_dst[(it % kMetaTokens) * K + lane]; w = m_w[(it % kMetaTokens) * K + lane]; }
      bool ok = true;
      if (lane == 0) {
        const int nxt = it + pre;
        if (nxt < ntok) {
          if (D) bulk_wait_read<1>(); else bulk_wait_read<0>();
          const int ns = nxt % stages;
          mbar_expect_tx(&bars[ns], row_bytes);
          bulk_g2s(ring + (size_t)ns * row_bytes, a.hidden + (size_t)(first + nxt * stride) * c.H, row_bytes, &bars[ns]);
        }
        ok = mbar_wait_bounded(&bars[st], parity, c.wait_budget_ns);
        if (!ok) { report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_DISPATCH, 20, s, 0, 0); s_err = 1; }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      // a plan entry that names a rank outside the group (corrupt or foreign plan) is reported and
      // dropped before any address is formed from it
      bool entry_ok = lane < K;
      if (entry_ok) {
        const int raw = dval >= 0 ? dval : -dval - 1;
        if (raw / NvS >= c.R) {
          report(c, MEP_ERR_BOUNDS, MEP_K_DISPATCH, 41, s, (uint32_t)raw, (uint32_t)(c.R * NvS));
          entry_ok = false; dval = -1;          // negative: the send loop below skips it as well
        }
      }
      // route weights: every entry (primary or duplicate) owns a slot on its destination
      if (entry_ok && a.weights) {
        const int raw = dval >= 0 ? dval : -dval - 1;
        const int d = raw / NvS, loff = raw - d * NvS;
        ((float*)peer_ptr(c, d, c.off_weights))[loff] = w;
      }
      if (entry_ok && a.srcinfo_off) {
        const int raw = dval >= 0 ? dval : -dval - 1;
        const int d = raw / NvS, loff = raw - d * NvS;
        ((int*)peer_ptr(c, d, (size_t)a.srcinfo_off))[loff] = c.rank * (S * K) + s * K + lane;
      }
      for (int k = 0; k < K; ++k) {
        const int dv = __shfl_sync(0xffffffffu, dval, k);
        if (dv >= 0 && lane == 0) {
          const int d = dv / NvS, loff = dv - d * NvS;
          bulk_s2g(peer_ptr(c, d, c.off_hidden) + (size_t)loff * row_bytes, ring + (size_t)st * row_bytes, row_bytes);
          if (c.counters) atomicAdd(&s_peer[d], 1);
        }
      }
      if (lane == 0) bulk_commit();
    }
    if (lane == 0) trace_mark(c, MEP_K_DISPATCH, 2);
    zero_fill_work();
    if (lane == 0) { bulk_wait_all<0>(); fence_proxy_async(); trace_mark(c, MEP_K_DISPATCH, 3); }
  } else {
    zero_fill_work();
  }
  if (lane == 0 && warp == kSendWarps) trace_mark(c, MEP_K_DISPATCH, 4);
  cross_rank_barrier(c, nb, 1, MEP_K_DISPATCH, 30);
  if (c.counters) {
    if (tid < c.R && s_peer[tid]) {
      if (tid < 48) count(c, MEP_CNT_PEER_ROWS + tid, (unsigned long long)s_peer[tid]);
      count(c, MEP_CNT_ROWS_SENT, (unsigned long long)s_peer[tid]);
      if (tid != c.rank) count(c, MEP_CNT_ROWS_REMOTE, (unsigned long long)s_peer[tid]);
    }
    if (tid == 0 && blockIdx.x == 0) count(c, MEP_CNT_DISPATCHES, 1);
  }
  if (tid == 0) trace_mark(c, MEP_K_DISPATCH, 5);
  pdl_trigger();                               // the duplicate expansion may be scheduled while this grid drains
}

// ---------------------------------------------------------------------------------------
// dup_finalize: compact the per-source staging regions [R][cap] of this rank into the
// plan-owned dup_groups[NvS,3] / dup_loffs[NvS] / dup_counts[2] (order = source-rank major,
// then arrival order inside a source: a set, as in the reference).
struct DupFinalizeArgs { int32_t* dup_groups; int32_t* dup_loffs; int32_t* dup_counts; };
struct DupFinalizeArgsPack { DupFinalizeArgs a[MEP_MAX_VRANKS]; };

__global__ void dup_finalize_kernel(MepCtxPack P, DupFinalizeArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const DupFinalizeArgs& a = A.a[blockIdx.y];
  __shared__ int s_goff[MEP_MAX_RANKS + 1], s_loff[MEP_MAX_RANKS + 1];
  const int* cnt = (const int*)peer_ptr(c, c.rank, c.off_dupcnt);
  if (threadIdx.x == 0) {
    int g = 0, l = 0;
    for (int r = 0; r < c.R; ++r) { s_goff[r] = g; s_loff[r] = l; g += __ldcg(cnt + 2 * r); l += __ldcg(cnt + 2 * r + 1); }
    s_goff[c.R] = g; s_loff[c.R] = l;
    if (blockIdx.x == 0) { a.dup_counts[0] = g; a.dup_counts[1] = l; }
  }
  __syncthreads();
  const int* sg = (const int*)peer_ptr(c, c.rank, c.off_dupgroups);
  const int* sl = (const int*)peer_ptr(c, c.rank, c.off_duploffs);
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gnt = gridDim.x * blockDim.x;
  for (int r = 0; r < c.R; ++r) {
    const int ng = s_goff[r + 1] - s_goff[r], nl = s_loff[r + 1] - s_loff[r];
    for (int j = gtid; j < ng; j += gnt) {
      const int* src = sg + ((size_t)r * c.dup_group_cap + j) * 3;
      int* dstp = a.dup_groups + (size_t)(s_goff[r] + j) * 3;
      dstp[0] = __ldcg(src); dstp[1] = __ldcg(src + 1) + s_loff[r]; dstp[2] = __ldcg(src + 2);
    }
    for (int j = gtid; j < nl; j += gnt)
      a.dup_loffs[s_loff[r] + j] = __ldcg(sl + (size_t)r * c.dup_loff_cap + j);
  }
}

// ---------------------------------------------------------------------------------------
// dup_expand: copy each primary row of `buf` onto its duplicate rows (one warp per group).
struct DupArgs { __nv_bfloat16* buf; const int32_t* dup_groups; const int32_t* dup_loffs; const int32_t* dup_counts; };
struct DupArgsPack { DupArgs a[MEP_MAX_VRANKS]; };

__global__ void __launch_bounds__(256) dup_expand_kernel(MepCtxPack P, DupArgsPack A) {
  pdl_wait();                                // the plan tables and the rows come from the kernel before
  const MepRankCtx* cp = P.ctx[blockIdx.y];  // two fields only (see dup_reduce_kernel; checked mode: dup_check_kernel)
  const int NvS = cp->NvS;
  const DupArgs& a = A.a[blockIdx.y];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int ng = a.dup_counts[0];
  const size_t row_bytes = (size_t)cp->H * 2;
  const int nvec = (int)(row_bytes >> 4);
  char* base = (char*)a.buf;
  // a block copies one column part [vb, ve) of all groups (see dup_reduce_kernel)
  const int part = blockIdx.x % kDupParts, nsteps = (nvec + 127) >> 7;
  const int vb = (part * nsteps / kDupParts) << 7;
  int ve = ((part + 1) * nsteps / kDupParts) << 7; if (ve > nvec) ve = nvec;
  const int pgw = (blockIdx.x / kDupParts) * wpb + (threadIdx.x >> 5);
  const int pnw = ((gridDim.x - part + kDupParts - 1) / kDupParts) * wpb;
  for (int g = pgw; g < ng; g += pnw) {
    const int p = a.dup_groups[3 * g], st = a.dup_groups[3 * g + 1], n = a.dup_groups[3 * g + 2];
    if ((unsigned)p >= (unsigned)NvS || n <= 0 || n >= MEP_MAX_TOPK) continue;
    const char* src = base + (size_t)p * row_bytes;
    // duplicate offsets of this group live in lanes 0..n-1
    int myq = -1;
    if (lane < n) {
      myq = a.dup_loffs[st + lane];
      if ((unsigned)myq >= (unsigned)NvS) myq = -1;
    }
    for (int v0 = vb; v0 < ve; v0 += 128) {           // 4 x 16-byte loads in flight per lane
      int4 x[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) { const int v = v0 + j * 32 + lane; if (v < nvec) x[j] = ld_nc_v4(src + (size_t)v * 16); }
      for (int d = 0; d < n; ++d) {
        const int q = __shfl_sync(0xffffffffu, myq, d);
        if (q < 0) continue;
        char* drow = base + (size_t)q * row_bytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) { const int v = v0 + j * 32 + lane; if (v < nvec) st_na_v4(drow + (size_t)v * 16, x[j]); }
      }
    }
  }
}


// ---------------------------------------------------------------------------------------
// dup_expand_fresh: the two steps above in one launch for a fresh dispatch. Every CTA derives the
// per-source prefixes itself, all CTAs share the compaction into the plan-owned tables, and the
// expansion reads the groups straight from the staging regions.
struct DupFreshArgs { __nv_bfloat16* buf; int32_t* dup_groups; int32_t* dup_loffs; int32_t* dup_counts; };
struct DupFreshArgsPack { DupFreshArgs a[MEP_MAX_VRANKS]; };

__global__ void __launch_bounds__(256) dup_expand_fresh_kernel(MepCtxPack P, DupFreshArgsPack A) {
  pdl_wait();                                // the plan tables and the rows come from the kernel before
  const MepRankCtx c = *P.ctx[blockIdx.y];
  const DupFreshArgs& a = A.a[blockIdx.y];
  __shared__ int s_goff[MEP_MAX_RANKS + 1], s_loff[MEP_MAX_RANKS + 1];
  const int* cnt = (const int*)peer_ptr(c, c.rank, c.off_dupcnt);
  if (threadIdx.x == 0) {
    int g = 0, l = 0;
    for (int r = 0; r < c.R; ++r) { s_goff[r] = g; s_loff[r] = l; g += __ldcg(cnt + 2 * r); l += __ldcg(cnt + 2 * r + 1); }
    s_goff[c.R] = g; s_loff[c.R] = l;
    if (blockIdx.x == 0) { a.dup_counts[0] = g; a.dup_counts[1] = l; }
  }
  __syncthreads();
  const int* sg = (const int*)peer_ptr(c, c.rank, c.off_dupgroups);
  const int* sl = (const int*)peer_ptr(c, c.rank, c.off_duploffs);
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gnt = gridDim.x * blockDim.x;
  for (int r = 0; r < c.R; ++r) {
    const int ng = s_goff[r + 1] - s_goff[r], nl = s_loff[r + 1] - s_loff[r];
    for (int j = gtid; j < ng; j += gnt) {
      const int* src = sg + ((size_t)r * c.dup_group_cap + j) * 3;
      int* dstp = a.dup_groups + (size_t)(s_goff[r] + j) * 3;
      dstp[0] = __ldcg(src); dstp[1] = __ldcg(src + 1) + s_loff[r]; dstp[2] = __ldcg(src + 2);
    }
    for (int j = gtid; j < nl; j += gnt)
      a.dup_loffs[s_loff[r] + j] = __ldcg(sl + (size_t)r * c.dup_loff_cap + j);
  }
  // expansion, one warp per group, groups addressed through the staging regions
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int total = s_goff[c.R];
  const size_t row_bytes = (size_t)c.H * 2;
  const int nvec = (int)(row_bytes >> 4);
  char* base = (char*)a.buf;
  // a block copies one column part [vb, ve) of all groups (see dup_reduce_kernel)
  const int part = blockIdx.x % kDupParts, nsteps = (nvec + 127) >> 7;
  const int vb = (part * nsteps / kDupParts) << 7;
  int ve = ((part + 1) * nsteps / kDupParts) << 7; if (ve > nvec) ve = nvec;
  const int pgw = (blockIdx.x / kDupParts) * wpb + (threadIdx.x >> 5);
  const int pnw = ((gridDim.x - part + kDupParts - 1) / kDupParts) * wpb;
  for (int g = pgw; g < total; g += pnw) {
    int lo = 0, hi = c.R - 1;                         // source r with s_goff[r] <= g < s_goff[r+1]
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (s_goff[mid] <= g) lo = mid; else hi = mid - 1; }
    const int r = lo, j = g - s_goff[r];
    const int* grp = sg + ((size_t)r * c.dup_group_cap + j) * 3;
    const int p = __ldcg(grp), st = __ldcg(grp + 1), n = __ldcg(grp + 2);
    if ((unsigned)p >= (unsigned)c.NvS || n <= 0 || n >= MEP_MAX_TOPK) continue;
    const char* src = base + (size_t)p * row_bytes;
    int myq = -1;
    if (lane < n) { myq = __ldcg(sl + (size_t)r * c.dup_loff_cap + st + lane); if ((unsigned)myq >= (unsigned)c.NvS) myq = -1; }
    for (int v0 = vb; v0 < ve; v0 += 128) {
      int4 x[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) { const int v = v0 + jj * 32 + lane; if (v < nvec) x[jj] = ld_nc_v4(src + (size_t)v * 16); }
      for (int d = 0; d < n; ++d) {
        const int q = __shfl_sync(0xffffffffu, myq, d);
        if (q < 0) continue;
        char* drow = base + (size_t)q * row_bytes;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) { const int v = v0 + jj * 32 + lane; if (v < nvec) st_na_v4(drow + (size_t)v * 16, x[jj]); }
      }
    }
  }
}

}  // namespace mep

extern "C" int mep_dispatch_smem_stages(int H, int* stages_out, size_t* smem_out) {
  const size_t row = (size_t)H * 2;
  const size_t budget = 180 * 1024;
  int stages = (int)(budget / (row * mep::kSendWarps));
  if (stages > mep::kMaxStages) stages = mep::kMaxStages;
  MEP_REQUIRE(stages >= 1, "dispatch: H=%d rows (%zu B) do not fit the shared-memory ring", H, row);
  *stages_out = stages; *smem_out = row * mep::kSendWarps * stages;
  return 0;
}

extern "C" int mep_launch_dispatch(int nv, const MepRankCtx* const* ctxs, const mep::DispatchArgs* args,
                                   int num_sms, int H, int epn, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "dispatch: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::DispatchArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  int stages; size_t smem;
  if (mep_dispatch_smem_stages(H, &stages, &smem)) return -1;
  smem += (size_t)(4 * epn + 2) * sizeof(int);      // padding-row tables behind the rings
  smem += (size_t)mep::kSendWarps * 2 * mep::kMetaTokens * MEP_MAX_TOPK * sizeof(int);   // per-warp plan staging
  MEP_REQUIRE(smem <= 226 * 1024, "dispatch: epn=%d padding tables do not fit shared memory", epn);
  return mep::launch_cooperative(mep::dispatch_kernel, dim3(num_sms, nv), dim3(mep::kDispThreads), smem,
                                 stream, false, P, A, stages);
}

extern "C" int mep_launch_dup_finalize(int nv, const MepRankCtx* const* ctxs, const mep::DupFinalizeArgs* args,
                                       cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupFinalizeArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain(mep::dup_finalize_kernel, dim3(8, nv), dim3(256), 0, stream, P, A);
}

extern "C" int mep_launch_dup_expand(int nv, const MepRankCtx* const* ctxs, const mep::DupArgs* args,
                                     int num_blocks, int pdl, cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain_pdl(mep::dup_expand_kernel, dim3(mep::dup_grid(num_blocks), nv), dim3(256), 0, stream, pdl != 0, P, A);
}

extern "C" int mep_launch_dup_expand_fresh(int nv, const MepRankCtx* const* ctxs, const mep::DupFreshArgs* args,
                                           int num_blocks, int pdl, cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupFreshArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain_pdl(mep::dup_expand_fresh_kernel, dim3(mep::dup_grid(num_blocks), nv), dim3(256), 0, stream, pdl != 0, P, A);
}

MEP_EXPORT_SIZEOF(DispatchArgs, mep::DispatchArgs)
MEP_EXPORT_SIZEOF(DupFinalizeArgs, mep::DupFinalizeArgs)
MEP_EXPORT_SIZEOF(DupArgs, mep::DupArgs)
MEP_EXPORT_SIZEOF(DupFreshArgs, mep::DupFreshArgs)
