// Combine: local duplicate pre-reduction, fused unpermute + K-sum over peers, and the
// stand-alone rank sync.
//
// Counterpart of the reference's CombinePrologueKernel (moonep/combine_prologue.py:41-484),
// CombineKernel (moonep/combine.py:40-511) and InterRankSyncKernel
// (moonep/inter_rank_sync.py:22-83). Semantics kept: combine is an UNWEIGHTED sum of a
// token's rows; duplicates of one destination rank are summed in fp32 and rounded to bf16
// once into the primary row, the per-rank partial sums are then added in fp32 (ascending k)
// and rounded once; the optional [S,K] channel gathers the per-slot fp32 route weights back
// bit-exactly. Peer rows are pulled by a producer warp with plain (single-CTA) bulk copies into a
// shared-memory ring and summed by consumer warps.
#include "prims.cuh"
#include "../host/launch.h"
#include <stdlib.h>

namespace mep {

__device__ __forceinline__ void acc_bf16x8(float* acc, const int4& x) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
}
__device__ __forceinline__ int4 pack_bf16x8(const float* acc) {
  int4 o; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}


// Sum `np` bf16 rows (row pointers held by the lanes flagged in `prim`, ascending lane order)
// into one bf16 row. PB rows x CB 16-byte column chunks are loaded per lane before any add, so
// PB*CB loads are in flight per lane whatever the number of rows; fp32 accumulation, one
// rounding. `PEER` selects loads that bypass L1 for rows other GPUs may have written.
template <int PB, int CB, bool PEER>
__device__ __forceinline__ void reduce_rows(const char* myrow, unsigned prim, int np, char* orow, int nvec, int lane) {
  for (int v0 = 0; v0 < nvec; v0 += 32 * CB) {
    float acc[CB][8];
#pragma unroll
    for (int cx = 0; cx < CB; ++cx)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[cx][i] = 0.f;
    unsigned rest = prim;
    for (int j0 = 0; j0 < np; j0 += PB) {
      int4 x[PB][CB];
#pragma unroll
      for (int j = 0; j < PB; ++j) {
        const bool on = j0 + j < np;
        const int src = on ? __ffs(rest) - 1 : 0;
        if (on) rest &= rest - 1;
        const char* rp = (const char*)__shfl_sync(0xffffffffu, (unsigned long long)myrow, src);
#pragma unroll
        for (int cx = 0; cx < CB; ++cx) {
          const int v = v0 + cx * 32 + lane;
          x[j][cx] = make_int4(0, 0, 0, 0);
          if (on && v < nvec) x[j][cx] = PEER ? ld_peer_v4(rp + (size_t)v * 16) : ld_nc_v4(rp + (size_t)v * 16);
        }
      }
#pragma unroll
      for (int j = 0; j < PB; ++j)
#pragma unroll
        for (int cx = 0; cx < CB; ++cx) acc_bf16x8(acc[cx], x[j][cx]);
    }
#pragma unroll
    for (int cx = 0; cx < CB; ++cx) {
      const int v = v0 + cx * 32 + lane;
      if (v < nvec) st_na_v4(orow + (size_t)v * 16, pack_bf16x8(acc[cx]));
    }
  }
}

template <bool PEER>
__device__ __forceinline__ void reduce_rows_auto(const char* myrow, unsigned prim, int np, char* orow, int nvec, int lane) {
  if (np <= 2) reduce_rows<2, 4, PEER>(myrow, prim, np, orow, nvec, lane);
  else if (np <= 4) reduce_rows<4, 2, PEER>(myrow, prim, np, orow, nvec, lane);
  else reduce_rows<8, 1, PEER>(myrow, prim, np, orow, nvec, lane);
}

// ------------------------------------------------------------------ dup_reduce
struct DupArgs { __nv_bfloat16* buf; const int32_t* dup_groups; const int32_t* dup_loffs; const int32_t* dup_counts; };
struct DupArgsPack { DupArgs a[MEP_MAX_VRANKS]; };

__global__ void __launch_bounds__(256) dup_reduce_kernel(MepCtxPack P, DupArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const DupArgs& a = A.a[blockIdx.y];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5), nw = gridDim.x * wpb;
  const int ng = a.dup_counts[0];
  const size_t row_bytes = (size_t)c.H * 2;
  const int nvec = (int)(row_bytes >> 4);
  char* base = (char*)a.buf;
  for (int g = gw; g < ng; g += nw) {
    const int p = a.dup_groups[3 * g], st = a.dup_groups[3 * g + 1], n = a.dup_groups[3 * g + 2];
    if ((unsigned)p >= (unsigned)c.NvS || n <= 0 || n >= MEP_MAX_TOPK) continue;
    // lane 0 holds the primary row, lanes 1..n the duplicates in table order
    const char* myrow = nullptr;
    if (lane == 0) myrow = base + (size_t)p * row_bytes;
    else if (lane <= n) {
      const int q = a.dup_loffs[st + lane - 1];
      if ((unsigned)q < (unsigned)c.NvS) myrow = base + (size_t)q * row_bytes;
    }
    const unsigned rows = __ballot_sync(0xffffffffu, myrow != nullptr);
    reduce_rows_auto<false>(myrow, rows, __popc(rows), base + (size_t)p * row_bytes, nvec, lane);
  }
}

// ------------------------------------------------------------------ combine
struct CombineArgs {
  const int32_t* dst;       // [N] plan
  __nv_bfloat16* out;       // [S, H]
  float* out_weights;       // [S, K] or null
  int32_t entry_barrier;    // cross-rank barrier before the first peer read (normally 1)
};
struct CombineArgsPack { CombineArgs a[MEP_MAX_VRANKS]; };

constexpr int kCombConsumers = 128;                 // 4 accumulate warps
constexpr int kCombThreads = 32 + kCombConsumers + 32;   // + producer warp + route-weight gather warp
constexpr int kCombMaxStages = 16;
constexpr int kCombSegVecs = 1024;                  // a stage holds at most 16 KB of one row
constexpr int kCombMetaTokens = 128;                // tokens whose plan entries are staged at once

// One producer warp keeps up to `stages` row segments in flight with bulk copies (peer or local
// memory -> this CTA's shared memory ring); four consumer warps add the arriving rows of a token
// in fp32 registers (ascending k) and write the bf16 result once. In-flight data lives in shared
// memory, so the bytes outstanding per SM are not limited by registers.
__global__ void __launch_bounds__(kCombThreads, 1)
combine_kernel(MepCtxPack P, CombineArgsPack A, int stages, int nseg, int seg_vecs, int dbg) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const CombineArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kCombMaxStages], empty_bar[kCombMaxStages];
  __shared__ int s_tok[kCombMaxStages], s_meta[kCombMaxStages];   // meta: seg << 2 | last << 1 | sentinel
  __shared__ volatile int s_abort;
  __shared__ long long s_tp[64], s_tc[64], s_td[64];
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = c.K, S = c.S, NvS = c.NvS;
  const size_t row_bytes = (size_t)c.H * 2;
  const int nvec = (int)(row_bytes >> 4);
  const size_t seg_bytes = (size_t)seg_vecs * 16;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < kCombMaxStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], kCombConsumers / 32); }
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 1);
  if (a.entry_barrier) { if (!cross_rank_barrier(c, nb, 2, MEP_K_COMBINE, 10)) return; }
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 2);

  if (warp == 0) {
    // ---------------- producer
    int it = 0;
    long long dbg_wait = 0, dbg_issue = 0; const long long dbg_t0 = clock64();
    // plan entries are staged in shared memory one chunk of tokens at a time (all loads of a
    // chunk in flight together), so no global-memory latency sits between two row copies
    int* s_dst = reinterpret_cast<int*>(smem + (size_t)stages * seg_bytes);
    const int ntok = blockIdx.x < S ? (S - blockIdx.x + nb - 1) / nb : 0;
    for (int t = 0; t < ntok && !s_abort; ++t) {
      const int s = blockIdx.x + t * nb;
      if ((t % kCombMetaTokens) == 0) {
        const int cnt = (ntok - t < kCombMetaTokens ? ntok - t : kCombMetaTokens) * K;
        __syncwarp();
        for (int i = lane; i < cnt; i += 32) {
          const int tt = i / K, k = i - tt * K;
          s_dst[i] = a.dst[((size_t)blockIdx.x + (size_t)(t + tt) * nb) * K + k];
        }
        __syncwarp();
      }
      const int dval = lane < K ? s_dst[(t % kCombMetaTokens) * K + lane] : -1;
      const char* myrow = nullptr;
      if (lane < K && dval >= 0) {
        const int d = dval / NvS, loff = dval - d * NvS;
        myrow = peer_ptr(c, d, c.off_hidden) + (size_t)loff * row_bytes;
      }
      const unsigned prim = __ballot_sync(0xffffffffu, myrow != nullptr);
      const int np = __popc(prim);
      for (int sg = 0; sg < nseg; ++sg) {
        const int v_beg = sg * seg_vecs;
        const uint32_t bytes = (uint32_t)((nvec - v_beg < seg_vecs ? nvec - v_beg : seg_vecs) * 16);
        unsigned rest = prim;
        for (int j = 0; j < np; ++j, ++it) {
          const int src = __ffs(rest) - 1; rest &= rest - 1;
          const char* rp = (const char*)__shfl_sync(0xffffffffu, (unsigned long long)myrow, src);
          const int st = it % stages; const uint32_t ph = (uint32_t)(it / stages) & 1u;
          int ok = 1;
          if (lane == 0) {
            const long long tw0 = clock64();
            ok = mbar_wait_bounded(&empty_bar[st], ph ^ 1u, c.wait_budget_ns) ? 1 : 0;
            dbg_wait += clock64() - tw0;
            if (ok) {
              const long long ti0 = clock64();
              s_tok[st] = s; s_meta[st] = (sg << 2) | ((j == np - 1) ? 2 : 0);
              mbar_expect_tx(&full_bar[st], (dbg & 4) ? 1024u : bytes);
              bulk_g2s(smem + (size_t)st * seg_bytes, rp + (size_t)v_beg * 16, (dbg & 4) ? 1024u : bytes, &full_bar[st]);
              dbg_issue += clock64() - ti0;
              if (it < 64) s_tp[it] = clock64();
            } else { report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_COMBINE, 20, s, 0, 0); s_abort = 1; }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (s_abort) break;
      }
    }
    // sentinel stage: tells the consumers that no more rows follow
    if (lane == 0 && !s_abort) {
      const int st = it % stages; const uint32_t ph = (uint32_t)(it / stages) & 1u;
      if (mbar_wait_bounded(&empty_bar[st], ph ^ 1u, c.wait_budget_ns)) { s_meta[st] = 1; mbar_arrive(&full_bar[st]); }
      else { report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_COMBINE, 21, -1, 0, 0); s_abort = 1; }
      trace_mark(c, MEP_K_COMBINE, 3);
      trace_value(c, MEP_K_COMBINE, 20, (unsigned long long)dbg_wait);
      trace_value(c, MEP_K_COMBINE, 24, (unsigned long long)dbg_issue);
      trace_value(c, MEP_K_COMBINE, 21, (unsigned long long)(clock64() - dbg_t0));
    }
  } else if (warp == kCombThreads / 32 - 1) {
    // ---------------- route-weight gather: [S, K] fp32 pulled from the slots' owners
    if (a.out_weights) {
      const int ntok = blockIdx.x < S ? (S - blockIdx.x + nb - 1) / nb : 0;
      const int total = ntok * K;
      for (int i0 = 0; i0 < total; i0 += 128) {
        float w[4]; long long pos[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 32 + lane;
          pos[u] = -1; w[u] = 0.f;
          if (i < total) {
            const int t = i / K, k = i - t * K;
            pos[u] = ((long long)blockIdx.x + (long long)t * nb) * K + k;
            const int dv = a.dst[pos[u]];
            const int raw = dv >= 0 ? dv : -dv - 1;
            const int d = raw / NvS, loff = raw - d * NvS;
            w[u] = __ldcg((const float*)peer_ptr(c, d, c.off_weights) + loff);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) if (pos[u] >= 0) a.out_weights[pos[u]] = w[u];
      }
    }
    if (lane == 0) trace_mark(c, MEP_K_COMBINE, 5);
  } else {
    // ---------------- consumers
    const int ct = tid - 32;
    float acc[8][8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[q][i] = 0.f;
    long long dbg_cw = 0; const long long dbg_c0 = clock64();
    for (int it = 0; !s_abort; ++it) {
      const int st = it % stages; const uint32_t ph = (uint32_t)(it / stages) & 1u;
      int ok = 1;
      const long long tw0 = clock64();
      if (lane == 0) ok = mbar_wait_bounded(&full_bar[st], ph, c.wait_budget_ns) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      dbg_cw += clock64() - tw0;
      if (it < 64 && tid == 32) s_tc[it] = clock64();
      if (!ok) { if (lane == 0) { report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_COMBINE, 22, it, 0, 0); s_abort = 1; } break; }
      const int meta = s_meta[st];
      if (meta & 1) break;
      const int sg = meta >> 2, v_beg = sg * seg_vecs;
      const int len = nvec - v_beg < seg_vecs ? nvec - v_beg : seg_vecs;
      const unsigned char* stage = smem + (size_t)st * seg_bytes;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = ct + q * kCombConsumers;
        if (v < len && !(dbg & 2)) acc_bf16x8(acc[q], *reinterpret_cast<const int4*>(stage + (size_t)v * 16));
      }
      if (meta & 2) {
        char* orow = (char*)a.out + (size_t)s_tok[st] * row_bytes + (size_t)v_beg * 16;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int v = ct + q * kCombConsumers;
          if (v < len && !(dbg & 1)) st_na_v4(orow + (size_t)v * 16, pack_bf16x8(acc[q]));
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[q][i] = 0.f;
        }
      }
      __syncwarp();
      if (it < 64 && tid == 32) s_td[it] = clock64();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
    }
    if (lane == 0) { trace_mark(c, MEP_K_COMBINE, 4); trace_value(c, MEP_K_COMBINE, 22, (unsigned long long)dbg_cw); trace_value(c, MEP_K_COMBINE, 23, (unsigned long long)(clock64() - dbg_c0)); }
  }
  __syncthreads();
  if (blockIdx.x == 0 && tid == 0 && c.trace) {
    for (int i = 0; i < 64; ++i) { trace_value(c, MEP_K_COMBINE, 30, (unsigned long long)(s_tp[i] - s_tp[0])); trace_value(c, MEP_K_COMBINE, 31, (unsigned long long)(s_tc[i] - s_tp[0])); trace_value(c, MEP_K_COMBINE, 32, (unsigned long long)(s_td[i] - s_tp[0])); }
  }
}

// ------------------------------------------------------------------ stand-alone rank sync
__global__ void rank_sync_kernel(MepCtxPack P) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  if (c.R > 1) cross_rank_arrive_wait(c, 3, MEP_K_SYNC, 1);
}

// ------------------------------------------------------------------ bounded-wait self test
// Waits on a flag that only the host could set; with nobody setting it the wait must give
// up after the Buffer's budget, record MEP_ERR_FLAG_TIMEOUT and return normally.
__global__ void wait_probe_kernel(MepCtxPack P, const uint32_t* flag, uint32_t expected) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  if (threadIdx.x == 0) {
    uint32_t seen = 0;
    const bool ok = bounded_wait(c, [&] { seen = ld_acquire_sys(flag); return seen == expected; });
    if (!ok) report(c, MEP_ERR_FLAG_TIMEOUT, MEP_K_WAIT_PROBE, 1, -1, seen, expected);
  }
}

}  // namespace mep

extern "C" int mep_launch_dup_reduce(int nv, const MepRankCtx* const* ctxs, const mep::DupArgs* args,
                                     int num_blocks, cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain(mep::dup_reduce_kernel, dim3(num_blocks, nv), dim3(256), 0, stream, P, A);
}

extern "C" int mep_launch_combine(int nv, const MepRankCtx* const* ctxs, const mep::CombineArgs* args,
                                  int num_sms, int H, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "combine: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::CombineArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  const int nvec = H / 8;
  const int nseg = (nvec + mep::kCombSegVecs - 1) / mep::kCombSegVecs;
  const int seg_vecs = (nvec + nseg - 1) / nseg;
  const size_t meta = (size_t)mep::kCombMetaTokens * MEP_MAX_TOPK * sizeof(int);
  int stages = (int)((200 * 1024 - meta) / ((size_t)seg_vecs * 16));
  if (stages > mep::kCombMaxStages) stages = mep::kCombMaxStages;
  MEP_REQUIRE(stages >= 2, "combine: H=%d does not fit the shared-memory ring", H);
  const size_t smem = (size_t)stages * seg_vecs * 16 + meta;
  return mep::launch_cooperative(mep::combine_kernel, dim3(num_sms, nv), dim3(mep::kCombThreads), smem,
                                 stream, false, P, A, stages, nseg, seg_vecs, getenv("MEP_DBG_COMBINE") ? atoi(getenv("MEP_DBG_COMBINE")) : 0);
}

extern "C" int mep_launch_rank_sync(int nv, const MepRankCtx* const* ctxs, cudaStream_t stream) {
  MepCtxPack P = {};
  for (int i = 0; i < nv; ++i) P.ctx[i] = ctxs[i];
  return mep::launch_cooperative(mep::rank_sync_kernel, dim3(1, nv), dim3(128), 0, stream, false, P);
}

extern "C" int mep_launch_wait_probe(const MepRankCtx* ctx, const uint32_t* flag, uint32_t expected,
                                     cudaStream_t stream) {
  MepCtxPack P = {}; P.ctx[0] = ctx;
  return mep::launch_plain(mep::wait_probe_kernel, dim3(1, 1), dim3(32), 0, stream, P, flag, expected);
}
