// Combine: local duplicate pre-reduction, fused unpermute + K-sum over peers, and the
// stand-alone rank sync.
//
// Counterpart of the reference's CombinePrologueKernel (moonep/combine_prologue.py:41-484),
// CombineKernel (moonep/combine.py:40-511) and InterRankSyncKernel
// (moonep/inter_rank_sync.py:22-83). Semantics kept: combine is an UNWEIGHTED sum of a
// token's rows; duplicates of one destination rank are summed in fp32 and rounded to bf16
// once into the primary row, the per-rank partial sums are then added in fp32 (ascending k)
// and rounded once; the optional [S,K] channel gathers the per-slot fp32 route weights back
// bit-exactly. Peer rows are pulled with untiled bulk copies into shared memory
// (see combine_kernel).
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

// Checked mode (MOONEP_CHECKED=1): a pass of its own over the duplicate tables that reports entries the
// expansion / reduction kernels skip silently. A separate kernel on purpose: with the report inside
// dup_reduce_kernel, that kernel went from 56 to 92-98 registers and lost a third of its throughput.
__global__ void __launch_bounds__(256) dup_check_kernel(MepCtxPack P, DupArgsPack A, int kernel_id) {
  const MepRankCtx* cp = P.ctx[blockIdx.y];
  const DupArgs& a = A.a[blockIdx.y];
  const int NvS = cp->NvS, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5), nw = gridDim.x * wpb;
  const int ng = a.dup_counts[0];
  for (int g = gw; g < ng; g += nw) {
    const int p = a.dup_groups[3 * g], st = a.dup_groups[3 * g + 1], n = a.dup_groups[3 * g + 2];
    const bool bad_head = (unsigned)p >= (unsigned)NvS || n <= 0 || n >= MEP_MAX_TOPK;
    int q = 0;
    if (!bad_head && lane < n) q = a.dup_loffs[st + lane];
    if (bad_head) { if (lane == 0) report(*cp, MEP_ERR_BOUNDS, kernel_id, 1, g, (uint32_t)p, (uint32_t)n); }
    else if ((unsigned)q >= (unsigned)NvS) report(*cp, MEP_ERR_BOUNDS, kernel_id, 2, g, (uint32_t)q, (uint32_t)NvS);
  }
}

__global__ void __launch_bounds__(256) dup_reduce_kernel(MepCtxPack P, DupArgsPack A) {
  const MepRankCtx* cp = P.ctx[blockIdx.y];   // two fields only: no need to copy the whole context
  const int NvS = cp->NvS;
  const DupArgs& a = A.a[blockIdx.y];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int ng = a.dup_counts[0];
  const size_t row_bytes = (size_t)cp->H * 2;
  const int nvec = (int)(row_bytes >> 4);
  char* base = (char*)a.buf;
  // Every row is split into kDupParts column parts (runs of whole 128-vector steps) and a block works on
  // one part of all groups: with one warp per whole group a launch has only two or three groups per warp,
  // and the warps with one group more set the time.
  const int part = blockIdx.x % kDupParts, nsteps = (nvec + 127) >> 7;
  const int vb = (part * nsteps / kDupParts) << 7;
  int ve = ((part + 1) * nsteps / kDupParts) << 7; if (ve > nvec) ve = nvec;
  if (vb >= ve) { pdl_trigger(); return; }
  const int pgw = (blockIdx.x / kDupParts) * wpb + (threadIdx.x >> 5);
  const int pnw = ((gridDim.x - part + kDupParts - 1) / kDupParts) * wpb;
  for (int g = pgw; g < ng; g += pnw) {
    const int p = a.dup_groups[3 * g], st = a.dup_groups[3 * g + 1], n = a.dup_groups[3 * g + 2];
    if ((unsigned)p >= (unsigned)NvS || n <= 0 || n >= MEP_MAX_TOPK) continue;
    // lane 0 holds the primary row, lanes 1..n the duplicates in table order
    const char* myrow = nullptr;
    if (lane == 0) myrow = base + (size_t)p * row_bytes + (size_t)vb * 16;
    else if (lane <= n) {
      const int q = a.dup_loffs[st + lane - 1];
      if ((unsigned)q < (unsigned)NvS) myrow = base + (size_t)q * row_bytes + (size_t)vb * 16;
    }
    const unsigned rows = __ballot_sync(0xffffffffu, myrow != nullptr);
    reduce_rows_auto<false>(myrow, rows, __popc(rows), base + (size_t)p * row_bytes + (size_t)vb * 16, ve - vb, lane);
  }
  pdl_trigger();                               // the combine may be scheduled while this grid drains
}

// ------------------------------------------------------------------ combine
struct CombineArgs {
  const int32_t* dst;       // [N] plan
  __nv_bfloat16* out;       // [S, H]
  float* out_weights;       // [S, K] or null
  int32_t entry_barrier;    // cross-rank barrier before the first peer read (normally 1)
};
struct CombineArgsPack { CombineArgs a[MEP_MAX_VRANKS]; };

constexpr int kCombWarps = 14;
constexpr int kCombThreads = kCombWarps * 32;
constexpr int kCombSlots = 32;                      // 16-byte vectors per lane in one warp stage (16 KB per warp)

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Each warp owns a 16 KB shared-memory stage and walks its tokens: for a token with np rows it
// fetches, per pass, floor(16/np) 16-byte vectors per lane from EVERY row -- one untiled bulk copy per
// row (peer or local memory -> shared memory, issued by the warp's first lane, completion on a barrier
// of the stage half; no multicast, no tensor map) -- into one half of the stage while the other half
// is summed: the rows are added in fp32 (ascending k) and the bf16 result is stored.
// A token with more than 16 rows takes the unpipelined path (one 16-byte asynchronous copy per lane
// and vector into the whole stage). With 14 warps per CTA up to 224 KB per SM are in flight.
__global__ void __launch_bounds__(kCombThreads, 1) combine_kernel(MepCtxPack P, CombineArgsPack A) {
  pdl_wait();                                // rows of this shard were pre-reduced by the kernel before
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const CombineArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) unsigned char smem[];
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = c.K, S = c.S, NvS = c.NvS;
  const size_t row_bytes = (size_t)c.H * 2;
  const int nvec = (int)(row_bytes >> 4);
  const int vpl = (nvec + 31) >> 5;                  // vectors per lane in a full row

  __shared__ __align__(8) uint64_t s_cbar[kCombWarps * 2];     // one barrier per warp and stage half
  if (tid < kCombWarps * 2) mbar_init(&s_cbar[tid], 1);
  fence_mbar_init();
  __syncthreads();
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 1);
  if (a.entry_barrier) { if (!cross_rank_barrier(c, nb, 2, MEP_K_COMBINE, 10)) return; }
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 2);

  if (tid == 0 && blockIdx.x == 0) count(c, MEP_CNT_COMBINES, 1);
  int pulled = 0;
  const uint32_t stage = smem_u32(smem) + (uint32_t)warp * (kCombSlots * 32 * 16);
  unsigned char* stage_g = smem + (size_t)warp * (kCombSlots * 32 * 16);
  uint64_t* bars = s_cbar + warp * 2;
  uint32_t half_phase = 0;                   // parity of the two halves' barriers
  // A token's K table entries as one lane each sees them. They are fetched one token ahead (the route
  // weight comes from the peer, a full NVLink round trip), and the first pass of the next token is issued
  // before the last pass of this one is summed, so a warp always has copies outstanding.
  struct Tok { int dval; const char* myrow; float w; int bad; };
  auto fetch = [&](int s) {
    Tok t; t.dval = -1; t.myrow = nullptr; t.w = 0.f; t.bad = 0;
    if (s < S && lane < K) {
      t.dval = a.dst[(size_t)s * K + lane];
      const int raw = t.dval >= 0 ? t.dval : -t.dval - 1;
      const int d = raw / NvS, loff = raw - d * NvS;
      if (d >= c.R) t.bad = raw + 1;      // corrupt or foreign plan: form no address from the entry
      else {
        if (a.out_weights) t.w = __ldcg((const float*)peer_ptr(c, d, c.off_weights) + loff);
        if (t.dval >= 0) t.myrow = peer_ptr(c, d, c.off_hidden) + (size_t)loff * row_bytes;
      }
    }
    return t;
  };
  // One pass moves `per` 16-byte vectors per lane from EVERY row of the token into the warp's stage,
  // then sums them. With up to kCombSlots / 2 rows the stage is split in two halves and the next pass
  // is already in flight while this one is summed.
  struct Shape { unsigned prim; int np, per, npass; bool pipelined; };
  auto shape_of = [&](const Tok& t) {
    Shape h; h.prim = __ballot_sync(0xffffffffu, t.myrow != nullptr); h.np = __popc(h.prim);
    h.pipelined = h.np > 0 && h.np <= kCombSlots / 2;
    h.per = h.np ? (h.pipelined ? kCombSlots / 2 : kCombSlots) / h.np : 1;
    if (h.per > vpl) h.per = vpl;
    h.npass = (vpl + h.per - 1) / h.per;
    return h;
  };
  unsigned pending = 0;                      // halves with a bulk copy issued and not yet waited for
  // pipelined pass p of a token into half h: one bulk copy per row -- this pass's share of a row is
  // contiguous there and in the stage
  auto issue_bulk = [&](const Tok& t, const Shape& sh, int p, int h) {
    const int j0 = p * sh.per, nj = vpl - j0 < sh.per ? vpl - j0 : sh.per;
    const size_t b0 = (size_t)j0 * 512;
    const uint32_t bytes = (uint32_t)(row_bytes - b0 < (size_t)nj * 512 ? row_bytes - b0 : (size_t)nj * 512);
    __syncwarp();                            // every lane has finished reading the half that is refilled now
    if (lane == 0) mbar_expect_tx(&bars[h], bytes * (uint32_t)sh.np);
    unsigned rest = sh.prim;
    for (int r = 0; r < sh.np; ++r) {
      const int src = __ffs(rest) - 1; rest &= rest - 1;
      const char* rp = (const char*)__shfl_sync(0xffffffffu, (unsigned long long)t.myrow, src);
      if (lane == 0)
        bulk_g2s(stage_g + (size_t)h * (kCombSlots / 2 * 32 * 16) + (size_t)r * sh.per * 512, rp + b0, bytes, &bars[h]);
    }
    pending |= 1u << h;
  };
  auto consume = [&](const Shape& sh, int p, const unsigned char* base, char* orow) {
    const int j0 = p * sh.per, nj = vpl - j0 < sh.per ? vpl - j0 : sh.per;
    for (int j = 0; j < nj; ++j) {
      const int v = (j0 + j) * 32 + lane;
      if (v >= nvec) continue;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < sh.np; ++r)
        acc_bf16x8(acc, *reinterpret_cast<const int4*>(base + (size_t)((r * sh.per + j) * 32 + lane) * 16));
      st_na_v4(orow + (size_t)v * 16, pack_bf16x8(acc));
    }
  };
  const int stride = nb * kCombWarps;
  int s = blockIdx.x * kCombWarps + warp;
  Tok cur = fetch(s);
  Shape cs = shape_of(cur);
  uint32_t q = 0;                            // passes waited for so far: the next one sits in half q & 1
  bool cur_issued = false, ok = true;
  if (s < S && cs.pipelined) { issue_bulk(cur, cs, 0, 0); cur_issued = true; }
  for (; s < S && ok; s += stride) {
    const int sn = s + stride;
    const Tok nxt = fetch(sn);
    const Shape nsh = shape_of(nxt);
    bool nxt_issued = false;
    if (lane < K) {
      if (cur.bad) {
        report(c, MEP_ERR_BOUNDS, MEP_K_COMBINE, 20, s, (uint32_t)(cur.bad - 1), (uint32_t)(c.R * NvS));
        if (a.out_weights) a.out_weights[(size_t)s * K + lane] = 0.f;
      } else if (a.out_weights) a.out_weights[(size_t)s * K + lane] = cur.w;
    }
    char* orow = (char*)a.out + (size_t)s * row_bytes;
    pulled += cs.np;
    if (cs.np == 0) {         // no valid primary row (only possible with a corrupt plan): the token's output is zero
      if (lane == 0) report(c, MEP_ERR_BOUNDS, MEP_K_COMBINE, 21, s, 0u, (uint32_t)K);
      for (int v = lane; v < nvec; v += 32) st_na_v4(orow + (size_t)v * 16, make_int4(0, 0, 0, 0));
    } else if (!cs.pipelined) {
      // more than kCombSlots / 2 rows: whole stage per pass, one 16-byte asynchronous copy per lane and vector
      for (int p = 0; p < cs.npass; ++p) {
        const int j0 = p * cs.per, nj = vpl - j0 < cs.per ? vpl - j0 : cs.per;
        unsigned rest = cs.prim;
        for (int r = 0; r < cs.np; ++r) {
          const int src = __ffs(rest) - 1; rest &= rest - 1;
          const char* rp = (const char*)__shfl_sync(0xffffffffu, (unsigned long long)cur.myrow, src);
          for (int j = 0; j < nj; ++j) {
            const int v = (j0 + j) * 32 + lane;
            if (v < nvec) cp_async16(stage + (uint32_t)((r * cs.per + j) * 32 + lane) * 16, rp + (size_t)v * 16);
          }
        }
        cp_async_commit_wait_all();
        consume(cs, p, stage_g, orow);
      }
    } else {
      if (!cur_issued) issue_bulk(cur, cs, 0, q & 1);
      for (int p = 0; p < cs.npass; ++p) {
        const int h = q & 1;
        if (p + 1 < cs.npass) issue_bulk(cur, cs, p + 1, h ^ 1);
        else if (sn < S && nsh.pipelined) { issue_bulk(nxt, nsh, 0, h ^ 1); nxt_issued = true; }
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[h], (half_phase >> h) & 1u, c.wait_budget_ns))) {
          if (lane == 0) report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_COMBINE, 22, s, (uint32_t)p, 0);
          ok = false; break;
        }
        half_phase ^= 1u << h; pending &= ~(1u << h);
        consume(cs, p, stage_g + (size_t)h * (kCombSlots / 2 * 32 * 16), orow);
        ++q;
      }
    }
    cur = nxt; cs = nsh; cur_issued = nxt_issued;
  }
  if (!ok) {                  // a copy never arrived: give the other one its time too before the stage goes away
    for (int h = 0; h < 2; ++h)
      if (((pending >> h) & 1u) && h != (int)(q & 1)) mbar_wait_bounded(&bars[h], (half_phase >> h) & 1u, c.wait_budget_ns);
  }
  if (lane == 0 && pulled) count(c, MEP_CNT_ROWS_PULLED, (unsigned long long)pulled);
}

// ------------------------------------------------------------------ push-combine: local reduction
// Counterpart of the combine for the "push" path: the down-projection GEMM's epilogue has already
// stored every row into its source rank's receive area [S*K, H] (row s*K + k = contribution of
// the token's k-th expert), so once all ranks have finished (entry barrier) the combine is a purely
// local sum over k (ascending, fp32) -- no peer reads, no duplicate pre-reduction.
struct PushReduceArgs {
  __nv_bfloat16* out;       // [S, H]
  float* out_weights;       // [S, K] or null: copy of the pushed per-slot values
  int64_t push_off;         // byte offsets of the receive areas inside this rank's chunk
  int64_t pushw_off;
};
struct PushReduceArgsPack { PushReduceArgs a[MEP_MAX_VRANKS]; };

__global__ void __launch_bounds__(256) push_reduce_kernel(MepCtxPack P, PushReduceArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];
  const PushReduceArgs& a = A.a[blockIdx.y];
  const int nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const int K = c.K, S = c.S;
  const size_t row_bytes = (size_t)c.H * 2;
  const int nvec = (int)(row_bytes >> 4);
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 11);
  if (!cross_rank_barrier(c, nb, 2, MEP_K_COMBINE, 40)) return;
  if (tid == 0) trace_mark(c, MEP_K_COMBINE, 12);
  const char* recv = peer_ptr(c, c.rank, (size_t)a.push_off);
  for (int s = blockIdx.x * nwarp + warp; s < S; s += nb * nwarp) {
    const char* base = recv + (size_t)s * K * row_bytes;
    char* orow = (char*)a.out + (size_t)s * row_bytes;
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k0 = 0; k0 < K; k0 += 8) {        // eight independent 16-byte loads in flight per lane
        int4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (k0 + j < K) x[j] = __ldcg(reinterpret_cast<const int4*>(base + (size_t)(k0 + j) * row_bytes + (size_t)v * 16));
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (k0 + j < K) acc_bf16x8(acc, x[j]);
      }
      st_na_v4(orow + (size_t)v * 16, pack_bf16x8(acc));
    }
  }
  if (a.out_weights) {
    const float* w = (const float*)peer_ptr(c, c.rank, (size_t)a.pushw_off);
    for (int i = blockIdx.x * blockDim.x + tid; i < S * K; i += nb * blockDim.x) a.out_weights[i] = __ldcg(w + i);
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

// Checked-mode validation of the duplicate tables (see dup_check_kernel); `kernel_id` names the caller in the report.
extern "C" int mep_launch_dup_check(int nv, const MepRankCtx* const* ctxs, const mep::DupArgs* args,
                                    int num_blocks, int kernel_id, cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain(mep::dup_check_kernel, dim3(num_blocks, nv), dim3(256), 0, stream, P, A, kernel_id);
}

extern "C" int mep_launch_dup_reduce(int nv, const MepRankCtx* const* ctxs, const mep::DupArgs* args,
                                     int num_blocks, cudaStream_t stream) {
  MepCtxPack P = {}; mep::DupArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain(mep::dup_reduce_kernel, dim3(mep::dup_grid(num_blocks), nv), dim3(256), 0, stream, P, A);
}

extern "C" int mep_launch_combine(int nv, const MepRankCtx* const* ctxs, const mep::CombineArgs* args,
                                  int num_sms, int pdl, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "combine: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::CombineArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  const size_t smem = (size_t)mep::kCombWarps * mep::kCombSlots * 32 * 16;
  return mep::launch_cooperative(mep::combine_kernel, dim3(num_sms, nv), dim3(mep::kCombThreads), smem,
                                 stream, pdl != 0, P, A);
}

extern "C" int mep_launch_push_reduce(int nv, const MepRankCtx* const* ctxs, const mep::PushReduceArgs* args,
                                      int num_blocks, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "push_reduce: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::PushReduceArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_cooperative(mep::push_reduce_kernel, dim3(num_blocks, nv), dim3(256), 0, stream, false, P, A);
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

MEP_EXPORT_SIZEOF(CombineArgs, mep::CombineArgs)
MEP_EXPORT_SIZEOF(PushReduceArgs, mep::PushReduceArgs)
