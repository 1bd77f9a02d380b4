// Online redundant-expert planner, replicated on every rank.
//
// Produces, with no host synchronisation, the same tables as the reference's
// rank-0-centralised PlanningKernel (moonep/planning.py:328-1101; executable spec
// tests/planning_reference.py:25-311): dst[N], cu_seqlens[2epn], experts_to_copy[R,epn],
// zero_fill_ranges[2epn,2], remote_stats[2] -- plus the duplicate-row groups, which this
// kernel emits from the sender side straight into the destination rank's staging tables.
//
// Structure (one cooperative launch, grid = num_sms CTAs x 1024 threads per rank):
//   P0  CTA 0 stores this rank's expert histogram into row `rank` of every peer's table;
//       all CTAs histogram their 1024-entry blocks of the local top-k table;
//       ONE cross-rank barrier (the reference needs three).
//   P1  CTA 0 solves the plan from the all-gathered histograms -- every rank computes the
//       identical result, so nothing is broadcast; the other CTAs turn the block
//       histograms into exclusive offsets.
//   P2  every entry gets its index among the same-expert entries (stable order), its
//       destination rank by binary search in the per-expert prefix over ranks, and its
//       slot; per token, later entries to an already used rank are marked duplicates and
//       (primary, duplicates) groups are appended to the destination's staging tables.
#include "prims.cuh"
#include "planning_args.h"
#include "../host/launch.h"
#include <limits.h>

namespace mep {

__device__ __forceinline__ int vload(const int* p) { return *(const volatile int*)p; }
__device__ __forceinline__ void vstore(int* p, int v) { *(volatile int*)p = v; }

// ---- P1 on CTA 0: receiver selection, expert split, layout (see file header).
__device__ void solve(const MepRankCtx& c, const PlanArgs& a, int* s_e, bool e_in_smem, bool emit = true) {
  __shared__ int s_bal[MEP_MAX_RANKS];
  __shared__ int s_recv_from[MEP_MAX_RANKS];
  __shared__ int s_quota[MEP_MAX_RANKS];
  __shared__ int s_send[MEP_MAX_RANKS];
  __shared__ int s_recvn[MEP_MAX_RANKS];
  const int R = c.R, E = c.E, epn = c.epn, cap = c.N, pad = c.token_padding;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int* tpeall = (const int*)peer_ptr(c, c.rank, c.off_tpe);
  int* remaining = e_in_smem ? s_e : c.remaining;

  // S1: totals per expert, my exclusive prefix over source ranks
  for (int e = tid; e < E; e += nt) {
    int run = 0;
    for (int r = 0; r < R; ++r) {
      if (r == c.rank) c.tpe_prefix[e] = run;
      run += __ldcg(tpeall + (size_t)r * E + e);
    }
    c.count[e] = run;
    remaining[e] = run;
  }
  for (int r = tid; r < R; r += nt) { s_recv_from[r] = -1; s_quota[r] = 0; s_send[r] = 0; s_recvn[r] = 0; }
  __syncthreads();
  for (int h = warp; h < R; h += nwarps) {
    int sum = 0;
    for (int j = lane; j < epn; j += 32) sum += vload(remaining + h * epn + j);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) s_bal[h] = sum - cap;
  }
  __syncthreads();

  // S2: receivers. Most loaded group feeds the emptiest rank until it holds exactly S*K.
  if (warp == 0) {
    for (int it = 0; it < R; ++it) {
      long long kmax = LLONG_MIN, kmin = LLONG_MIN;
      for (int r = lane; r < R; r += 32) {
        const int b = s_bal[r];
        const long long k1 = argmax_key(b, r), k2 = argmax_key(-b, r);
        kmax = k1 > kmax ? k1 : kmax; kmin = k2 > kmin ? k2 : kmin;
      }
      kmax = warp_max64(kmax); kmin = warp_max64(kmin);
      const int h = key_index(kmax), bh = key_value(kmax);
      const int u = key_index(kmin), bu = -key_value(kmin);
      if (bh <= 0 || bu >= 0) break;
      if (lane == 0) { s_recv_from[u] = h; s_quota[u] = -bu; s_bal[h] = bh + bu; s_bal[u] = 0; }
      __syncwarp();
    }
  }
  // S3a: dense allocation table starts with every expert at home
  for (int i = tid; i < E * R; i += nt) {
    const int e = i / R, d = i - e * R;
    c.alloc[i] = (d == e / epn) ? c.count[e] : 0;
  }
  __syncthreads();

  // S3b: split each donor group's tokens over its receivers (one warp per home group)
  for (int h = warp; h < R; h += nwarps) {
    for (int guard = 0; guard < R + epn + 2; ++guard) {
      long long kq = LLONG_MIN;
      for (int u = lane; u < R; u += 32)
        if (s_recv_from[u] == h) { const long long k = argmax_key(s_quota[u], u); kq = k > kq ? k : kq; }
      kq = warp_max64(kq);
      if (kq == LLONG_MIN || key_value(kq) <= 0) break;
      long long kr = LLONG_MIN;
      for (int j = lane; j < epn; j += 32) { const long long k = argmax_key(vload(remaining + h * epn + j), j); kr = k > kr ? k : kr; }
      kr = warp_max64(kr);
      const int d = key_index(kq), quota = key_value(kq), le = key_index(kr), rem = key_value(kr);
      const int take = rem < quota ? rem : quota;
      if (take <= 0) break;
      if (lane == 0) {
        const int e = h * epn + le;
        c.alloc[(size_t)e * R + d] += take;
        c.alloc[(size_t)e * R + h] -= take;
        vstore(remaining + e, rem - take);
        s_quota[d] = quota - take;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // S5: prefix over destination ranks per expert (binary-searched in P2)
  for (int e = tid; e < E; e += nt) {
    int run = 0;
    for (int d = 0; d < R; ++d) { run += c.alloc[(size_t)e * R + d]; c.alloc_cumsum[(size_t)e * R + d] = run; }
  }
  // S4: layout of every destination rank (one warp each)
  for (int d = warp; d < R; d += nwarps) {
    const int h = s_recv_from[d];
    int* etc = c.etc_all + (size_t)d * epn;
    for (int b = lane; b < epn; b += 32) { vstore(etc + b, -1); if (emit) a.experts_to_copy[(size_t)d * epn + b] = -1; }
    __syncwarp();
    int nrem = 0;
    if (h >= 0) {
      for (int j0 = 0; j0 < epn; j0 += 32) {
        const int j = j0 + lane;
        const bool has = j < epn && c.alloc[(size_t)(h * epn + j) * R + d] > 0;
        const unsigned bal = __ballot_sync(0xffffffffu, has);
        if (has) {
          const int pos = nrem + __popc(bal & lanemask_lt());
          vstore(etc + pos, h * epn + j);
          if (emit) a.experts_to_copy[(size_t)d * epn + pos] = h * epn + j;
        }
        nrem += __popc(bal);
      }
    }
    if (lane == 0) { s_recvn[d] = nrem; if (h >= 0 && nrem) atomicAdd(&s_send[h], nrem); }
    __syncwarp();
    int start = 0;
    for (int g0 = 0; g0 < 2 * epn; g0 += 32) {
      const int g = g0 + lane;
      int e = -1, cnt = 0;
      if (g < epn) e = d * epn + g; else if (g < 2 * epn) e = vload(etc + g - epn);
      if (e >= 0) cnt = c.alloc[(size_t)e * R + d];
      const int padded = cnt > 0 ? (cnt + pad - 1) / pad * pad : 0;
      const int incl = warp_incl_scan(padded);
      const int beg = start + incl - padded, end = start + incl;
      if (g < 2 * epn) {
        if (cnt > 0) c.expert_off[(size_t)d * E + e] = beg;
        if (d == c.rank && emit) {
          a.cu_seqlens[g] = end;
          const bool haspad = cnt > 0 && padded > cnt;
          a.zero_fill[2 * g] = haspad ? beg + cnt : 0;
          a.zero_fill[2 * g + 1] = haspad ? padded - cnt : 0;
        }
      }
      start += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (tid == 0 && emit) { a.remote_stats[0] = s_recvn[c.rank]; a.remote_stats[1] = s_send[c.rank]; }
  for (int r = tid; r < R; r += nt) { c.stats_all[2 * r] = s_recvn[r]; c.stats_all[2 * r + 1] = s_send[r]; }
}

struct PlanTables { const int* tpe_prefix; const int* alloc_cumsum; const int* expert_off; };
template <bool SM> __device__ __forceinline__ int ldt(const int* p) { return SM ? *p : __ldcg(p); }

struct PlanSmem {
  int raw[kPlanThreads];
  unsigned char dest[kPlanThreads];
  int pos[kPlanThreads];                 // CTA-local (group<<16 | loff) position of a primary's group
  unsigned long long cnt[MEP_MAX_RANKS]; // groups<<32 | loffs reserved by this CTA per destination
  unsigned long long base[MEP_MAX_RANKS];
};

// P2 for one block of entries: `cnt[e]` holds, on entry, the number of entries of expert e in earlier
// blocks of this rank. FAST: the lookup tables live in this CTA's shared memory.
template <bool FAST>
__device__ __forceinline__ void assign_vblock(const MepRankCtx& c, const PlanArgs& a, const PlanTables& T, int v,
                                              int* cnt, PlanSmem& sm, int* tbl = nullptr) {
  int* s_raw = sm.raw; unsigned char* s_dest = sm.dest; int* s_pos = sm.pos;
  unsigned long long* s_cnt = sm.cnt; unsigned long long* s_base = sm.base;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int R = c.R, E = c.E, N = c.N, K = c.K, NvS = c.NvS, VB = c.vblock_entries;
  const int tok_per_vb = VB / K;
  {
    for (int d = tid; d < R; d += nt) s_cnt[d] = 0ull;
    __syncthreads();
    const int i = v * VB + tid;
    const bool active = tid < VB && i < N;
    int e = active ? a.topk[i] : 0;
    if ((unsigned)e >= (unsigned)E) e = 0;
    const int n_here = min(VB, N - v * VB);
    const int nw = (n_here + 31) >> 5;
    int local_cnt = 0;
    if (tbl != nullptr) {
      // table ranking (small E): tbl[w][e] = entries of expert e held by warp w; an exclusive scan
      // over the warps (plus the count from earlier blocks) gives every warp its starting rank
      for (int i = tid; i < 32 * E; i += nt) tbl[i] = 0;
      __syncthreads();
      unsigned m = 0;
      const unsigned act = __ballot_sync(0xffffffffu, active);
      if (active) {
        m = __match_any_sync(act, e);
        if (lane == __ffs(m) - 1) tbl[warp * E + e] = __popc(m);
      }
      __syncthreads();
      for (int e2 = tid; e2 < E; e2 += nt) {
        int run = cnt[e2];
        for (int w = 0; w < 32; ++w) { const int t = tbl[w * E + e2]; tbl[w * E + e2] = run; run += t; }
        cnt[e2] = run;
      }
      __syncthreads();
      if (active) local_cnt = tbl[warp * E + e] + __popc(m & lanemask_lt());
    } else
    for (int w = 0; w < nw; ++w) {       // warps in index order => stable ranking
      if (warp == w) {
        const unsigned act = __ballot_sync(0xffffffffu, active);
        if (active) {
          const unsigned m = __match_any_sync(act, e);
          const int leader = __ffs(m) - 1;
          int old = 0;
          if (lane == leader) { old = vload(cnt + e); vstore(cnt + e, old + __popc(m)); }
          old = __shfl_sync(m, old, leader);
          local_cnt = old + __popc(m & lanemask_lt());
        }
      }
      __syncthreads();
    }
    int raw = 0, dr = 0;
    if (active) {
      const int g = ldt<FAST>(T.tpe_prefix + e) + local_cnt;
      const int* ac = T.alloc_cumsum + (size_t)e * R;
      int lo = 0, hi = R - 1;
      while (lo < hi) { const int mid = (lo + hi) >> 1; if (ldt<FAST>(ac + mid) > g) hi = mid; else lo = mid + 1; }
      dr = lo;
      const int prev = dr ? ldt<FAST>(ac + dr - 1) : 0;
      const int loff = ldt<FAST>(T.expert_off + (size_t)dr * E + e) + (g - prev);
      if ((unsigned)loff >= (unsigned)NvS || g >= ldt<FAST>(ac + dr))
        report(c, MEP_ERR_BOUNDS, MEP_K_PLANNING, 2, i, (uint32_t)loff, (uint32_t)NvS);
      raw = dr * NvS + loff;
    }
    s_raw[tid] = raw; s_dest[tid] = (unsigned char)dr; s_pos[tid] = -1;
    __syncthreads();

    // token phase A: duplicate marking + CTA-local reservation of group slots
    const int s_tok = v * tok_per_vb + tid;
    const bool tok_active = tid < tok_per_vb && s_tok < c.S;
    if (tok_active) {
      const int base = tid * K;
      for (int k = 0; k < K; ++k) {
        const int d = s_dest[base + k];
        bool first = true;
        for (int k2 = 0; k2 < k; ++k2) first = first && (s_dest[base + k2] != d);
        const int r = s_raw[base + k];
        a.dst[(size_t)s_tok * K + k] = first ? r : -r - 1;
        if (first) {
          int n = 0;
          for (int k2 = k + 1; k2 < K; ++k2) n += (s_dest[base + k2] == d);
          if (n > 0) {
            const unsigned long long old = atomicAdd(&s_cnt[d], (1ull << 32) | (unsigned)n);
            s_pos[base + k] = (int)(((old >> 32) << 16) | (old & 0xffffu));
          }
        }
      }
    }
    __syncthreads();
    for (int d = tid; d < R; d += nt) {
      const unsigned long long add = s_cnt[d];
      s_base[d] = add ? atomicAdd(&c.send_cnt[d], add) : 0ull;
    }
    __syncthreads();
    // token phase B: append (primary, start, n) and the duplicate offsets to the
    // destination rank's staging tables (region reserved for this source rank)
    if (tok_active) {
      const int base = tid * K;
      for (int k = 0; k < K; ++k) {
        const int p = s_pos[base + k];
        if (p < 0) continue;
        const int d = s_dest[base + k];
        const unsigned long long b = s_base[d];
        const int gi = (int)(b >> 32) + (p >> 16);
        const int li = (int)(b & 0xffffffffu) + (p & 0xffff);
        int* grp = (int*)peer_ptr(c, d, c.off_dupgroups) + ((size_t)c.rank * c.dup_group_cap + gi) * 3;
        int* lof = (int*)peer_ptr(c, d, c.off_duploffs) + (size_t)c.rank * c.dup_loff_cap + li;
        int n = 0;
        for (int k2 = k + 1; k2 < K; ++k2)
          if (s_dest[base + k2] == d) lof[n++] = s_raw[base + k2] - d * NvS;
        grp[0] = s_raw[base + k] - d * NvS; grp[1] = li; grp[2] = n;
      }
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kPlanThreads, 1) planning_kernel(MepCtxPack P, PlanArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const PlanArgs& a = A.a[blockIdx.y];
  extern __shared__ int s_e[];
  const int nb = gridDim.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int R = c.R, E = c.E, N = c.N, K = c.K, NvS = c.NvS, VB = c.vblock_entries;
  const bool e_in_smem = E <= kSmemECap;

  // ---------------- P0
  if (blockIdx.x == 0) {
    if (c.mc_base != nullptr && (E & 3) == 0 && R > 1) {
      // NVSwitch multicast: one 16-byte store per four experts reaches every rank's table
      char* row = c.mc_base + c.off_tpe + (size_t)c.rank * E * 4;
      for (int e4 = tid; e4 < E / 4; e4 += nt)
        multimem_st_v4(row + (size_t)e4 * 16, *reinterpret_cast<const int4*>(a.tpe + 4 * e4));
      fence_proxy_alias();
    } else {
      for (int i = tid; i < R * E; i += nt) {
        const int p = i / E, e = i - p * E;
        ((int*)peer_ptr(c, p, c.off_tpe))[(size_t)c.rank * E + e] = a.tpe[e];
      }
    }
    for (int d = tid; d < R; d += nt) c.send_cnt[d] = 0ull;
  }
  for (int v = blockIdx.x; v < c.num_vblocks; v += nb) {
    int* row = c.hist + (size_t)v * E;
    int* h = e_in_smem ? s_e : row;
    for (int e = tid; e < E; e += nt) h[e] = 0;
    __syncthreads();
    const int i = v * VB + tid;
    if (tid < VB && i < N) {
      const int e = a.topk[i];
      if ((unsigned)e < (unsigned)E) atomicAdd(&h[e], 1);
      else report(c, MEP_ERR_BOUNDS, MEP_K_PLANNING, 1, i, (uint32_t)e, (uint32_t)E);
    }
    __syncthreads();
    if (e_in_smem) for (int e = tid; e < E; e += nt) row[e] = s_e[e];
    __syncthreads();
  }
  if (!cross_rank_barrier(c, nb, 0, MEP_K_PLANNING, 10)) return;

  // ---------------- P1
  if (blockIdx.x == 0) { solve(c, a, s_e, e_in_smem); __syncthreads(); }
  if (nb == 1 || blockIdx.x != 0) {
    const int workers = nb == 1 ? 1 : nb - 1, me = nb == 1 ? 0 : blockIdx.x - 1;
    for (int e = me * nt + tid; e < E; e += workers * nt) {
      int run = 0;
      for (int v = 0; v < c.num_vblocks; ++v) {
        int* p = c.hist + (size_t)v * E + e;
        const int t = __ldcg(p);
        *p = run; run += t;
      }
    }
  }
  if (!grid_sync(c, nb, MEP_K_PLANNING, 20)) return;
  if (aborted(c)) return;

  // ---------------- P2
  __shared__ PlanSmem sm;
  const PlanTables T = {c.tpe_prefix, c.alloc_cumsum, c.expert_off};
  for (int v = blockIdx.x; v < c.num_vblocks; v += nb) {
    int* row = c.hist + (size_t)v * E;
    int* cnt = e_in_smem ? s_e : row;
    if (e_in_smem) for (int e = tid; e < E; e += nt) s_e[e] = __ldcg(row + e);
    assign_vblock<false>(c, a, T, v, cnt, sm);
  }
}


// ---------------------------------------------------------------------------------------------
// Fast path (E <= 2048, E*R <= 8192): no grid-wide barrier at all.
//   * CTA 0 publishes this rank's histogram and then release-stores the launch epoch into every
//     peer's flag slot. The epoch lives in device memory (word `vb_flags[num_vblocks]`, the number
//     of fast plannings this rank has completed; identical on all ranks because planning is
//     collective): every CTA reads it on entry, and the last CTA to leave the kernel advances it,
//     so a captured CUDA graph can be replayed without the host counting anything;
//   * EVERY CTA waits for all peers' epochs itself and then solves the plan redundantly into its
//     own shared memory (the solve is a few microseconds and fully deterministic), so nothing has
//     to be exchanged between the CTAs of a rank;
//   * every CTA publishes the expert histogram of each of its 1024-entry blocks and raises that
//     block's flag to the launch epoch; the count of same-expert entries in earlier blocks is a
//     column sum over the earlier blocks' rows (no rescan of the top-k table).
// send_cnt is double-buffered by epoch parity: this launch accumulates into half (epoch & 1) and
// clears the other half for the next launch.
__global__ void __launch_bounds__(kPlanThreads, 1) planning_fast_kernel(MepCtxPack P, PlanArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];
  const PlanArgs a = A.a[blockIdx.y];
  extern __shared__ int s_dyn[];
  __shared__ PlanSmem sm;
  __shared__ int s_fail;
  const int nb = gridDim.x, tid = threadIdx.x, nt = blockDim.x;
  const int R = c.R, E = c.E, N = c.N, VB = c.vblock_entries;
  int* s_cnt = s_dyn;
  int* s_rem = s_cnt + E;
  int* s_count = s_rem + E;
  int* s_tpre = s_count + E;
  int* s_etc = s_tpre + E;
  int* s_stats = s_etc + E;
  int* s_alloc = s_stats + 2 * MEP_MAX_RANKS;
  int* s_acum = s_alloc + E * R;
  int* s_expoff = s_acum + E * R;
  int* s_tbl = E <= kFastTableE ? s_expoff + E * R : nullptr;     // [32, E] ranking table
  uint32_t* const epoch_word = c.vb_flags + c.num_vblocks;      // [0] completed epochs, [1] CTAs that left
  const uint32_t ep = __ldcg(epoch_word) + 1u;
  unsigned long long* send_cur = c.send_cnt + (size_t)(ep & 1u) * R;
  // every exit path runs this: the last CTA out advances the epoch for the next launch
  auto leave = [&]() {
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(epoch_word + 1, 1u) == (uint32_t)nb - 1u) { epoch_word[1] = 0u; epoch_word[0] = ep; __threadfence(); }
    }
  };

  if (tid == 0) { s_fail = 0; trace_mark(c, MEP_K_PLANNING, 1); }
  if (blockIdx.x == 0) {
    if (c.mc_base != nullptr && (E & 3) == 0 && R > 1) {
      char* row = c.mc_base + c.off_tpe + (size_t)c.rank * E * 4;
      for (int e4 = tid; e4 < E / 4; e4 += nt)
        multimem_st_v4(row + (size_t)e4 * 16, *reinterpret_cast<const int4*>(a.tpe + 4 * e4));
      fence_proxy_alias();
    } else {
      for (int i = tid; i < R * E; i += nt) {
        const int p = i / E, e = i - p * E;
        ((int*)peer_ptr(c, p, c.off_tpe))[(size_t)c.rank * E + e] = a.tpe[e];
      }
    }
    for (int d = tid; d < R; d += nt) c.send_cnt[(size_t)((ep & 1u) ^ 1u) * R + d] = 0ull;
    __syncthreads();
    if (R > 1)
      for (int p = tid; p < R; p += nt) {
        __threadfence_system();
        st_release_sys((uint32_t*)peer_ptr(c, p, c.off_bar) + c.rank, ep);
      }
  }

  // Block histograms: every CTA publishes the histogram of each of its 1024-entry blocks and raises
  // that block's flag to the launch epoch. The number of same-expert entries in earlier blocks is
  // then a column sum over the earlier blocks' rows -- no rescan of the top-k table, no grid barrier.
  for (int v = blockIdx.x; v < c.num_vblocks; v += nb) {
    for (int e = tid; e < E; e += nt) s_cnt[e] = 0;
    __syncthreads();
    const int i = v * VB + tid;
    if (tid < VB && i < N) {
      const int e = __ldg(a.topk + i);
      if ((unsigned)e < (unsigned)E) atomicAdd(&s_cnt[e], 1);
      else report(c, MEP_ERR_BOUNDS, MEP_K_PLANNING, 1, i, (uint32_t)e, (uint32_t)E);
    }
    __syncthreads();
    int* row = c.hist + (size_t)v * E;
    for (int e = tid; e < E; e += nt) row[e] = s_cnt[e];
    __syncthreads();
    if (tid == 0) { __threadfence(); asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(c.vb_flags + v), "r"(ep) : "memory"); }
  }
  auto count_prefix = [&](int v) {        // s_cnt[e] = entries of expert e in blocks < v of this rank
    for (int u = tid; u < v; u += nt) {
      uint32_t seen = 0;
      const bool ok = bounded_wait(c, [&] { seen = ld_acquire_gpu(c.vb_flags + u); return (int32_t)(seen - ep) >= 0; });
      if (!ok) { report(c, MEP_ERR_GRID_SYNC_TIMEOUT, MEP_K_PLANNING, 12, u, seen, ep); s_fail = 1; }
    }
    __syncthreads();
    for (int e = tid; e < E; e += nt) {
      int run = 0;
      for (int u = 0; u < v; ++u) run += __ldcg(c.hist + (size_t)u * E + e);
      s_cnt[e] = run;
    }
    __syncthreads();
  };
  if ((int)blockIdx.x < c.num_vblocks) count_prefix(blockIdx.x);
  if (tid == 0) trace_mark(c, MEP_K_PLANNING, 2);

  if (R > 1) {
    for (int p = tid; p < R; p += nt) {
      const uint32_t* slot = (const uint32_t*)peer_ptr(c, c.rank, c.off_bar) + p;
      uint32_t seen = 0;
      const bool ok = bounded_wait(c, [&] { seen = ld_acquire_sys(slot); return (int32_t)(seen - ep) >= 0; });
      if (!ok) { report(c, MEP_ERR_PEER_TIMEOUT, MEP_K_PLANNING, 11, p, seen, ep); s_fail = 1; }
    }
  }
  __syncthreads();
  if (s_fail) { leave(); return; }
  if (tid == 0) trace_mark(c, MEP_K_PLANNING, 3);

  MepRankCtx cl = c;
  cl.count = s_count; cl.tpe_prefix = s_tpre; cl.remaining = s_rem; cl.alloc = s_alloc;
  cl.alloc_cumsum = s_acum; cl.expert_off = s_expoff; cl.etc_all = s_etc; cl.stats_all = s_stats;
  solve(cl, a, s_rem, true, blockIdx.x == 0);
  __syncthreads();
  if (tid == 0) trace_mark(c, MEP_K_PLANNING, 4);

  cl.send_cnt = send_cur;
  const PlanTables T = {s_tpre, s_acum, s_expoff};
  for (int v = blockIdx.x; v < c.num_vblocks; v += nb) {
    if (v != (int)blockIdx.x) count_prefix(v);
    assign_vblock<true>(cl, a, T, v, s_cnt, sm, s_tbl);
  }
  if (tid == 0) trace_mark(c, MEP_K_PLANNING, 5);
  leave();
}

}  // namespace mep

extern "C" int mep_launch_planning(int nv, const MepRankCtx* const* ctxs, const mep::PlanArgs* args,
                                   int num_sms, int E, int R, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "planning: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::PlanArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  if (E <= mep::kFastMaxE && (long long)E * R <= mep::kFastMaxER && args[0].epoch != 0) {
    const size_t smem = ((size_t)6 * E + 2 * MEP_MAX_RANKS + (size_t)3 * E * R + (E <= mep::kFastTableE ? 32 * (size_t)E : 0)) * sizeof(int);
    return mep::launch_cooperative(mep::planning_fast_kernel, dim3(num_sms, nv), dim3(mep::kPlanThreads), smem,
                                   stream, false, P, A);
  }
  const size_t smem = (E <= mep::kSmemECap ? (size_t)E : 1) * sizeof(int);
  return mep::launch_cooperative(mep::planning_kernel, dim3(num_sms, nv), dim3(mep::kPlanThreads), smem,
                                 stream, false, P, A);
}

// 1 if a geometry is served by the barrier-free planning kernel (selected with PlanArgs.epoch != 0).
extern "C" int mep_planning_is_fast(int E, int R) {
  return (E <= mep::kFastMaxE && (long long)E * R <= mep::kFastMaxER) ? 1 : 0;
}

MEP_EXPORT_SIZEOF(PlanArgs, mep::PlanArgs)
