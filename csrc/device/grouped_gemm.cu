// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 -> fp32.
//
// The reference ships no GEMM: it hands `cu_seqlens[2*epn]` and the `[2*epn, in, out]`
// compute views to the integrating framework's "VM group GEMM" (README.md:45,54 of the
// reference). This file is that consumer, written for sm_100a:
//   * persistent CTAs (one per SM), warp-specialised: warp 0 = TMA producer, warp 1 = MMA
//     issuer (one elected thread issues tcgen05.mma), warps 2-5 = epilogue;
//   * operands staged by 2-D tiled TMA (128-byte swizzle) from LOCAL memory into a 4-stage
//     shared-memory ring; accumulators live in TMEM, double-buffered (2 x 256 columns) so the
//     epilogue of tile i overlaps the main loop of tile i+1;
//   * the tile list comes from `cu_seqlens` on the device (no host sync); every group is padded
//     to a multiple of 128 rows by the planner, so a 128-row tile never straddles two experts;
//     tiles are walked in a fixed strided order or, when the launch passes a ticket counter,
//     handed out dynamically (tile_queue.cuh) so that the kernel keeps its efficiency while a
//     communication kernel owns some of the SMs for part of its run.
// Tile: 128 x 256 x 64. Modes (weights stored [group, in, out], i.e. "N-contiguous"):
//   GATE_UP   act = silu(x Wg) * (x Wu)       A K-major, B MN-major from two tensors (128+128)
//   DOWN      y = (act Wd) * row_scale         A K-major, B MN-major
//   DGRAD     dA = dY W^T                      A K-major, B K-major
//   DGRAD_GU  dx = dG Wg^T + dU Wu^T           A = [dG | dU] K-major, B K-major from two tensors
//   WGRAD     dW[g] (+)= X_g^T dY_g  (fp32)    A and B MN-major, K = rows of the group
#include "tcgen05.cuh"
#include "tile_queue.cuh"
#include "gemm_args.h"
#include "../host/driver_api.h"
#include "../host/launch.h"

namespace mep {



// Same for a flag that another GPU writes (system scope).
__device__ __forceinline__ bool wait_flag_bounded_sys(const uint32_t* flag, uint32_t epoch, uint64_t budget_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const long long t0 = clock64(), lim = budget_cycles(budget_ns);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) { __nanosleep(200); if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true; }
    if (clock64() - t0 > lim) return false;
  }
}

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kABytes = kBM * kBK * 2;            // 16 KB
constexpr int kBBytes = kBN * kBK * 2;            // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;   // 48 KB per ring stage
constexpr int kAtomBytes = 64 * kBK * 2;          // one 64-wide MN-major atom: 64 k-rows x 128 B
// WGRAD has a short K loop (rows of one group) and a large fp32 tile to drain, so it runs 8
// epilogue warps (two per TMEM lane quarter, each draining half of the columns) on a 3-stage ring;
// the other modes run 4 epilogue warps on a 4-stage ring.
template <int MODE> struct GemmCfg {
  static constexpr int kEpiWarps = MODE == 4 ? 8 : 4;
  static constexpr int kRing = MODE == 4 ? 3 : 4;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr size_t kSmem = (size_t)kRing * (16384 + 32768) + (size_t)kEpiWarps * 2 * 4096 + 1024;
};
constexpr int kMaxGroups = 192;

// Bounded poll of a tile flag (see GemmArgs.tile_done): true once *flag has reached `epoch`.
__device__ __forceinline__ bool wait_flag_bounded(const uint32_t* flag, uint32_t epoch, uint64_t budget_ns) {
  if ((int32_t)(ld_acquire_gpu(flag) - epoch) >= 0) return true;
  const long long t0 = clock64(), lim = budget_cycles(budget_ns);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) { __nanosleep(100); if ((int32_t)(ld_acquire_gpu(flag) - epoch) >= 0) return true; }
    if (clock64() - t0 > lim) return false;
  }
}
constexpr int kSlabBytes = 32 * 128;             // epilogue staging: 32 rows x 128 B per warp and buffer
constexpr int kTmemCols = 512;

struct TileInfo { int g, row0, m0, n0, kblocks; };

template <int MODE>
__global__ void __launch_bounds__(GemmCfg<MODE>::kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b0,
                    const __grid_constant__ CUtensorMap tma_b1, const __grid_constant__ CUtensorMap tma_out, GemmArgs args) {
  constexpr bool A_MN = MODE == GEMM_WGRAD;
  constexpr bool B_MN = MODE == GEMM_GATE_UP || MODE == GEMM_DOWN || MODE == GEMM_WGRAD;
  constexpr int kStages = GemmCfg<MODE>::kRing;       // shadows the file-scope default
  constexpr int kEpiWarps = GemmCfg<MODE>::kEpiWarps;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;
  __shared__ int s_ntiles, s_nact;
  __shared__ tq::Ring s_ring;
  __shared__ int s_cu[kMaxGroups + 1];      // s_cu[g] = first row of group g (s_cu[G] = end)
  __shared__ int s_start[kMaxGroups + 1];   // non-WGRAD: first tile of group; WGRAD: active group ids
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = args.G;

  // ---------------- setup
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], kEpiWarps); }
    tq::init(&s_ring, 1 + kEpiWarps);
    fence_mbar_init();
    s_cu[0] = 0;
    for (int g = 0; g < G; ++g) s_cu[g + 1] = args.cu_seqlens[g];
    if (MODE == GEMM_WGRAD) {
      int n = 0, prev = 0;
      for (int g = 0; g < G; ++g) { const int e = s_cu[g + 1]; const bool in = g >= args.g_begin && g < args.g_end;
        if (in && (e > prev || (!args.accumulate && g < args.zero_empty_below))) s_start[n++] = g; prev = e; }
      s_nact = n;
      s_ntiles = n * (args.M_w / kBM) * (args.N / kBN);
    } else {
      const int nblk = MODE == GEMM_GATE_UP ? args.N / 128 : args.N / kBN;
      int run = 0, prev = 0;
      for (int g = 0; g < G; ++g) { const int e = s_cu[g + 1]; s_start[g] = run; if (g >= args.g_begin && g < args.g_end) run += ((e - prev) / kBM) * nblk; prev = e; }
      s_start[G] = run;
      s_ntiles = run;
    }
    tc::prefetch_tmap(&tma_a); tc::prefetch_tmap(&tma_b0); tc::prefetch_tmap(&tma_b1); tc::prefetch_tmap(&tma_out);
  }
  if (warp == 1) { tc::tmem_alloc(&s_tmem_base, kTmemCols); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = s_tmem_base;
  const int ntiles = s_ntiles;
  const bool dyn = args.sched != nullptr;

  auto fail = [&](int site, int tile) {
    const int code = site == 9 ? MEP_ERR_FLAG_TIMEOUT : MEP_ERR_MBAR_TIMEOUT;
    if (atomicCAS(&args.status[0], 0, code) == 0) {
      args.status[1] = site; args.status[2] = blockIdx.x; args.status[3] = tile;
      if (args.status_host) { *(volatile int32_t*)args.status_host = code; __threadfence_system(); }
    }
    s_abort = 1;
  };

  // tile index -> coordinates; `gcur` is a monotone cursor over groups (non-WGRAD)
  auto get_tile = [&](int t, int& gcur, TileInfo& ti) {
    if (MODE == GEMM_WGRAD) {
      const int mblk = args.M_w / kBM, per = mblk * (args.N / kBN);
      const int ai = t / per, local = t - ai * per;
      const int g = s_start[ai];
      const int beg = s_cu[g];
      ti.g = g; ti.row0 = beg; ti.kblocks = (s_cu[g + 1] - beg) / kBK;
      ti.m0 = (local % mblk) * kBM; ti.n0 = (local / mblk) * kBN;
    } else {
      while (gcur + 1 <= G && s_start[gcur + 1] <= t) ++gcur;
      const int g = gcur;
      const int beg = s_cu[g];
      const int mblk = (s_cu[g + 1] - beg) / kBM;
      const int local = t - s_start[g];
      ti.g = g; ti.row0 = beg + (local % mblk) * kBM; ti.m0 = 0;
      ti.n0 = (local / mblk) * (MODE == GEMM_GATE_UP ? 128 : kBN);
      ti.kblocks = args.K / kBK;
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer (one thread)
    if (lane == 0) {
      int it = 0, gcur = 0; TileInfo ti;
      tq::Scheduler<false> sched; if (dyn) sched.setup(&s_ring, args.sched, ntiles);
      tq::Strided seq{(int)blockIdx.x, (int)gridDim.x, ntiles};
      const uint32_t flag_ep = args.tile_done ? *(volatile const uint32_t*)args.tile_epoch : 0u;
      int flag_tile = -1;                  // last row tile whose flag was seen complete
      const uint32_t group_ep = args.group_flags ? *(volatile const uint32_t*)args.group_epoch : 0u;
      int flag_group = -1;                 // last group whose weights were seen complete
      for (int t; !s_abort && (t = dyn ? sched.next(args.budget_ns) : seq.next()) != -1;) {
        if (t == -2) { fail(5, sched.n); break; }
        get_tile(t, gcur, ti);
        if (!A_MN && args.tile_done && ti.kblocks > 0 && (ti.row0 >> 7) != flag_tile) {
          // rows of this tile come from a dispatch that may still be running: wait until they have all
          // landed and the duplicates are expanded, then order the TMA engine's reads behind that
          const uint32_t* f = args.tile_done + (ti.row0 >> 7);
          if (!wait_flag_bounded(f, flag_ep, args.budget_ns)) { fail(9, t); break; }
          fence_proxy_async();
          flag_tile = ti.row0 >> 7;
        }
        if (args.group_flags && ti.kblocks > 0 && ti.g >= args.group_first && ti.g != flag_group) {
          // the weights of this group are a prefetched expert that may still be on its way
          if (!wait_flag_bounded_sys(args.group_flags + (ti.g - args.group_first), group_ep, args.budget_ns)) { fail(9, t); break; }
          fence_proxy_async();
          flag_group = ti.g;
        }
        for (int kb = 0; kb < ti.kblocks; ++kb, ++it) {
          const int s = it % kStages; const uint32_t ph = (uint32_t)(it / kStages) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, args.budget_ns)) { fail(1, t); break; }
          unsigned char* sa = smem + (size_t)s * kStageBytes;
          unsigned char* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          const int k0 = kb * kBK;
          if (A_MN) {   // x[rows, in]: two 64-wide atoms along M, 64 token rows of K
            tc::tma_load_2d(sa, &tma_a, ti.m0, ti.row0 + k0, &full_bar[s]);
            tc::tma_load_2d(sa + kAtomBytes, &tma_a, ti.m0 + 64, ti.row0 + k0, &full_bar[s]);
          } else {
            tc::tma_load_2d(sa, &tma_a, k0, ti.row0, &full_bar[s]);
          }
          if (MODE == GEMM_GATE_UP) {
            const int r = ti.g * args.b_group_rows + k0;
            tc::tma_load_3d(sb, &tma_b0, 0, r, ti.n0 / 64, &full_bar[s]);
            tc::tma_load_3d(sb + 2 * kAtomBytes, &tma_b1, 0, r, ti.n0 / 64, &full_bar[s]);
          } else if (MODE == GEMM_DOWN) {
            const int r = ti.g * args.b_group_rows + k0;
            tc::tma_load_3d(sb, &tma_b0, 0, r, ti.n0 / 64, &full_bar[s]);
          } else if (MODE == GEMM_WGRAD) {
#pragma unroll
            for (int i = 0; i < 4; ++i) tc::tma_load_2d(sb + i * kAtomBytes, &tma_b0, ti.n0 + 64 * i, ti.row0 + k0, &full_bar[s]);
          } else if (MODE == GEMM_DGRAD) {
            tc::tma_load_2d(sb, &tma_b0, k0, ti.g * args.b_group_rows + ti.n0, &full_bar[s]);
          } else {  // DGRAD_GU: first half of K from Wg, second half from Wu
            const int half = args.K / 2;
            if (k0 < half) tc::tma_load_2d(sb, &tma_b0, k0, ti.g * args.b_group_rows + ti.n0, &full_bar[s]);
            else tc::tma_load_2d(sb, &tma_b1, k0 - half, ti.g * args.b_group_rows + ti.n0, &full_bar[s]);
          }
        }
      }
      // drain: do not leave the CTA while copies into its shared memory may still be in flight
      if (it > 0) {
        const int last = it - 1;
        const int s = last % kStages; const uint32_t ph = (uint32_t)(last / kStages) & 1u;
        mbar_wait_bounded(&full_bar[s], ph, args.budget_ns);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc_bf16(kBM, kBN, A_MN, B_MN);
      int it = 0, tcnt = 0, gcur = 0; TileInfo ti;
      tq::Consumer<false> tiles; tiles.setup(&s_ring);
      tq::Strided seq{(int)blockIdx.x, (int)gridDim.x, ntiles};
      for (int t; !s_abort && (t = dyn ? tiles.next(args.budget_ns) : seq.next()) != -1; ++tcnt) {
        if (t == -2) { fail(6, tiles.n); break; }
        get_tile(t, gcur, ti);
        if (ti.kblocks == 0) { --tcnt; continue; }     // empty group: the epilogue writes zeros on its own
        const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, args.budget_ns)) { fail(2, t); break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * kBN;
        bool ok = true;
        for (int kb = 0; kb < ti.kblocks; ++kb, ++it) {
          const int s = it % kStages; const uint32_t ph = (uint32_t)(it / kStages) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, args.budget_ns)) { fail(3, t); ok = false; break; }
          tc::fence_after_sync();
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t ad = A_MN ? tc::smem_desc(sa + k * 2048, kAtomBytes, 1024) : tc::smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? tc::smem_desc(sb + k * 2048, kAtomBytes, 1024) : tc::smem_desc(sb + k * 32, 16, 1024);
            tc::mma_bf16(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
          }
          tc::mma_commit(&empty_bar[s]);      // frees the stage when these MMAs have read it
        }
        if (!ok) break;
        tc::mma_commit(&tfull_bar[acc]);      // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue warps (TMEM lane quarter = warp % 4)
    const int q = warp & 3;
    const int r_in_tile = q * 32 + lane;
    // coalesced output: each warp transposes its 32-row slab through shared memory (128-byte
    // swizzle) and one lane writes it with a TMA store, double-buffered per warp
    const uint32_t stg = smem_u32(smem + (size_t)kStages * kStageBytes) + (uint32_t)(warp - 2) * 2 * kSlabBytes;
    int chunk_no = 0;
    int tcnt = 0, gcur = 0; TileInfo ti;
    tq::Consumer<false> tiles; tiles.setup(&s_ring);
    tq::Strided seq{(int)blockIdx.x, (int)gridDim.x, ntiles};
    for (;; ++tcnt) {
      int t = -1;
      if (!dyn) { if (!s_abort) t = seq.next(); }
      else {
        if (lane == 0 && !s_abort) { t = tiles.next(args.budget_ns); if (t == -2) fail(7, tiles.n); }
        t = __shfl_sync(0xffffffffu, t, 0);
      }
      if (t < 0) break;
      get_tile(t, gcur, ti);
      if (ti.kblocks == 0) {
        if (MODE == GEMM_WGRAD) {
          float* orow = (float*)args.out + ((size_t)ti.g * args.M_w + ti.m0 + r_in_tile) * args.N + ti.n0;
          const int h0 = ((warp - 2) >> 2) * (kBN / 8);
          for (int j = h0; j < h0 + kBN / 8; ++j) reinterpret_cast<float4*>(orow)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        --tcnt; continue;
      }
      const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
      int ok = 1;
      if (lane == 0) ok = mbar_wait_bounded(&tfull_bar[acc], aph, args.budget_ns) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) fail(4, t); break; }
      tc::fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * kBN;
      if (MODE == GEMM_GATE_UP) {
        const size_t row = (size_t)ti.row0 + r_in_tile;
        __nv_bfloat16* orow = (__nv_bfloat16*)args.out + row * args.ldo + ti.n0;
        __nv_bfloat16* grow = args.out2 ? (__nv_bfloat16*)args.out2 + row * (size_t)(2 * args.N) + ti.n0 : nullptr;
        const float sc = args.row_scale ? __ldcg(args.row_scale + row) : 1.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t gr[32], ur[32];
          tc::tmem_ld32(taddr + c * 32, gr);
          tc::tmem_ld32(taddr + 128 + c * 32, ur);
          tc::tmem_ld_wait();
          uint32_t o[16], og[16], ou[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(gr[2 * j]), g1 = __uint_as_float(gr[2 * j + 1]);
            const float u0 = __uint_as_float(ur[2 * j]), u1 = __uint_as_float(ur[2 * j + 1]);
            const float a0 = g0 / (1.f + __expf(-g0)) * u0 * sc, a1 = g1 / (1.f + __expf(-g1)) * u1 * sc;
            __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1); o[j] = *reinterpret_cast<uint32_t*>(&h);
            __nv_bfloat162 hg = __floats2bfloat162_rn(g0, g1); og[j] = *reinterpret_cast<uint32_t*>(&hg);
            __nv_bfloat162 hu = __floats2bfloat162_rn(u0, u1); ou[j] = *reinterpret_cast<uint32_t*>(&hu);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            st_v4(orow + c * 32 + j * 8, make_int4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
            if (grow) {
              st_v4(grow + c * 32 + j * 8, make_int4(og[4 * j], og[4 * j + 1], og[4 * j + 2], og[4 * j + 3]));
              st_v4(grow + args.N + c * 32 + j * 8, make_int4(ou[4 * j], ou[4 * j + 1], ou[4 * j + 2], ou[4 * j + 3]));
            }
          }
        }
      } else if (MODE == GEMM_WGRAD) {
        const int orow0 = ti.g * args.M_w + ti.m0 + q * 32;
        const int c_beg = ((warp - 2) >> 2) * 4;      // second set of four warps drains columns 128..255
#pragma unroll 1
        for (int c = c_beg; c < c_beg + 4; ++c, ++chunk_no) {
          const uint32_t buf = stg + (uint32_t)(chunk_no & 1) * kSlabBytes;
          if (lane == 0) bulk_wait_read<1>();          // the store issued two chunks ago has read this buffer
          __syncwarp();
          uint32_t r[32];
          tc::tmem_ld32(taddr + c * 32, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tc::st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (args.accumulate) tc::tma_reduce_add_2d(&tma_out, buf, ti.n0 + c * 32, orow0);
            else tc::tma_store_2d(&tma_out, buf, ti.n0 + c * 32, orow0);
            bulk_commit();
          }
        }
      } else if (args.push_info) {
        // "push" epilogue: every output row goes straight to the rank its token came from (peer
        // memory, plain 16-byte stores; 8 lanes cover one 128-byte line of a row). The per-row
        // destinations sit in the second staging buffer of the warp, the first one transposes.
        const size_t row = (size_t)ti.row0 + r_in_tile;
        const float sc = (MODE == GEMM_DOWN && args.row_scale) ? __ldcg(args.row_scale + row) : 1.f;
        const int info = args.push_info[row];
        unsigned char* dst = nullptr;
        if (info >= 0) {
          const int src = info / args.push_rows, idx = info - src * args.push_rows;
          if (src < args.push_ranks) {
            dst = args.push_base + (size_t)src * args.push_stride + ((size_t)idx * args.N + ti.n0) * 2;
            if (args.push_wsrc && ti.n0 == 0)
              *reinterpret_cast<float*>(args.push_wbase + (size_t)src * args.push_stride + (size_t)idx * 4) = args.push_wsrc[row];
          } else if (atomicCAS(&args.status[0], 0, MEP_ERR_BOUNDS) == 0) {
            args.status[1] = 8; args.status[2] = blockIdx.x; args.status[3] = (int)row;
            if (args.status_host) { *(volatile int32_t*)args.status_host = MEP_ERR_BOUNDS; __threadfence_system(); }
          }
        }
        const uint32_t buf = stg, ptrs = stg + kSlabBytes;
        __syncwarp();
        asm volatile("st.shared.b64 [%0], %1;" :: "r"(ptrs + lane * 8), "l"(dst) : "memory");
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[64];
          tc::tmem_ld32(taddr + c * 64, r);
          tc::tmem_ld32(taddr + c * 64 + 32, r + 32);
          tc::tmem_ld_wait();
          uint32_t o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * sc, __uint_as_float(r[2 * j + 1]) * sc);
            o[j] = *reinterpret_cast<uint32_t*>(&h);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tc::st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3), j = lane & 7;
            unsigned long long dp;
            asm volatile("ld.shared.b64 %0, [%1];" : "=l"(dp) : "r"(ptrs + rr * 8) : "memory");
            const int4 v = tc::ld_shared_v4(buf + rr * 128 + ((j ^ (rr & 7)) << 4));
            if (dp) st_v4(reinterpret_cast<unsigned char*>(dp) + c * 128 + j * 16, v);
          }
          __syncwarp();
        }
      } else {
        const size_t row = (size_t)ti.row0 + r_in_tile;
        const float sc = (MODE == GEMM_DOWN && args.row_scale) ? __ldcg(args.row_scale + row) : 1.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c, ++chunk_no) {       // 64 output columns (128 B of bf16) per chunk
          const uint32_t buf = stg + (uint32_t)(chunk_no & 1) * kSlabBytes;
          if (lane == 0) bulk_wait_read<1>();
          __syncwarp();
          uint32_t r[64];
          tc::tmem_ld32(taddr + c * 64, r);
          tc::tmem_ld32(taddr + c * 64 + 32, r + 32);
          tc::tmem_ld_wait();
          uint32_t o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * sc, __uint_as_float(r[2 * j + 1]) * sc);
            o[j] = *reinterpret_cast<uint32_t*>(&h);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tc::st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tc::tma_store_2d(&tma_out, buf, ti.n0 + c * 64, ti.row0 + q * 32);
            bulk_commit();
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    if (lane == 0) bulk_wait_all<0>();       // shared memory must outlive the stores reading it
  }

  // ---------------- teardown: everyone joins, then the allocating warp frees TMEM
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (warp == 1) tc::tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0) tq::scheduler_done(args.sched, args.sched_ctas > 0 ? args.sched_ctas : (int)gridDim.x);
}

static int make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
                    bool f32 = false) {
  const DriverApi* d = driver(); if (!d) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const int es_bytes = f32 ? 4 : 2;
  cuuint64_t strides[1] = {(cuuint64_t)ld * es_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  MEP_REQUIRE(((uintptr_t)base & 15) == 0 && (ld * es_bytes) % 16 == 0 && ld >= cols,
              "gemm: tensor base/stride must be 16-byte aligned");
  MEP_CU_CHECK(d->TensorMapEncodeTiled(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return 0;
}

// MN-major operand [rows (k), cols (m or n)] viewed as (64 elements, rows, cols/64): one box of
// `atoms` 64-wide atoms x 64 rows lands in shared memory atom after atom.
static int make_map_mn(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int atoms) {
  const DriverApi* d = driver(); if (!d) return -1;
  MEP_REQUIRE(cols % 64 == 0, "gemm: MN-major operand width %lld must be a multiple of 64", (long long)cols);
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, 64, (cuuint32_t)atoms};
  cuuint32_t es[3] = {1, 1, 1};
  MEP_REQUIRE(((uintptr_t)base & 15) == 0 && (ld * 2) % 16 == 0 && ld >= cols, "gemm: tensor base/stride must be 16-byte aligned");
  MEP_CU_CHECK(d->TensorMapEncodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return 0;
}

}  // namespace mep

// One grouped GEMM launch. `a` is a row-major bf16 matrix [a_rows, a_cols]; `b0`/`b1` are the
// weight tensors flattened to 2-D [b_rows, b_cols] (WGRAD: b0 = dY [rows, N]); `a_ld` / `b_ld` are
// the row pitches in elements (>= the column count). See the file
// header for what each mode computes.
extern "C" int mep_grouped_gemm(int mode, const void* a, int64_t a_rows, int64_t a_cols, int64_t a_ld,
                                const void* b0, const void* b1, int64_t b_rows, int64_t b_cols, int64_t b_ld,
                                const mep::GemmArgs* args_in, int num_ctas, cudaStream_t stream) {
  using namespace mep;
  GemmArgs args = *args_in;
  MEP_REQUIRE(args.G >= 1 && args.G <= kMaxGroups, "gemm: G=%d out of range [1,%d]", args.G, kMaxGroups);
  CUtensorMap ma, mb0, mb1, mo;
  const bool b_mn = mode == GEMM_GATE_UP || mode == GEMM_DOWN || mode == GEMM_WGRAD;
  if (mode == GEMM_WGRAD) {
    MEP_REQUIRE(args.M_w % kBM == 0 && args.N % kBN == 0, "wgrad: weight shape [%d,%d] must be multiples of [128,256]", args.M_w, args.N);
    if (make_map(&ma, a, a_rows, a_cols, a_ld, 64, 64)) return -1;
  } else {
    MEP_REQUIRE(args.K % kBK == 0, "gemm: K=%d must be a multiple of 64", args.K);
    MEP_REQUIRE(args.N % (mode == GEMM_GATE_UP ? 128 : kBN) == 0, "gemm: N=%d not tileable", args.N);
    if (make_map(&ma, a, a_rows, a_cols, a_ld, 64, kBM)) return -1;
  }
  const int b_atoms = mode == GEMM_GATE_UP ? 2 : 4;
  if (mode == GEMM_WGRAD) { if (make_map(&mb0, b0, b_rows, b_cols, b_ld, 64, 64)) return -1; }   // token-major operands: 2-D boxes are faster
  else if (b_mn) { if (make_map_mn(&mb0, b0, b_rows, b_cols, b_ld, b_atoms)) return -1; }
  else      { if (make_map(&mb0, b0, b_rows, b_cols, b_ld, 64, kBN)) return -1; }
  if (b1) { if (b_mn ? make_map_mn(&mb1, b1, b_rows, b_cols, b_ld, b_atoms) : make_map(&mb1, b1, b_rows, b_cols, b_ld, 64, kBN)) return -1; }
  else mb1 = mb0;
  // output map: one 32-row x 128-byte box per epilogue warp and chunk
  if (mode == GEMM_WGRAD) { if (make_map(&mo, args.out, (int64_t)args.G * args.M_w, args.N, args.N, 32, 32, true)) return -1; }
  else if (mode == GEMM_GATE_UP) mo = ma;
  else { if (make_map(&mo, args.out, a_rows, args.N, args.ldo, 64, 32)) return -1; }
  dim3 grid(num_ctas);
#define MEP_GEMM_CASE(M)                                                                             \
  case M:                                                                                            \
    MEP_CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<M>::kSmem)); \
    grouped_gemm_kernel<M><<<grid, dim3(GemmCfg<M>::kThreads), GemmCfg<M>::kSmem, stream>>>(ma, mb0, mb1, mo, args);                       \
    break;
  switch (mode) {
    MEP_GEMM_CASE(GEMM_GATE_UP) MEP_GEMM_CASE(GEMM_DOWN) MEP_GEMM_CASE(GEMM_DGRAD)
    MEP_GEMM_CASE(GEMM_DGRAD_GU) MEP_GEMM_CASE(GEMM_WGRAD)
    default: return set_error("gemm: unknown mode %d", mode);
  }
#undef MEP_GEMM_CASE
  MEP_CUDA_CHECK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

MEP_EXPORT_SIZEOF(GemmArgs, mep::GemmArgs)
