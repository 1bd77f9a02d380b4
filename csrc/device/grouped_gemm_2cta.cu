// Weight-gradient grouped GEMM on CTA pairs: dW[g] (+)= X_g^T dY_g with tcgen05.mma.cta_group::2.
//
// Two CTAs of a cluster (two SMs) compute one 256 x 256 fp32 tile: each CTA stages ITS half of both
// operands (128 weight rows of X^T and 128 of the 256 output columns of dY, 32 KB per 64-token
// k-block) with ordinary single-CTA TMA loads from local memory, and the pair's tensor cores read
// both halves. Per SM that is 32 KB of shared-memory fill per k-block instead of 48 KB for the same
// amount of math, which is what limits the single-CTA kernel (operand feed, not the tensor pipe).
// No cluster-wide copy is used: every load lands in the issuing CTA only and merely counts its bytes
// on the leader CTA's mbarrier. The M tile is over weight rows, so it never straddles experts.
// Roles per CTA: warp 0 = TMA producer, warp 1 = TMEM allocation (+ MMA issue in the leader CTA),
// warps 2-9 = epilogue (each CTA drains its own 128 accumulator rows through shared memory + TMA
// store / reduce-add).
#include "tcgen05.cuh"
#include "tile_queue.cuh"
#include "gemm_args.h"
#include "../host/driver_api.h"
#include "../host/launch.h"

namespace mep {
namespace w2 {

constexpr int kBK = 64, kRing = 5, kEpiWarps = 8, kThreads = 64 + 32 * kEpiWarps;
constexpr int kHalfBytes = 128 * kBK * 2;            // 16 KB: one operand half per CTA and k-block
constexpr int kStageBytes = 2 * kHalfBytes;          // 32 KB
constexpr int kAtomBytes = 64 * kBK * 2;
constexpr int kSlabBytes = 32 * 128;
constexpr int kMaxGroups = 192;
constexpr size_t kSmem = (size_t)kRing * kStageBytes + (size_t)kEpiWarps * 2 * kSlabBytes + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// cta_group::2 form: the destination is this CTA's shared memory, the mbarrier may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_bar(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               :: "r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on ONE barrier (own or peer CTA, given as a cluster address) when the pair's MMAs are done
__device__ __forceinline__ void mma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_cluster_addr) : "memory");
}

struct Tile { int g, row0, m0, n0, kblocks; };

__global__ void __launch_bounds__(kThreads, 1)
wgrad_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const __grid_constant__ CUtensorMap tma_out, GemmArgs args) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[kRing], empty_bar[kRing], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;
  __shared__ int s_ntiles;
  __shared__ tq::Ring s_ring;
  __shared__ int s_cu[kMaxGroups + 1], s_act[kMaxGroups];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const bool leader = cr == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int G = args.G;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kRing; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 2 * kEpiWarps); }
    tq::init(&s_ring, 2 * kEpiWarps + 2);      // both CTAs' epilogue warps, the MMA issuer, the peer's producer
    fence_mbar_init();
    s_cu[0] = 0;
    for (int g = 0; g < G; ++g) s_cu[g + 1] = args.cu_seqlens[g];
    int n = 0;
    for (int g = 0; g < G; ++g) {
      const bool in = g >= args.g_begin && g < args.g_end;
      if (in && (s_cu[g + 1] > s_cu[g] || (!args.accumulate && g < args.zero_empty_below))) s_act[n++] = g;
    }
    s_ntiles = n * (args.M_w / 256) * (args.N / 256);
    tc::prefetch_tmap(&tma_a); tc::prefetch_tmap(&tma_b); tc::prefetch_tmap(&tma_out);
  }
  if (warp == 1) { tmem_alloc2(&s_tmem_base, 512); tmem_relinquish2(); }
  tc::fence_before_sync();
  __syncthreads();
  cluster_sync();                       // both CTAs' barriers exist before anyone touches the peer's
  tc::fence_after_sync();
  const uint32_t tmem_base = s_tmem_base;
  const int ntiles = s_ntiles;
  const bool dyn = args.sched != nullptr;

  auto fail = [&](int site, int tile) {
    if (atomicCAS(&args.status[0], 0, MEP_ERR_MBAR_TIMEOUT) == 0) {
      args.status[1] = 100 + site; args.status[2] = blockIdx.x; args.status[3] = tile;
      if (args.status_host) { *(volatile int32_t*)args.status_host = MEP_ERR_MBAR_TIMEOUT; __threadfence_system(); }
    }
    s_abort = 1;
  };
  auto get_tile = [&](int t, Tile& ti) {
    const int mblk = args.M_w / 256, per = mblk * (args.N / 256);
    const int ai = t / per, local = t - ai * per;
    const int g = s_act[ai];
    ti.g = g; ti.row0 = s_cu[g]; ti.kblocks = (s_cu[g + 1] - s_cu[g]) / kBK;
    ti.m0 = (local % mblk) * 256; ti.n0 = (local / mblk) * 256;
  };

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's halves; bytes are counted on the LEADER's barrier
    if (lane == 0) {
      int it = 0; Tile ti;
      tq::Scheduler<true> sched; tq::Consumer<true> follow;
      if (dyn) { if (leader) sched.setup(&s_ring, args.sched, ntiles); else follow.setup(&s_ring); }
      tq::Strided seq{pair, npairs, ntiles};
      for (int t; !s_abort && (t = !dyn ? seq.next() : leader ? sched.next(args.budget_ns) : follow.next(args.budget_ns)) != -1;) {
        if (t == -2) { fail(5, it); break; }
        get_tile(t, ti);
        for (int kb = 0; kb < ti.kblocks; ++kb, ++it) {
          const int s = it % kRing; const uint32_t ph = (uint32_t)(it / kRing) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, args.budget_ns)) { fail(1, t); break; }
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kHalfBytes;
          const uint32_t bar = mapa(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);     // both CTAs' bytes
          const int k = ti.row0 + kb * kBK;
          const int am = ti.m0 + (int)cr * 128, bn = ti.n0 + (int)cr * 128;
          tma_load_2d_bar(sa, &tma_a, am, k, bar);
          tma_load_2d_bar(sa + kAtomBytes, &tma_a, am + 64, k, bar);
          tma_load_2d_bar(sb, &tma_b, bn, k, bar);
          tma_load_2d_bar(sb + kAtomBytes, &tma_b, bn + 64, k, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only): one instruction drives both SMs
    if (leader && lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc_bf16(256, 256, true, true);
      uint32_t empty_peer[kRing], tfull_peer[2];
      for (int i = 0; i < kRing; ++i) empty_peer[i] = mapa(smem_u32(&empty_bar[i]), 1);
      for (int i = 0; i < 2; ++i) tfull_peer[i] = mapa(smem_u32(&tfull_bar[i]), 1);
      int it = 0, tcnt = 0; Tile ti;
      tq::Consumer<true> tiles; tiles.setup(&s_ring);
      tq::Strided seq{pair, npairs, ntiles};
      for (int t; !s_abort && (t = dyn ? tiles.next(args.budget_ns) : seq.next()) != -1; ++tcnt) {
        if (t == -2) { fail(6, tiles.n); break; }
        get_tile(t, ti);
        if (ti.kblocks == 0) { --tcnt; continue; }
        const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, args.budget_ns)) { fail(2, t); break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * 256;
        bool ok = true;
        for (int kb = 0; kb < ti.kblocks; ++kb, ++it) {
          const int s = it % kRing; const uint32_t ph = (uint32_t)(it / kRing) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, args.budget_ns)) { fail(3, t); ok = false; break; }
          tc::fence_after_sync();
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kHalfBytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            mma2_bf16(d_tmem, tc::smem_desc(sa + k * 2048, kAtomBytes, 1024), tc::smem_desc(sb + k * 2048, kAtomBytes, 1024),
                      idesc, (kb | k) ? 1u : 0u);
          mma2_commit(smem_u32(&empty_bar[s]));
          mma2_commit(empty_peer[s]);
        }
        if (!ok) break;
        mma2_commit(smem_u32(&tfull_bar[acc]));
        mma2_commit(tfull_peer[acc]);
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 rows of the 256-row tile
    const int q = warp & 3, half = (warp - 2) >> 2;
    const uint32_t stg = smem_u32(smem + (size_t)kRing * kStageBytes) + (uint32_t)(warp - 2) * 2 * kSlabBytes;
    const uint32_t tempty_leader[2] = {mapa(smem_u32(&tempty_bar[0]), 0), mapa(smem_u32(&tempty_bar[1]), 0)};
    int tcnt = 0, chunk_no = 0; Tile ti;
    tq::Consumer<true> tiles; tiles.setup(&s_ring);
    tq::Strided seq{pair, npairs, ntiles};
    for (;; ++tcnt) {
      int t = -1;
      if (!dyn) { if (!s_abort) t = seq.next(); }
      else {
        if (lane == 0 && !s_abort) { t = tiles.next(args.budget_ns); if (t == -2) fail(7, tiles.n); }
        t = __shfl_sync(0xffffffffu, t, 0);
      }
      if (t < 0) break;
      get_tile(t, ti);
      const int orow0 = ti.g * args.M_w + ti.m0 + (int)cr * 128 + q * 32;
      // optimizer in the epilogue: this group's weights are updated in place and no gradient is written
      const bool upd = args.upd_mask != nullptr && args.upd_mask[ti.g] != 0;
      if (ti.kblocks == 0) {           // empty group that must end with a zero gradient (nothing to update)
        if (!upd) {
          float* orow = (float*)args.out + (size_t)(orow0 + lane) * args.N + ti.n0 + half * 128;
          for (int j = 0; j < 32; ++j) reinterpret_cast<float4*>(orow)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        --tcnt; continue;
      }
      // A chunk is 32 rows x 32 columns. The accumulator arrives with lane = row; the weights are read and
      // written with four lanes per row instead (16 bytes each, eight rows per instruction: whole sectors),
      // so the chunk takes the same trip through the warp's shared-memory slab as a stored gradient does.
      const __nv_bfloat16* wbase = upd ? (const __nv_bfloat16*)args.upd_w + (size_t)orow0 * args.N + ti.n0 + (half * 4) * 32 : nullptr;
      auto wptr = [&](int i, int k) {
        return const_cast<__nv_bfloat16*>(wbase) + (size_t)((lane >> 2) + 8 * k) * args.N + i * 32 + (lane & 3) * 8;
      };
      int4 wv[4][4];
      if (upd) {                       // the tile's weights (this warp's 32 x 128 part): in flight while its MMAs finish
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int k = 0; k < 4; ++k) wv[i][k] = *reinterpret_cast<const int4*>(wptr(i, k));
      }
      const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
      int ok = 1;
      if (lane == 0) ok = mbar_wait_bounded(&tfull_bar[acc], aph, args.budget_ns) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) fail(4, t); break; }
      tc::fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256;
      // software pipeline over the four 32-column chunks of this warp: the TMEM load of chunk i+1 is
      // in flight while chunk i goes through shared memory; the accumulator is handed back to the
      // MMA warp as soon as the last chunk sits in registers
      uint32_t r[2][32];
      tc::tmem_ld32(taddr + (half * 4) * 32, r[0]);
#pragma unroll
      for (int i = 0; i < 4; ++i, ++chunk_no) {
        const int c = half * 4 + i;
        tc::tmem_ld_wait();
        if (i + 1 < 4) {
          tc::tmem_ld32(taddr + (c + 1) * 32, r[(i + 1) & 1]);
        } else {
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) remote_arrive(tempty_leader[acc]);
        }
        if (upd) {
          const uint32_t ubuf = stg + (uint32_t)(chunk_no & 1) * kSlabBytes;
          if (lane == 0) bulk_wait_read<0>();      // a gradient stored from this slab earlier has left it
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tc::st_shared_v4(ubuf + lane * 128 + ((j ^ (lane & 7)) << 4), r[i & 1][4 * j], r[i & 1][4 * j + 1], r[i & 1][4 * j + 2], r[i & 1][4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int R = (lane >> 2) + 8 * k, p2 = (lane & 3) * 2;
            const int4 g0 = tc::ld_shared_v4(ubuf + R * 128 + ((p2 ^ (R & 7)) << 4));
            const int4 g1 = tc::ld_shared_v4(ubuf + R * 128 + (((p2 + 1) ^ (R & 7)) << 4));
            const float gg[8] = {__int_as_float(g0.x), __int_as_float(g0.y), __int_as_float(g0.z), __int_as_float(g0.w),
                                 __int_as_float(g1.x), __int_as_float(g1.y), __int_as_float(g1.z), __int_as_float(g1.w)};
            int4 x = wv[i][k];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float2 f = __bfloat1622float2(h[e]);
              f.x = fmaf(-args.upd_lr, gg[2 * e], f.x);           // as in sgd_kernel
              f.y = fmaf(-args.upd_lr, gg[2 * e + 1], f.y);
              h[e] = __floats2bfloat162_rn(f.x, f.y);
            }
            *reinterpret_cast<int4*>(wptr(i, k)) = x;
          }
          continue;
        }
        const uint32_t buf = stg + (uint32_t)(chunk_no & 1) * kSlabBytes;
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          tc::st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), r[i & 1][4 * j], r[i & 1][4 * j + 1], r[i & 1][4 * j + 2], r[i & 1][4 * j + 3]);
        tc::fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (args.accumulate) tc::tma_reduce_add_2d(&tma_out, buf, ti.n0 + c * 32, orow0);
          else tc::tma_store_2d(&tma_out, buf, ti.n0 + c * 32, orow0);
          bulk_commit();
        }
      }
    }
    if (lane == 0) bulk_wait_all<0>();
  }

  // ---------------- teardown: nobody leaves while the peer may still signal into this CTA
  tc::fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc::fence_after_sync();
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
  if (leader && threadIdx.x == 0) tq::scheduler_done(args.sched, args.sched_ctas > 0 ? args.sched_ctas / 2 : npairs);
}

static int make_map2(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows, bool f32) {
  const DriverApi* d = driver(); if (!d) return -1;
  const int es_bytes = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  MEP_REQUIRE(((uintptr_t)base & 15) == 0 && (ld * es_bytes) % 16 == 0 && ld >= cols, "wgrad: tensor base/stride must be 16-byte aligned");
  MEP_CU_CHECK(d->TensorMapEncodeTiled(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                                       dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return 0;
}

}  // namespace w2

// =============================================================================================
// Token-major GEMMs (GATE_UP, DOWN, DGRAD, DGRAD_GU) on CTA pairs: a pair computes a 256-token x 256
// output tile; CTA r stages token rows [r*128, r*128+128) of the tile and its half of the weight
// tile (GATE_UP: CTA 0 the gate columns, CTA 1 the up columns). Expert groups are multiples of 128
// rows, so a group with an odd number of 128-row blocks ends with a pair tile whose second half
// belongs to the next group: that half is computed (against the wrong expert) and thrown away.
namespace t2 {

using namespace w2;
constexpr int kTokRing = 6, kTokEpi = 4, kTokThreads = 64 + 32 * kTokEpi;
constexpr size_t kTokSmem = (size_t)kTokRing * kStageBytes + (size_t)kTokEpi * 2 * kSlabBytes + 1024;

__device__ __forceinline__ void tma_load_3d_bar(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               :: "r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

struct TTile { int g, row0, valid1, n0; };

template <int MODE>
__global__ void __launch_bounds__(kTokThreads, 1)
tok_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b0,
                const __grid_constant__ CUtensorMap tma_b1, const __grid_constant__ CUtensorMap tma_out, GemmArgs args) {
  constexpr bool B_MN = MODE == GEMM_GATE_UP || MODE == GEMM_DOWN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[kTokRing], empty_bar[kTokRing], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;
  __shared__ int s_ntiles;
  __shared__ tq::Ring s_ring;
  __shared__ int s_cu[kMaxGroups + 1], s_start[kMaxGroups + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const bool leader = cr == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int G = args.G;
  const int nblk = MODE == GEMM_GATE_UP ? args.N / 128 : args.N / 256;
  const int kblocks = args.K / kBK;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kTokRing; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 2 * kTokEpi); }
    tq::init(&s_ring, 2 * kTokEpi + 2);
    fence_mbar_init();
    s_cu[0] = 0;
    for (int g = 0; g < G; ++g) s_cu[g + 1] = args.cu_seqlens[g];
    int run = 0;
    for (int g = 0; g < G; ++g) {
      s_start[g] = run;
      if (g >= args.g_begin && g < args.g_end) run += (((s_cu[g + 1] - s_cu[g]) / 128 + 1) / 2) * nblk;
    }
    s_start[G] = run; s_ntiles = run;
    tc::prefetch_tmap(&tma_a); tc::prefetch_tmap(&tma_b0); tc::prefetch_tmap(&tma_b1); tc::prefetch_tmap(&tma_out);
  }
  if (warp == 1) { tmem_alloc2(&s_tmem_base, 512); tmem_relinquish2(); }
  tc::fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc::fence_after_sync();
  const uint32_t tmem_base = s_tmem_base;
  const int ntiles = s_ntiles;
  const bool dyn = args.sched != nullptr;

  auto fail = [&](int site, int tile) {
    if (atomicCAS(&args.status[0], 0, MEP_ERR_MBAR_TIMEOUT) == 0) {
      args.status[1] = 200 + site; args.status[2] = blockIdx.x; args.status[3] = tile;
      if (args.status_host) { *(volatile int32_t*)args.status_host = MEP_ERR_MBAR_TIMEOUT; __threadfence_system(); }
    }
    s_abort = 1;
  };
  auto get_tile = [&](int t, int& gcur, TTile& ti) {
    while (gcur + 1 <= G && s_start[gcur + 1] <= t) ++gcur;
    const int g = gcur, beg = s_cu[g];
    const int mblk = (s_cu[g + 1] - beg) / 128, pairs = (mblk + 1) / 2;
    const int local = t - s_start[g];
    const int pt = local % pairs;
    ti.g = g; ti.row0 = beg + pt * 256; ti.valid1 = (2 * pt + 1 < mblk) ? 1 : 0;
    ti.n0 = (local / pairs) * (MODE == GEMM_GATE_UP ? 128 : 256);
  };

  if (warp == 0) {
    if (lane == 0) {
      int it = 0, gcur = 0; TTile ti;
      tq::Scheduler<true> sched; tq::Consumer<true> follow;
      if (dyn) { if (leader) sched.setup(&s_ring, args.sched, ntiles); else follow.setup(&s_ring); }
      tq::Strided seq{pair, npairs, ntiles};
      for (int t; !s_abort && (t = !dyn ? seq.next() : leader ? sched.next(args.budget_ns) : follow.next(args.budget_ns)) != -1;) {
        if (t == -2) { fail(5, it); break; }
        get_tile(t, gcur, ti);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kTokRing; const uint32_t ph = (uint32_t)(it / kTokRing) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, args.budget_ns)) { fail(1, t); break; }
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kHalfBytes;
          const uint32_t bar = mapa(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);
          const int k0 = kb * kBK;
          tma_load_2d_bar(sa, &tma_a, k0, ti.row0 + (int)cr * 128, bar);
          if (MODE == GEMM_GATE_UP) {
            tma_load_3d_bar(sb, cr == 0 ? &tma_b0 : &tma_b1, 0, ti.g * args.b_group_rows + k0, ti.n0 / 64, bar);
          } else if (MODE == GEMM_DOWN) {
            tma_load_3d_bar(sb, &tma_b0, 0, ti.g * args.b_group_rows + k0, (ti.n0 + (int)cr * 128) / 64, bar);
          } else if (MODE == GEMM_DGRAD) {
            tma_load_2d_bar(sb, &tma_b0, k0, ti.g * args.b_group_rows + ti.n0 + (int)cr * 128, bar);
          } else {
            const int half = args.K / 2;
            if (k0 < half) tma_load_2d_bar(sb, &tma_b0, k0, ti.g * args.b_group_rows + ti.n0 + (int)cr * 128, bar);
            else tma_load_2d_bar(sb, &tma_b1, k0 - half, ti.g * args.b_group_rows + ti.n0 + (int)cr * 128, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc_bf16(256, 256, false, B_MN);
      uint32_t empty_peer[kTokRing], tfull_peer[2];
      for (int i = 0; i < kTokRing; ++i) empty_peer[i] = mapa(smem_u32(&empty_bar[i]), 1);
      for (int i = 0; i < 2; ++i) tfull_peer[i] = mapa(smem_u32(&tfull_bar[i]), 1);
      int it = 0, tcnt = 0;
      tq::Consumer<true> tiles; tiles.setup(&s_ring);
      tq::Strided seq{pair, npairs, ntiles};
      for (int t; !s_abort && (t = dyn ? tiles.next(args.budget_ns) : seq.next()) != -1; ++tcnt) {
        if (t == -2) { fail(6, tiles.n); break; }
        const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, args.budget_ns)) { fail(2, t); break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * 256;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kTokRing; const uint32_t ph = (uint32_t)(it / kTokRing) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, args.budget_ns)) { fail(3, t); ok = false; break; }
          tc::fence_after_sync();
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kHalfBytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t ad = tc::smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? tc::smem_desc(sb + k * 2048, kAtomBytes, 1024) : tc::smem_desc(sb + k * 32, 16, 1024);
            mma2_bf16(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
          }
          mma2_commit(smem_u32(&empty_bar[s]));
          mma2_commit(empty_peer[s]);
        }
        if (!ok) break;
        mma2_commit(smem_u32(&tfull_bar[acc]));
        mma2_commit(tfull_peer[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    const int r_in_half = q * 32 + lane;
    const uint32_t stg = smem_u32(smem + (size_t)kTokRing * kStageBytes) + (uint32_t)(warp - 2) * 2 * kSlabBytes;
    const uint32_t tempty_leader[2] = {mapa(smem_u32(&tempty_bar[0]), 0), mapa(smem_u32(&tempty_bar[1]), 0)};
    int tcnt = 0, gcur = 0, chunk_no = 0; TTile ti;
    tq::Consumer<true> tiles; tiles.setup(&s_ring);
    tq::Strided seq{pair, npairs, ntiles};
    for (;; ++tcnt) {
      int t = -1;
      if (!dyn) { if (!s_abort) t = seq.next(); }
      else {
        if (lane == 0 && !s_abort) { t = tiles.next(args.budget_ns); if (t == -2) fail(7, tiles.n); }
        t = __shfl_sync(0xffffffffu, t, 0);
      }
      if (t < 0) break;
      get_tile(t, gcur, ti);
      const int acc = tcnt & 1; const uint32_t aph = (uint32_t)(tcnt >> 1) & 1u;
      int ok = 1;
      if (lane == 0) ok = mbar_wait_bounded(&tfull_bar[acc], aph, args.budget_ns) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) fail(4, t); break; }
      tc::fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256;
      const bool live = cr == 0 || ti.valid1;            // second half of an odd group: discard
      const int hrow0 = ti.row0 + (int)cr * 128;
      if (!live) {
        // nothing to write; the accumulator is handed back below
      } else if (MODE == GEMM_GATE_UP) {
        const size_t row = (size_t)hrow0 + r_in_half;
        __nv_bfloat16* orow = (__nv_bfloat16*)args.out + row * args.ldo + ti.n0;
        __nv_bfloat16* grow = args.out2 ? (__nv_bfloat16*)args.out2 + row * (size_t)(2 * args.N) + ti.n0 : nullptr;
        const float sc = args.row_scale ? args.row_scale[row] : 1.f;
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
      } else {
        const size_t row = (size_t)hrow0 + r_in_half;
        const float sc = (MODE == GEMM_DOWN && args.row_scale) ? args.row_scale[row] : 1.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c, ++chunk_no) {
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
            tc::tma_store_2d(&tma_out, buf, ti.n0 + c * 64, hrow0 + q * 32);
            bulk_commit();
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) remote_arrive(tempty_leader[acc]);
    }
    if (lane == 0) bulk_wait_all<0>();
  }

  tc::fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc::fence_after_sync();
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
  if (leader && threadIdx.x == 0) tq::scheduler_done(args.sched, args.sched_ctas > 0 ? args.sched_ctas / 2 : npairs);
}

static int make_map_mn3(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int atoms) {
  const DriverApi* d = driver(); if (!d) return -1;
  MEP_REQUIRE(cols % 64 == 0, "gemm: MN-major operand width %lld must be a multiple of 64", (long long)cols);
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, 64, (cuuint32_t)atoms};
  cuuint32_t es[3] = {1, 1, 1};
  MEP_CU_CHECK(d->TensorMapEncodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return 0;
}

}  // namespace t2
}  // namespace mep

// dW[g] (+)= X_g^T dY_g on CTA pairs. x: [rows, M_w] bf16 (pitch x_ld), dy: [rows, N] bf16 (pitch dy_ld),
// args.out: fp32 [G, M_w, N]. Requires M_w % 256 == 0, N % 256 == 0 and an even CTA count.
extern "C" int mep_grouped_wgrad_2cta(const void* x, int64_t rows, int64_t x_ld, const void* dy, int64_t dy_ld,
                                      const mep::GemmArgs* args_in, int num_ctas, cudaStream_t stream) {
  using namespace mep;
  GemmArgs args = *args_in;
  MEP_REQUIRE(args.G >= 1 && args.G <= w2::kMaxGroups, "wgrad: G=%d out of range", args.G);
  MEP_REQUIRE(args.M_w % 256 == 0 && args.N % 256 == 0, "wgrad (2-CTA): weight shape [%d,%d] must be multiples of 256", args.M_w, args.N);
  num_ctas &= ~1;
  MEP_REQUIRE(num_ctas >= 2, "wgrad (2-CTA): needs at least two CTAs");
  CUtensorMap ma, mb, mo;
  if (w2::make_map2(&ma, x, rows, args.M_w, x_ld, 64, 64, false)) return -1;
  if (w2::make_map2(&mb, dy, rows, args.N, dy_ld, 64, 64, false)) return -1;
  if (w2::make_map2(&mo, args.out, (int64_t)args.G * args.M_w, args.N, args.N, 32, 32, true)) return -1;
  MEP_CUDA_CHECK(cudaFuncSetAttribute(w2::wgrad_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)w2::kSmem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_ctas); cfg.blockDim = dim3(w2::kThreads); cfg.dynamicSmemBytes = w2::kSmem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  MEP_CUDA_CHECK(cudaLaunchKernelEx(&cfg, w2::wgrad_2cta_kernel, ma, mb, mo, args));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

// Token-major grouped GEMMs on CTA pairs; same contract as mep_grouped_gemm for modes 0-3.
extern "C" int mep_grouped_gemm_2cta(int mode, const void* a, int64_t a_rows, int64_t a_cols, int64_t a_ld,
                                     const void* b0, const void* b1, int64_t b_rows, int64_t b_cols, int64_t b_ld,
                                     const mep::GemmArgs* args_in, int num_ctas, cudaStream_t stream) {
  using namespace mep;
  GemmArgs args = *args_in;
  MEP_REQUIRE(mode >= GEMM_GATE_UP && mode <= GEMM_DGRAD_GU, "gemm (2-CTA): mode %d not supported", mode);
  MEP_REQUIRE(args.G >= 1 && args.G <= w2::kMaxGroups, "gemm: G=%d out of range", args.G);
  MEP_REQUIRE(args.K % 64 == 0 && args.N % (mode == GEMM_GATE_UP ? 128 : 256) == 0, "gemm (2-CTA): K=%d N=%d not tileable", args.K, args.N);
  num_ctas &= ~1;
  MEP_REQUIRE(num_ctas >= 2, "gemm (2-CTA): needs at least two CTAs");
  const bool b_mn = mode == GEMM_GATE_UP || mode == GEMM_DOWN;
  CUtensorMap ma, mb0, mb1, mo;
  if (w2::make_map2(&ma, a, a_rows, a_cols, a_ld, 64, 128, false)) return -1;
  if (b_mn) { if (t2::make_map_mn3(&mb0, b0, b_rows, b_cols, b_ld, 2)) return -1; }
  else      { if (w2::make_map2(&mb0, b0, b_rows, b_cols, b_ld, 64, 128, false)) return -1; }
  if (b1) { if (b_mn ? t2::make_map_mn3(&mb1, b1, b_rows, b_cols, b_ld, 2) : w2::make_map2(&mb1, b1, b_rows, b_cols, b_ld, 64, 128, false)) return -1; }
  else mb1 = mb0;
  if (mode == GEMM_GATE_UP) mo = ma;
  else if (w2::make_map2(&mo, args.out, a_rows, args.N, args.ldo, 64, 32, false)) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_ctas); cfg.blockDim = dim3(t2::kTokThreads); cfg.dynamicSmemBytes = t2::kTokSmem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
#define MEP_T2_CASE(M)                                                                                                   \
  case M:                                                                                                                \
    MEP_CUDA_CHECK(cudaFuncSetAttribute(t2::tok_2cta_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t2::kTokSmem)); \
    MEP_CUDA_CHECK(cudaLaunchKernelEx(&cfg, t2::tok_2cta_kernel<M>, ma, mb0, mb1, mo, args));                              \
    break;
  switch (mode) {
    MEP_T2_CASE(GEMM_GATE_UP) MEP_T2_CASE(GEMM_DOWN) MEP_T2_CASE(GEMM_DGRAD) MEP_T2_CASE(GEMM_DGRAD_GU)
    default: return set_error("gemm (2-CTA): unknown mode %d", mode);
  }
#undef MEP_T2_CASE
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}
