// reduce_grad: owner-pull reduction of redundant experts' weight gradients.
//
// Counterpart of the reference's GradReduceKernel (moonep/grad_reduce.py:46-389), which is
// launched three times (gate, up, down); here ONE launch handles all projections:
//   1. prescan of experts_to_copy -> per local expert the list of (rank, slot) pairs holding
//      one of its replicas, sorted ascending;
//   1b. optional entry barrier: a replica may only be read once its holder's weight-gradient GEMM
//      has finished (the reference leaves this to the caller, api.py:1154-1158; here the public
//      call does it unless told otherwise, since nothing else orders the ranks at that point);
//   2. local_grad[e] += reduce[d0, b0] + reduce[d1, b1] + ...  in that fixed order (bitwise
//      reproducible), peer slots read with untiled bulk copies into shared memory (no multicast);
//   3. cross-rank barrier (every owner has consumed its replicas);
//   4. each rank zeroes ITS OWN consumed slots for the next microbatch (steps 3 and 4 can be
//      switched off by a caller whose next weight-gradient GEMM overwrites the slots it uses).
#include "prims.cuh"
#include "../host/launch.h"

namespace mep {

struct ReduceTensor {
  float* local;               // [epn, expert_elems] fp32 parameter grads
  char* pool;                 // rank 0's slot 0 of the [R, epn, ...] reduce view
  int64_t expert_elems;
  int64_t rank_stride;        // bytes
};
struct GradReduceArgs {
  const int32_t* etc;
  int32_t ntensors;
  int32_t flags;              // bit 0: cross-rank barrier before the first peer read; bit 1: leave the consumed slots as
                              // they are (no second barrier either); bit 2: second barrier, but the slots are cleared
                              // by grad_clear_kernel on all SMs afterwards instead of by this kernel's few CTAs
  ReduceTensor t[3];
};
struct GradReduceArgsPack { GradReduceArgs a[MEP_MAX_VRANKS]; };

constexpr int kRedThreads = 384;          // 12 warps
constexpr int kRedSlots = 32;             // 16-byte vectors per lane in one warp stage
constexpr int kRedDepth = 4;              // units in flight per warp when an expert has <= 8 replicas

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_but() {   // all but the newest N groups are done
  asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ float4 f4add(float4 a, const int4& b) {
  a.x += __int_as_float(b.x); a.y += __int_as_float(b.y); a.z += __int_as_float(b.z); a.w += __int_as_float(b.w);
  return a;
}

__global__ void __launch_bounds__(kRedThreads, 1) grad_reduce_kernel(MepCtxPack P, GradReduceArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const GradReduceArgs& a = A.a[blockIdx.y];
  extern __shared__ __align__(128) int s_mem[];
  const int nb = gridDim.x, tid = threadIdx.x, nt = blockDim.x;
  const int R = c.R, epn = c.epn, lo = c.rank * epn;
  int* s_cnt = s_mem;                 // [epn]
  int* s_off = s_mem + epn;           // [epn + 1]
  int* s_act = s_off + epn + 1;       // [epn] active local experts
  int* s_src = s_act + epn;           // [R * epn] sources grouped per expert
  unsigned char* s_stage = reinterpret_cast<unsigned char*>(s_mem) + (((size_t)(3 * epn + 1 + R * epn) * 4 + 127) & ~(size_t)127);
  __shared__ int s_nact;
  __shared__ __align__(8) uint64_t s_bar[(kRedThreads / 32) * kRedDepth];
  if (tid < (kRedThreads / 32) * kRedDepth) mbar_init(&s_bar[tid], 1);
  fence_mbar_init();

  for (int i = tid; i < epn; i += nt) s_cnt[i] = 0;
  if (tid == 0) s_nact = 0;
  __syncthreads();
  for (int i = tid; i < R * epn; i += nt) {
    const int e = a.etc[i];
    if (e >= lo && e < lo + epn && i / epn != c.rank) atomicAdd(&s_cnt[e - lo], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int i = 0; i < epn; ++i) { s_off[i] = run; run += s_cnt[i]; if (s_cnt[i]) s_act[s_nact++] = i; s_cnt[i] = 0; }
    s_off[epn] = run;
  }
  __syncthreads();
  for (int i = tid; i < R * epn; i += nt) {
    const int e = a.etc[i];
    if (e >= lo && e < lo + epn && i / epn != c.rank) s_src[s_off[e - lo] + atomicAdd(&s_cnt[e - lo], 1)] = i;
  }
  __syncthreads();
  for (int i = tid; i < epn; i += nt) {       // ascending (rank, slot) => fixed summation order
    int* l = s_src + s_off[i]; const int n = s_off[i + 1] - s_off[i];
    for (int x = 1; x < n; ++x) { const int v = l[x]; int y = x - 1; while (y >= 0 && l[y] > v) { l[y + 1] = l[y]; --y; } l[y + 1] = v; }
  }
  __syncthreads();
  const int nact = s_nact;
  if (tid == 0) trace_mark(c, MEP_K_GRAD_REDUCE, 1);
  if ((a.flags & 1) && !cross_rank_barrier(c, nb, kWeightLaneRow, MEP_K_GRAD_REDUCE, 5)) return;
  if (tid == 0) trace_mark(c, MEP_K_GRAD_REDUCE, 2);

  // Each warp owns a 16 KB shared-memory stage of 32 slots (one slot = one 16-byte vector per
  // lane). A work unit is P vectors per lane of ONE expert matrix: the warp fetches them from EVERY
  // replica with bulk copies issued by its first lane (nothing is held in registers while the NVLink
  // reads are in flight), loads the same vectors of the local grad, waits for the copies and adds the
  // replicas in list order. With few replicas (the common case: one or two) a unit fills only part of
  // the stage, so the stage is used as a ring of kRedDepth units and the copies of the next units are
  // already under way while this one is summed: 12 warps x 12 KB stay in flight per SM. An expert with
  // more than 8 replicas takes the unpipelined path below (one 16-byte copy per lane and vector).
  const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int gw = blockIdx.x * nwarps + warp, gnw = nb * nwarps;
  const uint32_t stage = smem_u32(s_stage) + (uint32_t)warp * (kRedSlots * 32 * 16);
  const unsigned char* stage_g = s_stage + (size_t)warp * (kRedSlots * 32 * 16);
  uint32_t ring_phase = 0;       // parity of each ring slot's barrier
  uint32_t ring_pending = 0;     // ring slots with a copy issued and not yet waited for
  bool failed = false;
  for (int ai = 0; ai < nact && !failed; ++ai) {
    const int le = s_act[ai];
    const int* srcs = s_src + s_off[le]; const int ns = s_off[le + 1] - s_off[le];
    const bool ring = ns * kRedDepth <= kRedSlots;               // up to 8 replicas: pipelined path
    int P = kRedSlots / (ring ? ns * kRedDepth : ns); if (P > 8) P = 8; if (P < 1) P = 1;
    const int npass_src = (ns + kRedSlots - 1) / kRedSlots;     // > 1 only if an expert has more than 32 replicas
    for (int t = 0; t < a.ntensors && !failed; ++t) {
      const ReduceTensor& T = a.t[t];
      const int64_t ebytes = T.expert_elems * 4;
      const int64_t nvec = T.expert_elems >> 2;
      float* lp = T.local + (int64_t)le * T.expert_elems;
      const int64_t unit_vecs = 32 * (int64_t)P;
      const int64_t nunits = (nvec + unit_vecs - 1) / unit_vecs;
      if (ring) {
        const int uslots = ns * P;                                // slots of one unit
        uint64_t* bars = s_bar + warp * kRedDepth;
        // One bulk copy per replica and unit: the unit's vectors are contiguous in the slot and in the
        // stage (measured on two B200s, 176 MB from one peer: 780 GB/s this way against 560 GB/s with one
        // 16-byte asynchronous copy per lane and vector).
        auto issue = [&](int64_t u, int r) {
          ring_pending |= 1u << r;
          if (lane != 0) return;
          const int64_t v0 = u * unit_vecs;
          const int64_t left = nvec - v0;
          const uint32_t bytes = (uint32_t)((left < unit_vecs ? left : unit_vecs) * 16);
          mbar_expect_tx(&bars[r], bytes * (uint32_t)ns);
          for (int j = 0; j < ns; ++j) {
            const int idx = srcs[j], d = idx / epn, b = idx - d * epn;
            const char* rp = T.pool + (int64_t)d * T.rank_stride + (int64_t)b * ebytes;
            bulk_g2s(s_stage + (size_t)warp * (kRedSlots * 32 * 16) + (size_t)((r * uslots + j * P) * 32) * 16, rp + v0 * 16, bytes, &bars[r]);
          }
        };
        // Ring slot r has a barrier of its own; a slot is refilled kRedDepth-1 steps ahead of its use.
        int64_t ui = gw;
        for (int k = 0; k < kRedDepth - 1; ++k, ui += gnw) { if (ui < nunits) issue(ui, k); }
        int r = 0;
        for (int64_t u = gw; u < nunits; u += gnw, ui += gnw) {
          int rn = r + kRedDepth - 1; if (rn >= kRedDepth) rn -= kRedDepth;
          __syncwarp();                // every lane has finished reading the slot that is refilled now
          if (ui < nunits) issue(ui, rn);
          const int64_t v0 = u * unit_vecs;
          float4 acc[8];
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const int64_t v = v0 + (int64_t)p * 32 + lane;
            acc[p] = (p < P && v < nvec) ? *reinterpret_cast<const float4*>(lp + v * 4) : make_float4(0, 0, 0, 0);
          }
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[r], (ring_phase >> r) & 1u, c.wait_budget_ns))) {
            if (lane == 0) report(c, MEP_ERR_MBAR_TIMEOUT, MEP_K_GRAD_REDUCE, 20, r, (uint32_t)u, 0);
            // give the copies issued into the other ring slots their time too before the stage goes away
            for (int k = 0; k < kRedDepth; ++k)
              if (k != r && ((ring_pending >> k) & 1u)) mbar_wait_bounded(&bars[k], (ring_phase >> k) & 1u, c.wait_budget_ns);
            failed = true; break;
          }
          ring_phase ^= 1u << r; ring_pending &= ~(1u << r);
          for (int j = 0; j < ns; ++j)
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              const int64_t v = v0 + (int64_t)p * 32 + lane;
              if (p < P && v < nvec)
                acc[p] = f4add(acc[p], *reinterpret_cast<const int4*>(stage_g + (size_t)((r * uslots + j * P + p) * 32 + lane) * 16));
            }
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const int64_t v = v0 + (int64_t)p * 32 + lane;
            if (p < P && v < nvec) *reinterpret_cast<float4*>(lp + v * 4) = acc[p];
          }
          if (++r == kRedDepth) r = 0;
        }
        __syncwarp();                // the last unit's reads are done before another tensor refills the ring
      } else
      for (int64_t u = gw; u < nunits; u += gnw) {
        const int64_t v0 = u * unit_vecs;
        float4 acc[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const int64_t v = v0 + (int64_t)p * 32 + lane;
          acc[p] = (p < P && v < nvec) ? *reinterpret_cast<const float4*>(lp + v * 4) : make_float4(0, 0, 0, 0);
        }
        for (int sp = 0; sp < npass_src; ++sp) {
          const int j_beg = sp * kRedSlots, j_end = ns < j_beg + kRedSlots ? ns : j_beg + kRedSlots;
          for (int j = j_beg; j < j_end; ++j) {
            const int idx = srcs[j], d = idx / epn, b = idx - d * epn;
            const char* rp = T.pool + (int64_t)d * T.rank_stride + (int64_t)b * ebytes;
            for (int p = 0; p < P; ++p) {
              const int64_t v = v0 + (int64_t)p * 32 + lane;
              if (v < nvec) cp_async16(stage + (uint32_t)(((j - j_beg) * P + p) * 32 + lane) * 16, rp + v * 16);
            }
          }
          cp_async_commit_wait_all();
          for (int j = j_beg; j < j_end; ++j)
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              const int64_t v = v0 + (int64_t)p * 32 + lane;
              if (p < P && v < nvec)
                acc[p] = f4add(acc[p], *reinterpret_cast<const int4*>(stage_g + (size_t)(((j - j_beg) * P + p) * 32 + lane) * 16));
            }
        }
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const int64_t v = v0 + (int64_t)p * 32 + lane;
          if (p < P && v < nvec) *reinterpret_cast<float4*>(lp + v * 4) = acc[p];
        }
      }
      if (blockIdx.x == 0) {     // ragged tail (expert size not a multiple of four floats)
        for (int64_t i = (nvec << 2) + tid; i < T.expert_elems; i += nt) {
          float accs = lp[i];
          for (int j = 0; j < ns; ++j) {
            const int idx = srcs[j], d = idx / epn, b = idx - d * epn;
            accs += __ldcg(reinterpret_cast<const float*>(T.pool + (int64_t)d * T.rank_stride + (int64_t)b * ebytes) + i);
          }
          lp[i] = accs;
        }
      }
    }
  }

  if (tid == 0) trace_mark(c, MEP_K_GRAD_REDUCE, 3);
  if (a.flags & 2) return;
  if (!cross_rank_barrier(c, nb, kWeightLaneRow, MEP_K_GRAD_REDUCE, 10)) return;
  if (tid == 0) trace_mark(c, MEP_K_GRAD_REDUCE, 4);
  if (a.flags & 4) return;

  // clear my own consumed slots
  const int4 z = make_int4(0, 0, 0, 0);
  for (int b = 0; b < epn; ++b) {
    if (a.etc[(size_t)c.rank * epn + b] < 0) continue;
    for (int t = 0; t < a.ntensors; ++t) {
      const ReduceTensor& T = a.t[t];
      char* sp = T.pool + (int64_t)c.rank * T.rank_stride + (int64_t)b * T.expert_elems * 4;
      const int64_t nvec = T.expert_elems >> 2;
      for (int64_t v = (int64_t)blockIdx.x * nt + tid; v < nvec; v += (int64_t)nb * nt) st_v4(sp + v * 16, z);
      if (blockIdx.x == 0) for (int64_t i = (nvec << 2) + tid; i < T.expert_elems; i += nt) reinterpret_cast<float*>(sp)[i] = 0.f;
    }
  }
}

// Zero this rank's consumed slots (the slots named by experts_to_copy[rank, :]). Launched behind
// grad_reduce_kernel, whose second barrier guarantees that every owner has read them: a plain grid
// over all SMs, because the 32 CTAs of the cooperative kernel can only store ~55 GB/s each.
__global__ void __launch_bounds__(256) grad_clear_kernel(MepCtxPack P, GradReduceArgsPack A) {
  const MepRankCtx* cp = P.ctx[blockIdx.y];
  const GradReduceArgs& a = A.a[blockIdx.y];
  const int epn = cp->epn, rank = cp->rank;
  const int4 z = make_int4(0, 0, 0, 0);
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, gnt = (int64_t)gridDim.x * blockDim.x;
  for (int b = 0; b < epn; ++b) {
    if (a.etc[(size_t)rank * epn + b] < 0) continue;
    for (int t = 0; t < a.ntensors; ++t) {
      const ReduceTensor& T = a.t[t];
      char* sp = T.pool + (int64_t)rank * T.rank_stride + (int64_t)b * T.expert_elems * 4;
      const int64_t nvec = T.expert_elems >> 2;
      for (int64_t v = gtid; v < nvec; v += gnt) st_v4(sp + v * 16, z);
      if (blockIdx.x == 0) for (int64_t i = (nvec << 2) + threadIdx.x; i < T.expert_elems; i += blockDim.x) reinterpret_cast<float*>(sp)[i] = 0.f;
    }
  }
}

}  // namespace mep

extern "C" int mep_launch_grad_clear(int nv, const MepRankCtx* const* ctxs, const mep::GradReduceArgs* args,
                                     int num_blocks, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "grad_clear: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::GradReduceArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  return mep::launch_plain(mep::grad_clear_kernel, dim3(num_blocks, nv), dim3(256), 0, stream, P, A);
}

extern "C" int mep_launch_grad_reduce(int nv, const MepRankCtx* const* ctxs, const mep::GradReduceArgs* args,
                                      int num_sms, int R, int epn, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "grad_reduce: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::GradReduceArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  const size_t lists = ((((size_t)3 * epn + 1 + (size_t)R * epn) * sizeof(int)) + 127) & ~(size_t)127;
  MEP_REQUIRE(lists <= 30 * 1024, "grad_reduce: R*epn=%d exceeds the source-list capacity", R * epn);
  const size_t smem = lists + (size_t)(mep::kRedThreads / 32) * mep::kRedSlots * 32 * 16;
  return mep::launch_cooperative(mep::grad_reduce_kernel, dim3(num_sms, nv), dim3(mep::kRedThreads), smem,
                                 stream, false, P, A);
}

MEP_EXPORT_SIZEOF(GradReduceArgs, mep::GradReduceArgs)
