// reduce_grad: owner-pull reduction of redundant experts' weight gradients.
//
// Counterpart of the reference's GradReduceKernel (moonep/grad_reduce.py:46-389), which is
// launched three times (gate, up, down); here ONE launch handles all projections:
//   1. prescan of experts_to_copy -> per local expert the list of (rank, slot) pairs holding
//      one of its replicas, sorted ascending;
//   2. local_grad[e] += reduce[d0, b0] + reduce[d1, b1] + ...  in that fixed order (bitwise
//      reproducible), peer slots read with plain 16-byte loads;
//   3. cross-rank barrier (every owner has consumed its replicas);
//   4. each rank zeroes ITS OWN consumed slots for the next microbatch.
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
  int32_t pad;
  ReduceTensor t[3];
};
struct GradReduceArgsPack { GradReduceArgs a[MEP_MAX_VRANKS]; };

constexpr int kRedThreads = 512;
constexpr int kRedVec = 4;            // float4 per thread and pass
constexpr int64_t kRedChunk = (int64_t)kRedThreads * kRedVec * 4;   // floats per work unit

__device__ __forceinline__ float4 f4add(float4 a, const int4& b) {
  a.x += __int_as_float(b.x); a.y += __int_as_float(b.y); a.z += __int_as_float(b.z); a.w += __int_as_float(b.w);
  return a;
}

__global__ void __launch_bounds__(kRedThreads, 1) grad_reduce_kernel(MepCtxPack P, GradReduceArgsPack A) {
  const MepRankCtx c = *P.ctx[blockIdx.y];   // by value: fields stay in registers across asm memory clobbers
  const GradReduceArgs& a = A.a[blockIdx.y];
  extern __shared__ int s_mem[];
  const int nb = gridDim.x, tid = threadIdx.x, nt = blockDim.x;
  const int R = c.R, epn = c.epn, lo = c.rank * epn;
  int* s_cnt = s_mem;                 // [epn]
  int* s_off = s_mem + epn;           // [epn + 1]
  int* s_act = s_off + epn + 1;       // [epn] active local experts
  int* s_src = s_act + epn;           // [R * epn] sources grouped per expert
  __shared__ int s_nact;

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

  int64_t chunks_per_exp = 0;
  for (int t = 0; t < a.ntensors; ++t) chunks_per_exp += (a.t[t].expert_elems + kRedChunk - 1) / kRedChunk;
  const int64_t total = (int64_t)nact * chunks_per_exp;
  for (int64_t u = blockIdx.x; u < total; u += nb) {
    const int ai = (int)(u / chunks_per_exp);
    int64_t ck = u - (int64_t)ai * chunks_per_exp;
    int t = 0;
    for (;; ++t) { const int64_t n = (a.t[t].expert_elems + kRedChunk - 1) / kRedChunk; if (ck < n) break; ck -= n; }
    const ReduceTensor& T = a.t[t];
    const int le = s_act[ai];
    const int* srcs = s_src + s_off[le]; const int ns = s_off[le + 1] - s_off[le];
    const int64_t beg = ck * kRedChunk;
    const int64_t len = (T.expert_elems - beg) < kRedChunk ? (T.expert_elems - beg) : kRedChunk;
    float* lp = T.local + (int64_t)le * T.expert_elems + beg;
    const int64_t ebytes = T.expert_elems * 4;
    const int nvec = (int)(len >> 2);
    for (int v0 = 0; v0 < nvec; v0 += kRedVec * nt) {
      float4 acc[kRedVec];
#pragma unroll
      for (int q = 0; q < kRedVec; ++q) {
        const int v = v0 + q * nt + tid;
        acc[q] = v < nvec ? *reinterpret_cast<const float4*>(lp + (size_t)v * 4) : make_float4(0, 0, 0, 0);
      }
      for (int j0 = 0; j0 < ns; j0 += 2) {          // 2 sources x kRedVec vectors in flight per thread
        int4 x[2][kRedVec];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const bool on = j0 + j < ns;
          const int idx = on ? srcs[j0 + j] : 0, d = idx / epn, b = idx - d * epn;
          const char* rp = T.pool + (int64_t)d * T.rank_stride + (int64_t)b * ebytes + beg * 4;
#pragma unroll
          for (int q = 0; q < kRedVec; ++q) {
            const int v = v0 + q * nt + tid;
            x[j][q] = make_int4(0, 0, 0, 0);
            if (on && v < nvec) x[j][q] = ld_peer_v4(rp + (size_t)v * 16);
          }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (j0 + j < ns) {
#pragma unroll
            for (int q = 0; q < kRedVec; ++q) acc[q] = f4add(acc[q], x[j][q]);
          }
      }
#pragma unroll
      for (int q = 0; q < kRedVec; ++q) {
        const int v = v0 + q * nt + tid;
        if (v < nvec) *reinterpret_cast<float4*>(lp + (size_t)v * 4) = acc[q];
      }
    }
    for (int64_t i = ((int64_t)nvec << 2) + tid; i < len; i += nt) {   // ragged tail
      float acc = lp[i];
      for (int j = 0; j < ns; ++j) {
        const int idx = srcs[j], d = idx / epn, b = idx - d * epn;
        acc += __ldcg(reinterpret_cast<const float*>(T.pool + (int64_t)d * T.rank_stride + (int64_t)b * ebytes) + beg + i);
      }
      lp[i] = acc;
    }
  }

  if (!cross_rank_barrier(c, nb, 1, MEP_K_GRAD_REDUCE, 10)) return;

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

}  // namespace mep

extern "C" int mep_launch_grad_reduce(int nv, const MepRankCtx* const* ctxs, const mep::GradReduceArgs* args,
                                      int num_sms, int R, int epn, cudaStream_t stream) {
  MEP_REQUIRE(nv >= 1 && nv <= MEP_MAX_VRANKS, "grad_reduce: nv=%d out of range", nv);
  MepCtxPack P = {}; mep::GradReduceArgsPack A = {};
  for (int i = 0; i < nv; ++i) { P.ctx[i] = ctxs[i]; A.a[i] = args[i]; }
  const size_t smem = ((size_t)3 * epn + 1 + (size_t)R * epn) * sizeof(int);
  MEP_REQUIRE(smem <= 160 * 1024, "grad_reduce: R*epn=%d exceeds the source-list capacity", R * epn);
  return mep::launch_cooperative(mep::grad_reduce_kernel, dim3(num_sms, nv), dim3(mep::kRedThreads), smem,
                                 stream, false, P, A);
}
