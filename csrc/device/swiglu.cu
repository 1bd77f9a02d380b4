// Element-wise companions of the grouped GEMM (memory-bound, one pass each):
//   swiglu_bwd: from dA (= dY Wd^T, gradient w.r.t. the weighted activation), the saved
//               pre-activations (gate | up) and the per-row route weight w it produces
//               [dGate | dUp] and the route-weight gradient dW[row] = sum_j dA[row,j] * silu(g)*u.
//   sgd_step:   p -= lr * g for bf16 parameters with fp32 gradients (benchmark optimizer).
// Only rows below cu_seqlens[G-1] are defined; rows beyond are skipped.
#include "prims.cuh"
#include "../host/launch.h"

namespace mep {

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dA, const __nv_bfloat16* __restrict__ gu,
                                                         const float* __restrict__ w, __nv_bfloat16* __restrict__ dgu,
                                                         float* __restrict__ dw, const int32_t* __restrict__ cu_seqlens,
                                                         int G, int Hp) {
  const int nrows = cu_seqlens[G - 1];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nvec = Hp >> 3;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < nrows; row += gridDim.x * wpb) {
    const float wr = w ? w[row] : 1.f;
    const __nv_bfloat16* da = dA + (size_t)row * Hp;
    const __nv_bfloat16* g = gu + (size_t)row * 2 * Hp;
    const __nv_bfloat16* u = g + Hp;
    __nv_bfloat16* dg = dgu + (size_t)row * 2 * Hp;
    __nv_bfloat16* du = dg + Hp;
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const int4 xa = ld_nc_v4(da + v * 8), xg = ld_nc_v4(g + v * 8), xu = ld_nc_v4(u + v * 8);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&xa);
      const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&xg);
      const __nv_bfloat162* pu = reinterpret_cast<const __nv_bfloat162*>(&xu);
      int4 og, ou;
      __nv_bfloat162* qg = reinterpret_cast<__nv_bfloat162*>(&og);
      __nv_bfloat162* qu = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(pa[i]), fg = __bfloat1622float2(pg[i]), fu = __bfloat1622float2(pu[i]);
        float rg[2], ru[2];
        const float a_[2] = {fa.x, fa.y}, g_[2] = {fg.x, fg.y}, u_[2] = {fu.x, fu.y};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float sig = 1.f / (1.f + __expf(-g_[j]));
          const float silu = g_[j] * sig;
          dot += a_[j] * silu * u_[j];
          const float d = a_[j] * wr;
          rg[j] = d * u_[j] * sig * (1.f + g_[j] * (1.f - sig));
          ru[j] = d * silu;
        }
        qg[i] = __floats2bfloat162_rn(rg[0], rg[1]);
        qu[i] = __floats2bfloat162_rn(ru[0], ru[1]);
      }
      st_v4(dg + v * 8, og);
      st_v4(du + v * 8, ou);
    }
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0 && dw) dw[row] = dot;
  }
}

__global__ void __launch_bounds__(256) sgd_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ g, float lr, int64_t n8) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    int4 x = *reinterpret_cast<const int4*>(p + i * 8);
    const float4 g0 = *reinterpret_cast<const float4*>(g + i * 8), g1 = *reinterpret_cast<const float4*>(g + i * 8 + 4);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      f.x = fmaf(-lr, gg[2 * k], f.x); f.y = fmaf(-lr, gg[2 * k + 1], f.y);      // the form wgrad's fused update uses
      h[k] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<int4*>(p + i * 8) = x;
  }
}

// The same update for the groups of a [G, n] tensor whose mask word is zero (`want` = 0) or non-zero (1):
// used for the experts that the weight-gradient GEMM did not already update in its epilogue.
__global__ void __launch_bounds__(256) sgd_groups_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ g, float lr,
                                                         int64_t n8, const int32_t* __restrict__ mask, int want) {
  const int grp = blockIdx.y;
  if ((mask[grp] != 0) != (want != 0)) return;
  p += (int64_t)grp * n8 * 8; g += (int64_t)grp * n8 * 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    int4 x = *reinterpret_cast<const int4*>(p + i * 8);
    const float4 g0 = *reinterpret_cast<const float4*>(g + i * 8), g1 = *reinterpret_cast<const float4*>(g + i * 8 + 4);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      f.x = fmaf(-lr, gg[2 * k], f.x); f.y = fmaf(-lr, gg[2 * k + 1], f.y);      // the form wgrad's fused update uses
      h[k] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<int4*>(p + i * 8) = x;
  }
}

}  // namespace mep

extern "C" int mep_swiglu_bwd(const void* dA, const void* gu, const float* w, void* dgu, float* dw,
                              const int32_t* cu_seqlens, int G, int Hp, int num_blocks, cudaStream_t stream) {
  MEP_REQUIRE(Hp % 8 == 0, "swiglu_bwd: inner size %d must be a multiple of 8", Hp);
  return mep::launch_plain(mep::swiglu_bwd_kernel, dim3(num_blocks), dim3(256), 0, stream,
                           (const __nv_bfloat16*)dA, (const __nv_bfloat16*)gu, w, (__nv_bfloat16*)dgu, dw, cu_seqlens, G, Hp);
}

extern "C" int mep_sgd_step(void* p, const float* g, float lr, int64_t n, int num_blocks, cudaStream_t stream) {
  MEP_REQUIRE(n % 8 == 0, "sgd_step: element count must be a multiple of 8");
  return mep::launch_plain(mep::sgd_kernel, dim3(num_blocks), dim3(256), 0, stream, (__nv_bfloat16*)p, g, lr, n / 8);
}

extern "C" int mep_sgd_step_groups(void* p, const float* g, float lr, int64_t n_per_group, int G, const int32_t* mask, int want,
                                   int num_blocks, cudaStream_t stream) {
  MEP_REQUIRE(n_per_group % 8 == 0 && G >= 1 && G <= 65535, "sgd_step_groups: %d groups of %lld elements", G, (long long)n_per_group);
  return mep::launch_plain(mep::sgd_groups_kernel, dim3(num_blocks, G), dim3(256), 0, stream, (__nv_bfloat16*)p, g, lr,
                           n_per_group / 8, mask, want);
}
