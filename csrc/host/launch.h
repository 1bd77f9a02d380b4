// Host-side helpers shared by all launchers: error reporting through a thread-local
// message (no exit(), unlike the reference's CUCHECK/CUDACHECK macros,
// csrc/nvl_shared_buffer.cuh:17-39) and a cooperative-launch wrapper.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <atomic>
#include <string>
#include "../mep_types.h"

// Exports sizeof(type) as mep_sizeof_<name>() so that the Python side can check its ctypes
// mirror of an argument struct against the compiled layout.
#define MEP_EXPORT_SIZEOF(name, type) extern "C" int mep_sizeof_##name() { return (int)sizeof(type); }

namespace mep {

std::string& last_error();
extern std::atomic<long long> g_launches;
int set_error(const char* fmt, ...);

#define MEP_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return ::mep::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                              __FILE__, __LINE__);                                        \
  } while (0)

#define MEP_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return ::mep::set_error(__VA_ARGS__);          \
  } while (0)

// Launch `kernel` with CTAs guaranteed co-resident (needed by the software barriers).
template <class... KArgs, class... Args>
int launch_cooperative(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeCooperative; attr[n].val.cooperative = 1; ++n;
  if (pdl) { attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
             attr[n].val.programmaticStreamSerializationAllowed = 1; ++n; }
  cfg.attrs = attr; cfg.numAttrs = n;
  if (smem > 16 * 1024)
    MEP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MEP_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

template <class... KArgs, class... Args>
int launch_plain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                 cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cfg.attrs = nullptr; cfg.numAttrs = 0;
  if (smem > 16 * 1024)
    MEP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MEP_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

// launch_plain with an optional programmatic dependency on the previous kernel of the stream:
// the grid may be scheduled while that kernel drains; the kernel itself must execute
// griddepcontrol.wait (pdl_wait) before it touches anything its predecessor wrote.
template <class... KArgs, class... Args>
int launch_plain_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                     cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = pdl ? attr : nullptr; cfg.numAttrs = pdl ? 1 : 0;
  if (smem > 16 * 1024)
    MEP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MEP_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

}  // namespace mep
