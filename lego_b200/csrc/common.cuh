// Shared helpers of the CUDA translation units.
#pragma once

#include <atomic>
#include <utility>

#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/lego_b200.h"
#include "layout_host.h"

namespace lego {

inline int32_t cuda_status(cudaError_t e) {
  return e == cudaSuccess ? LEGO_OK : (int32_t)LEGO_ERR_CUDA_BASE + (int32_t)e;
}

#define LEGO_CUDA_TRY(expr)                                    \
  do {                                                         \
    cudaError_t _e = (expr);                                   \
    if (_e != cudaSuccess) {                                   \
      (void)cudaGetLastError(); /* do not leak into later calls */ \
      return ::lego::cuda_status(_e);                          \
    }                                                          \
  } while (0)

// Launch with programmatic stream serialization: the grid may become resident, and run
// everything before its ptx::grid_dependency_wait(), while the previous grid in the
// stream (if it called ptx::launch_dependents()) is still draining.  Kernels launched this
// way touch global memory only after that wait.  Also valid under stream capture.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
#ifdef LEGO_NO_PDL
  cfg.numAttrs = 0;
#else
  cfg.numAttrs = 1;
#endif
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Which devices a kernel has been set up on.  cudaFuncSetAttribute (the opt-in to more
// than 48 KiB of dynamic shared memory) and occupancy answers hold for the device that was
// current when they were made, so every launcher keeps one of these per kernel instead of a
// process-wide flag.  Two host threads that race both do the (idempotent) set-up.
struct PerDeviceFlag {
  std::atomic<uint64_t> mask{0};
  bool test(int dev) const {
    return dev >= 0 && dev < 64 && ((mask.load(std::memory_order_acquire) >> dev) & 1u) != 0;
  }
  void set(int dev) {
    if (dev >= 0 && dev < 64) mask.fetch_or(1ull << dev, std::memory_order_release);
  }
};

// Per-device facts and the lazily created workspace.
struct DeviceCtx {
  int device;
  int sm_count;
  int smem_optin;
  uint32_t* status_word;   // device: first failing wait of a kernel, 0 = none
  void* tmap_table;        // device: tensor maps of grouped GEMM calls
  size_t tmap_table_bytes;
};
// Context of the current device (created on first use); nullptr + *err on failure.
DeviceCtx* device_ctx(int32_t* err);
// Context of the current device if one exists; never creates (or allocates) anything.
DeviceCtx* device_ctx_if_any();
void release_all_ctx();

__device__ __forceinline__ uint32_t fd_div(uint32_t n, const FastDiv& f) {
  return f.mul ? (__umulhi(n, f.mul) >> f.shr) : (n >> f.shr);
}

}  // namespace lego
