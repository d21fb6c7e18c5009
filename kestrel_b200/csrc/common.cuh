// Shared definitions for the paged-KV kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>
#include <mutex>

#include "../../include/kestrel_b200.h"

namespace kb200 {

// ---------------------------------------------------------------------------
// Host-side error reporting: every entry point returns 0 or a negative code
// and leaves a message in a thread-local buffer.  Nothing throws or aborts.
// ---------------------------------------------------------------------------
inline char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define KB200_CUDA_OK(expr)                                                       \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess)                                                        \
      return ::kb200::fail(KB200_ERR_CUDA, "%s failed: %s", #expr,               \
                           cudaGetErrorString(_e));                               \
  } while (0)

#define KB200_REQUIRE(cond, ...)                                                  \
  do {                                                                            \
    if (!(cond)) return ::kb200::fail(KB200_ERR_INVALID, __VA_ARGS__);            \
  } while (0)

inline int dtype_size(int dt) {
  switch (dt) {
    case KB200_DTYPE_F32: return 4;
    case KB200_DTYPE_F16: return 2;
    case KB200_DTYPE_BF16: return 2;
    case KB200_DTYPE_E4M3: return 1;
    default: return 0;
  }
}

// RAII device switch: every entry point runs on the device its arguments live on.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    cur = dev;
  }
  ~DeviceGuard() {
    if (prev >= 0 && prev != cur) cudaSetDevice(prev);
  }
  int cur = -1;
};

// ---------------------------------------------------------------------------
// Device-side diagnostics.  Kernels never trap: a bad index or a wait that ran
// out is recorded here (one copy per GPU) and the offending access is skipped.
// word 0: OR of KB200_STATUS_* bits, word 1: first offending value,
// word 2: id of the kernel that reported, word 3: count of reports.
// ---------------------------------------------------------------------------
__device__ int g_status[4];

__device__ __forceinline__ void report(int bit, int value, int kernel_id) {
  int old = atomicOr(&g_status[0], bit);
  if ((old & bit) == 0) {
    g_status[1] = value;
    g_status[2] = kernel_id;
  }
  atomicAdd(&g_status[3], 1);
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the hot path is launched with the
// programmatic-stream-serialization attribute and calls pdl_wait() before it touches global
// memory, so its launch latency and shared-memory prologue overlap the tail of the kernel
// before it; results are unchanged because nothing is read or written before the wait.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device), safe under concurrent
// first calls from several threads.
struct SmemAttrOnce {
  std::once_flag flags[64];
  cudaError_t results[64] = {};
  template <typename K>
  int ensure(K kernel, int smem_bytes, int dev) {
    const int i = dev & 63;
    std::call_once(flags[i], [&] {
      results[i] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    });
    if (results[i] != cudaSuccess)
      return fail(KB200_ERR_CUDA, "cudaFuncSetAttribute(max dynamic shared memory) failed: %s",
                  cudaGetErrorString(results[i]));
    return KB200_OK;
  }
};

enum KernelId : int {
  KID_APPEND = 1,
  KID_SLOT_MAPPING = 2,
  KID_METADATA = 3,
  KID_COPY_PAGES = 4,
  KID_ATTN_PLAN = 5,
  KID_ATTN = 6,
  KID_ATTN_MERGE = 7,
  KID_ROPE_APPEND = 8,
  KID_PREFILL = 9,
  KID_SAMPLE = 10,
};

}  // namespace kb200
