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

enum KernelId : int {
  KID_APPEND = 1,
  KID_SLOT_MAPPING = 2,
  KID_METADATA = 3,
  KID_COPY_PAGES = 4,
  KID_ATTN_PLAN = 5,
  KID_ATTN = 6,
  KID_ATTN_MERGE = 7,
};

}  // namespace kb200
