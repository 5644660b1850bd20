// Host-side conventions of the C-ABI library: status codes, the thread-local error text, launch checks.
#pragma once

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/mek_gdn.h"

namespace mek {

// The text mek_last_error() returns on this thread.
char* error_buffer();

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// After a launch: report a launch-configuration error (no synchronisation; asynchronous faults surface later).
inline int launched(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MEK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return MEK_OK;
}

// Opt a kernel into more than 48 KiB of dynamic shared memory (once per device would do; the call is cheap).
template <typename Kernel>
inline int want_smem(Kernel kernel, size_t bytes, const char* what) {
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  if (err != cudaSuccess) return fail(MEK_ERR_CUDA, "%s: shared memory %zu B: %s", what, bytes, cudaGetErrorString(err));
  return MEK_OK;
}

// Device-side error word of a kernel that has bounded waits: 0 = fine; otherwise the code below in the low byte and
// where it happened (a stage number) above it.  The host reads it after the stream has been synchronised.
enum : int { kDevWaitTimeout = 1, kDevBadArgument = 2 };

}  // namespace mek
