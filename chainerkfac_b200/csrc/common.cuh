// Shared host/device helpers of the kfac_b200 library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/kfac_b200.h"

namespace kfac {

// Thread-local message behind kfac_last_error().
char* error_buffer();

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define KFAC_CUDA(expr)                                                     \
  do {                                                                      \
    cudaError_t e__ = (expr);                                               \
    if (e__ != cudaSuccess)                                                 \
      return ::kfac::fail(KFAC_ERR_CUDA, "%s: %s (%s:%d)", #expr,           \
                          cudaGetErrorString(e__), __FILE__, __LINE__);     \
  } while (0)

#define KFAC_LAUNCH_CHECK(name)                                             \
  do {                                                                      \
    ::kfac::count_launch();                                                 \
    cudaError_t e__ = cudaGetLastError();                                   \
    if (e__ != cudaSuccess)                                                 \
      return ::kfac::fail(KFAC_ERR_CUDA, "launch of %s failed: %s", name,   \
                          cudaGetErrorString(e__));                         \
  } while (0)

#define KFAC_REQUIRE(cond, ...)                                             \
  do {                                                                      \
    if (!(cond)) return ::kfac::fail(KFAC_ERR_INVALID, __VA_ARGS__);        \
  } while (0)

inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Counter behind kfac_launch_count().
void count_launch();
// Add n (replayed graph nodes; negative: launches that were only captured).
void count_launches(long long n);
long long launch_count_now();

// Slice of a small per-device ring of device memory for descriptor tables
// built per call (see pack.cu).
int ring_alloc(size_t bytes, void** out);

// Status word of the inverse's diagonal kernel (inverse.cu).
int diag_status_read(int* out);

// Number of streaming multiprocessors of the current device (cached).
int sm_count();

}  // namespace kfac
