// Host-side helpers shared by the translation units of libqlin_b200.so.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../include/qlin_b200.h"

namespace qlin {

// Records the message returned by qlin_last_error_string() for the calling thread and
// returns `code`, so call sites can write `return fail(QLIN_ERR_..., "...")`.
int fail(int code, const char* fmt, ...);

// Number of SMs of the current device (cached per device id).
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dt) {
  switch (dt) {
    case QLIN_DT_I8:
    case QLIN_DT_U8:
    case QLIN_DT_F8E4M3:
      return 1;
    case QLIN_DT_F16:
    case QLIN_DT_BF16:
      return 2;
    case QLIN_DT_I32:
    case QLIN_DT_F32:
      return 4;
    default:
      return 0;
  }
}

#define QLIN_CHECK_LAUNCH(what)                                                      \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess)                                                          \
      return ::qlin::fail(QLIN_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e__)); \
  } while (0)

}  // namespace qlin
