// Error reporting shared by the C-ABI entry points: every entry point returns
// 0 on success or a negative code, and fp_last_error() returns the message of
// the calling thread's last failure.
#pragma once

#include <cuda_runtime.h>

#include "../../include/fragpack_b200.h"

namespace fpb {

int fail(int code, const char* fmt, ...);

// Returns FP_ERR_CUDA with the CUDA error text if `err` is not cudaSuccess.
int cuda_status(cudaError_t err, const char* what);

}  // namespace fpb

#define FP_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return fpb::fail(FP_ERR_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define FP_LAUNCH_CHECK(what)                                        \
  do {                                                               \
    const int rc_ = fpb::cuda_status(cudaGetLastError(), what);      \
    if (rc_) return rc_;                                             \
  } while (0)
