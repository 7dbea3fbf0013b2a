// Error reporting shared by the C-ABI entry points: every entry point returns
// 0 on success or a negative code, and fp_last_error() returns the message of
// the calling thread's last failure.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "../../include/fragpack_b200.h"

namespace fpb {

int fail(int code, const char* fmt, ...);

// Returns FP_ERR_CUDA with the CUDA error text if `err` is not cudaSuccess.
int cuda_status(cudaError_t err, const char* what);

// Raises `kernel`'s dynamic shared memory limit to `bytes` on the current
// device.  The attribute is per device, so `done` (one per kernel) remembers
// the devices already served (bit = device index; devices past 63 are set on
// every call).  A failure is reported and not remembered.
template <typename Kernel>
int allow_dynamic_smem(Kernel kernel, int bytes, std::atomic<uint64_t>& done) {
  int dev = 0;
  if (int rc = cuda_status(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  const uint64_t bit = dev >= 0 && dev < 64 ? 1ull << dev : 0ull;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return FP_OK;
  if (int rc = cuda_status(
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
          "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)"))
    return rc;
  if (bit) done.fetch_or(bit, std::memory_order_release);
  return FP_OK;
}

// Streaming multiprocessors of the current device (148 if the query fails).
int device_sms();

// Rejects a store whose tables are missing or whose geometry is impossible.
int check_store(const fp_store* store);

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
