// Shared-memory pipeline helpers: mbarrier, global -> shared bulk copies, and
// bounded waits.  Every wait gives up after kWaitCycles: it raises the CTA's
// abort flag, ORs FP_DECODE_WAIT_TIMEOUT (bit 0 of every status word in this
// library) into the caller's status word and returns false, so no kernel built
// on these can hang.
#pragma once

#include <stdint.h>

#include "../../include/fragpack_b200.h"
#include "fp_common.cuh"

namespace fpb {

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
// One try: the hardware may suspend the thread for up to `hint_ns` while the
// phase is incomplete, so a waiting warp does not burn issue slots polling.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}
// Global -> shared bulk copy (no multicast) completing on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Blocks the calling thread until the grids this launch depends on have
// completed and their writes are visible (returns at once otherwise).
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

constexpr long long kWaitCycles = 4000000000LL;  // about two seconds

// What a bounded wait needs besides the barrier, kept in the CTA's shared
// memory so that the fast path of a wait carries no extra registers: the abort
// flag, the status word to report into and the cycle budget (kWaitCycles in
// production; tests shorten it to make a wait run out on purpose).
struct WaitState {
  int abort;
  int32_t* status;
  long long limit;
};

// Waits for `parity` of `bar` to complete, at most ws->limit cycles.  Returns
// false (and raises the CTA's abort flag) when the wait ran out or the CTA had
// already given up.
static __device__ __noinline__ bool wait_slow(uint64_t* bar, uint32_t parity, WaitState* ws) {
  volatile int* abort = &ws->abort;
  const long long t0 = clock64();
  for (;;) {
    if (*abort) return false;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
      if (mbar_try(bar, parity, 20000u)) return true;
    if (clock64() - t0 > ws->limit) {
      *abort = 1;
      atomicOr(ws->status, FP_DECODE_WAIT_TIMEOUT);
      return false;
    }
  }
}
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, WaitState* ws) {
  if (mbar_try(bar, parity, 2000u)) return true;
  return wait_slow(bar, parity, ws);
}

// Test hook (host side): cycle budget of the bounded waits and the ordinal of
// one record per CTA that the producer warp leaves out, so that a consumer wait
// runs out.  Defaults: kWaitCycles, -1 (none).  Set by fp_debug_wait_limit.
struct WaitDebug {
  long long limit;
  long long skip_record;
};
WaitDebug wait_debug();

}  // namespace fpb
