// Device view of the store state (fp_store) shared by the lifecycle, writer,
// encoder and blob kernels: staging address arithmetic and the overflow pool.
#pragma once

#include <stdint.h>

#include "../../include/fragpack_b200.h"
#include "fp_common.cuh"

namespace fpb {

struct StoreView {
  fp_store s;

  // Staging record `rec` (= kv * H + head) of staging slot `slot` at `layer`.
  // Slots below S_p are persistent and hold one record set per layer; the
  // others are transient scratch holding a single layer, reused layer by layer
  // (a block that opens and closes within a step is encoded per layer).
  __device__ __forceinline__ uint8_t* staging(int slot, int layer, int rec) const {
    const int per = 2 * s.H;
    if (slot < s.S_p) return s.staging + (((int64_t)slot * s.L + layer) * per + rec) * kRawRecord;
    return s.scratch + ((int64_t)(slot - s.S_p) * per + rec) * kRawRecord;
  }
  __device__ __forceinline__ int64_t table_index(int layer, int block, int rec) const {
    return ((int64_t)layer * s.NB + block) * 2 * s.H + rec;
  }

  // ---- Overflow pool: 32 KB slots for records that do not code or do not fit
  // their page.  A bitmap (bit set = in use; the bits past the pool are preset)
  // says which slots are taken, so that the encoder and an import running on
  // another stream can take and return slots concurrently, and the counter
  // FP_CTR_OVF_FREE says how many are left, so that a full pool is refused
  // with one atomic instead of a walk over the whole bitmap.  Invariant: the
  // counter never exceeds the number of clear bits (a slot's bit is cleared
  // before the counter is raised, and the counter is lowered before a bit is
  // set), so whoever holds a reservation finds a clear bit.

  // Reserves one slot; false when the pool is full.
  __device__ __forceinline__ bool overflow_reserve() const {
    int32_t* left = &s.counters[FP_CTR_OVF_FREE];
    if (atomicSub(left, 1) > 0) return true;
    atomicAdd(left, 1);
    return false;
  }

  // Tries to set a clear bit of bitmap word `w`; returns the slot or -1.
  __device__ __forceinline__ int overflow_claim_in(int w) const {
    uint32_t seen = *reinterpret_cast<volatile uint32_t*>(&s.ovf_bits[w]);
    while (seen != 0xffffffffu) {
      const uint32_t bit = (~seen) & (seen + 1u);  // lowest clear bit
      const uint32_t before = atomicOr(&s.ovf_bits[w], bit);
      if (!(before & bit)) return 32 * w + (__ffs(bit) - 1);
      seen = before | bit;
    }
    return -1;
  }

  // Takes a slot for the calling WARP (all 32 lanes call; every lane gets the
  // result).  The lanes look at 32 consecutive bitmap words at a time, starting
  // at a word derived from `hint` so that concurrent callers spread out.
  // Returns -1 when the pool is full.
  __device__ int overflow_take_warp(uint32_t hint) const {
    const int lane = threadIdx.x & 31;
    int reserved = 0;
    if (lane == 0) reserved = overflow_reserve();
    if (!__shfl_sync(0xffffffffu, reserved, 0)) return -1;
    const uint32_t words = (uint32_t)s.ovf_words;
    const uint32_t start = (hint * 0x9e3779b1u) % words;
    // Two sweeps bound the loop: a slot freed behind the sweep is met again.
    for (uint32_t done = 0; done < 2 * words + 32; done += 32) {
      const uint32_t w = (start + done + (uint32_t)lane) % words;
      const bool in_sweep = done + (uint32_t)lane < 2 * words;
      const uint32_t bits = in_sweep ? *reinterpret_cast<volatile uint32_t*>(&s.ovf_bits[w])
                                     : 0xffffffffu;
      uint32_t open = __ballot_sync(0xffffffffu, bits != 0xffffffffu);
      while (open) {
        const int src = __ffs(open) - 1;
        int slot = -1;
        if (lane == src) slot = overflow_claim_in((int)w);
        slot = __shfl_sync(0xffffffffu, slot, src);
        if (slot >= 0) return slot;
        open &= open - 1;
      }
    }
    if (lane == 0) atomicAdd(&s.counters[FP_CTR_OVF_FREE], 1);  // give the reservation back
    return -1;
  }

  // The same for a single calling thread (the blob importer places records one
  // after another in one thread).
  __device__ int overflow_take(uint32_t hint) const {
    if (!overflow_reserve()) return -1;
    const uint32_t words = (uint32_t)s.ovf_words;
    const uint32_t start = (hint * 0x9e3779b1u) % words;
    for (uint32_t done = 0; done < 2 * words; ++done) {
      const int slot = overflow_claim_in((int)((start + done) % words));
      if (slot >= 0) return slot;
    }
    atomicAdd(&s.counters[FP_CTR_OVF_FREE], 1);
    return -1;
  }

  __device__ __forceinline__ bool in_overflow(int64_t addr) const {
    const int64_t base = reinterpret_cast<int64_t>(s.overflow);
    return addr >= base && addr < base + s.overflow_records * kRawRecord;
  }

  // Returns the overflow slot at `addr` to the pool; other addresses are ignored.
  __device__ __forceinline__ void overflow_give_back(int64_t addr) const {
    if (!in_overflow(addr)) return;
    const int slot = (int)((addr - reinterpret_cast<int64_t>(s.overflow)) / kRawRecord);
    const uint32_t bit = 1u << (slot & 31);
    if (atomicAnd(&s.ovf_bits[slot >> 5], ~bit) & bit) atomicAdd(&s.counters[FP_CTR_OVF_FREE], 1);
  }
};

}  // namespace fpb
