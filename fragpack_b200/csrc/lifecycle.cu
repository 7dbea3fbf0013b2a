// Step lifecycle of the HBM KV store for sm_100a: prepare (before the first
// layer of a step) and commit (after the last).  They decide where the blocks
// that receive tokens this step are staged; the token writer, the encoder and
// attention then only follow wslot / rec_addr.
//
// The contract is the reference's (fragpack/ops/hbm_kv.cu:110-219, 431-448,
// fragpack/ops/hbm_kv.py:16-38): a block is open from the step that writes its
// offset 0 until the step that writes its offset 127; an open block owns a
// staging slot; blocks that open and close within one step use transient
// scratch; a block that stays open needs a persistent slot and, when none is
// free but a block closing this step holds one, waits in scratch as that
// block's heir and moves into its slot when it has been encoded.
//
// How it is done here differs from the reference's single 1024-thread CTA:
//  * prepare_scan_kernel (a full grid over the step's tokens and the live
//    list) stamps the live and the closing blocks and collects the blocks seen
//    opening or closing, each once, with one atomic per warp;
//  * prepare_assign_kernel (one CTA; its work grows with the staging slots and
//    the opening / closing blocks, not with the tokens or the number of blocks
//    of the cache) releases the slots of blocks that are no longer live by
//    walking the slots' owners, then hands out slots by exclusive rank among
//    the waiting blocks (block-wide scans), so the assignment is a function of
//    the collected lists and not of which thread wins an atomic;
//  * prepare_repoint_kernel (a full grid over claimed blocks x layers x records)
//    points the claimed blocks' table entries at their staging, returns the
//    overflow slots they held and empties their pages.
#include "fp_api.h"
#include "fp_store.cuh"

namespace fpb {
namespace {

enum : int { kTagLive = 0, kTagClosing = 1, kTagOpening = 2 };
constexpr int kScanThreads = 256;
constexpr int kAssignThreads = 1024;

// Appends `value` of every lane with `wanted` set to list[0 .. *count), one
// atomic per warp; entries beyond `cap` are dropped.
__device__ __forceinline__ void warp_append(bool wanted, int value, int32_t* list, int32_t* count,
                                            int cap) {
  const uint32_t mask = __ballot_sync(0xffffffffu, wanted);
  if (mask == 0) return;
  const int lane = threadIdx.x & 31, leader = __ffs(mask) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(count, __popc(mask));
  base = __shfl_sync(0xffffffffu, base, leader);
  const int at = base + __popc(mask & ((1u << lane) - 1u));
  if (wanted && at < cap) list[at] = value;
}

__global__ void __launch_bounds__(kScanThreads)
prepare_scan_kernel(StoreView v, const int64_t* slots, int n_tok, const int32_t* live, int n_live,
                    int32_t step) {
  const fp_store& s = v.s;
  const int i = blockIdx.x * kScanThreads + threadIdx.x;
  if (i < n_live) {
    const int b = live[i];
    if (b >= 0 && b < s.NB) s.tags[kTagLive * s.NB + b] = step;
  }
  bool opens = false, closes = false;
  int block = 0;
  if (i < n_tok) {
    const int64_t slot = slots[i];
    if (slot >= 0 && (slot >> 7) < s.NB) {
      block = (int)(slot >> 7);
      const int off = (int)(slot & 127);
      // The exchange lets exactly one token of a block through per step, also
      // for a slot mapping that names an offset twice.
      if (off == 0) opens = atomicExch(&s.tags[kTagOpening * s.NB + block], step) != step;
      if (off == 127) closes = atomicExch(&s.tags[kTagClosing * s.NB + block], step) != step;
    }
  }
  warp_append(opens, block, s.seen_list, &s.counters[FP_CTR_SEEN_OPEN], s.cap);
  warp_append(closes, block, s.seen_list + s.cap, &s.counters[FP_CTR_SEEN_CLOSE], s.cap);
}

// Exclusive prefix sums of a and b over the CTA (kAssignThreads threads);
// total_a / total_b receive the sums.
__device__ __forceinline__ void block_scan2(int& a, int& b, int& total_a, int& total_b,
                                            int (*warp_sums)[2]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int ia = a, ib = b;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int ta = __shfl_up_sync(0xffffffffu, ia, d), tb = __shfl_up_sync(0xffffffffu, ib, d);
    if (lane >= d) {
      ia += ta;
      ib += tb;
    }
  }
  __syncthreads();  // the previous use of warp_sums is over
  if (lane == 31) {
    warp_sums[warp][0] = ia;
    warp_sums[warp][1] = ib;
  }
  __syncthreads();
  int before_a = 0, before_b = 0;
  total_a = total_b = 0;
#pragma unroll 4
  for (int w = 0; w < kAssignThreads / 32; ++w) {
    const int wa = warp_sums[w][0], wb = warp_sums[w][1];
    if (w < warp) {
      before_a += wa;
      before_b += wb;
    }
    total_a += wa;
    total_b += wb;
  }
  a = before_a + ia - a;
  b = before_b + ib - b;
}

__global__ void __launch_bounds__(kAssignThreads)
prepare_assign_kernel(StoreView v, int32_t step) {
  const fp_store& s = v.s;
  __shared__ int warp_sums[kAssignThreads / 32][2];
  const int tid = threadIdx.x;
  const int32_t* tag_live = s.tags + kTagLive * s.NB;
  const int32_t* tag_closing = s.tags + kTagClosing * s.NB;
  const int n_open = min(s.counters[FP_CTR_SEEN_OPEN], s.cap);
  const int n_close = min(s.counters[FP_CTR_SEEN_CLOSE], s.cap);
  int free_top = s.counters[FP_CTR_FREE_TOP];
  const int last_transient = min(s.counters[FP_CTR_TRANSIENT], s.S_t);
  __syncthreads();  // everyone has read the counters that thread 0 rewrites at the end

  // ---- 1. Slots come back.  Scratch never outlives its step; a persistent
  // slot comes back when its owner is not listed live any more.
  for (int t = tid; t < last_transient; t += kAssignThreads) {
    const int b = s.slot_owner[s.S_p + t];
    if (b >= 0 && s.wslot[b] == s.S_p + t) s.wslot[b] = -1;
    s.slot_owner[s.S_p + t] = -1;
  }
  for (int base = 0; base < s.S_p; base += kAssignThreads) {
    const int slot = base + tid;
    int freed = 0, unused = 0, total, unused_total;
    int owner = -1;
    if (slot < s.S_p) {
      owner = s.slot_owner[slot];
      freed = owner >= 0 && tag_live[owner] != step;
    }
    block_scan2(freed, unused, total, unused_total, warp_sums);
    if (owner >= 0 && tag_live[owner] != step) {
      s.wslot[owner] = -1;
      s.slot_owner[slot] = -1;
      s.free_stack[free_top + freed] = slot;
    }
    free_top += total;
  }
  __syncthreads();

  // ---- 2. Opening blocks.  A block that kept a slot keeps it.  Of the others,
  // those that also close this step take scratch; those that stay open take
  // the free persistent slots in list order, and the rest become heirs in
  // scratch.  First pass: how many of each; second pass: hand out by rank.
  int short_lived = 0, lasting = 0;
  for (int i = tid; i < n_open; i += kAssignThreads) {
    const int b = s.seen_list[i];
    if (s.wslot[b] >= 0) continue;
    if (tag_closing[b] == step) ++short_lived; else ++lasting;
  }
  {
    int ta, tb;
    block_scan2(short_lived, lasting, ta, tb, warp_sums);
    short_lived = ta;  // totals
    lasting = tb;
  }
  const int granted = min(lasting, free_top);    // lasting blocks that get a persistent slot
  const int heirs_wanted = lasting - granted;
  const int heirs = max(0, min(heirs_wanted, s.S_t - min(short_lived, s.S_t)));
  int claims = 0, seen_short = 0, seen_lasting = 0;
  for (int base = 0; base < n_open; base += kAssignThreads) {
    const int i = base + tid;
    int b = -1, kind = 0;  // 1: keeps its slot, 2: short-lived, 3: lasting
    if (i < n_open) {
      b = s.seen_list[i];
      kind = s.wslot[b] >= 0 ? 1 : (tag_closing[b] == step ? 2 : 3);
    }
    int rank_short = kind == 2, rank_lasting = kind == 3, tile_short, tile_lasting;
    block_scan2(rank_short, rank_lasting, tile_short, tile_lasting, warp_sums);
    int slot = -1, heir_index = -1;
    if (kind == 1) {
      slot = s.wslot[b];
    } else if (kind == 2) {
      const int t = seen_short + rank_short;
      if (t < s.S_t) slot = s.S_p + t;
    } else if (kind == 3) {
      const int r = seen_lasting + rank_lasting;
      if (r < granted) {
        slot = s.free_stack[free_top - 1 - r];
      } else if (r - granted < heirs) {
        heir_index = r - granted;
        slot = s.S_p + min(short_lived, s.S_t) + heir_index;
      }
    }
    int placed = slot >= 0, unused = 0, tile_placed, unused_total;
    block_scan2(placed, unused, tile_placed, unused_total, warp_sums);
    if (kind != 0) {
      s.wslot[b] = slot;
      if (slot >= 0) {
        s.slot_owner[slot] = b;
        s.claim_list[claims + placed] = b;
        if (heir_index >= 0) s.claim_list[s.cap + heir_index] = b;
      }
    }
    claims += tile_placed;
    seen_short += tile_short;
    seen_lasting += tile_lasting;
  }
  const int dropped = (short_lived - min(short_lived, s.S_t)) + (heirs_wanted - heirs);
  __syncthreads();

  // ---- 3. Closing blocks that own a slot are listed for the encoder; those
  // holding a persistent slot donate it, in list order, to the waiting heirs.
  int closes = 0, donors = 0;
  for (int base = 0; base < n_close; base += kAssignThreads) {
    const int i = base + tid;
    int b = -1, w = -1;
    if (i < n_close) {
      b = s.seen_list[s.cap + i];
      w = s.wslot[b];
    }
    int listed = w >= 0, donates = w >= 0 && w < s.S_p, tile_listed, tile_donors;
    block_scan2(listed, donates, tile_listed, tile_donors, warp_sums);
    if (w >= 0) {
      const int at = closes + listed;
      const int d = donors + donates;
      s.close_list[at] = b;
      s.close_list[s.cap + at] = (w < s.S_p && d < heirs) ? s.claim_list[s.cap + d] : -1;
    }
    closes += tile_listed;
    donors += tile_donors;
  }
  if (tid == 0) {
    s.counters[FP_CTR_FREE_TOP] = free_top - granted;
    s.counters[FP_CTR_TRANSIENT] = min(short_lived, s.S_t) + heirs;
    s.counters[FP_CTR_CLAIMS] = claims;
    s.counters[FP_CTR_CLOSES] = closes;
    s.counters[FP_CTR_HEIRS] = heirs;
    s.counters[FP_CTR_DONORS] = min(donors, heirs);
    // Blocks left without staging lose their tokens; an heir left without a
    // donor would lose its KV at commit.
    const int lost = dropped + max(0, heirs - donors);
    if (lost > 0) atomicAdd(&s.counters[FP_CTR_ERR_STAGING], lost);
    s.counters[FP_CTR_SEEN_OPEN] = 0;
    s.counters[FP_CTR_SEEN_CLOSE] = 0;
  }
}

// Every record of a claimed block points at its staging, the overflow slot it
// held is returned and the block's pages are emptied.
__global__ void __launch_bounds__(256) prepare_repoint_kernel(StoreView v) {
  const fp_store& s = v.s;
  const int per_block = s.L * 2 * s.H;
  const int64_t total = (int64_t)s.counters[FP_CTR_CLAIMS] * per_block;
  for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < total;
       x += (int64_t)gridDim.x * blockDim.x) {
    const int b = s.claim_list[x / per_block];
    const int within = (int)(x % per_block), layer = within / (2 * s.H), rec = within % (2 * s.H);
    const int64_t idx = v.table_index(layer, b, rec);
    v.overflow_give_back(s.rec_addr[idx]);
    s.rec_addr[idx] = reinterpret_cast<int64_t>(v.staging(s.wslot[b], layer, rec));
    s.rec_len[idx] = kRawVarLen;
    if (rec == 0) s.fill[(int64_t)layer * s.NB + b] = 0;
  }
}

// commit: every closed block lets go of its slot; a persistent slot goes to
// the block's heir (whose record the encoder has already moved in) or back to
// the free stack.
__global__ void __launch_bounds__(256) commit_kernel(StoreView v) {
  const fp_store& s = v.s;
  const int closes = s.counters[FP_CTR_CLOSES];
  for (int base = 0; base < closes; base += blockDim.x) {
    const int i = base + threadIdx.x;
    bool frees = false;
    int slot = -1;
    if (i < closes) {
      const int b = s.close_list[i], heir = s.close_list[s.cap + i];
      slot = s.wslot[b];
      s.wslot[b] = -1;
      if (heir >= 0) {
        s.wslot[heir] = slot;
        s.slot_owner[slot] = heir;
      } else if (slot >= 0 && slot < s.S_p) {
        s.slot_owner[slot] = -1;
        frees = true;
      }
    }
    warp_append(frees, slot, s.free_stack, &s.counters[FP_CTR_FREE_TOP], s.S_p);
  }
  __syncthreads();
  // An emptied close list makes a forward without a fresh prepare encode nothing.
  if (threadIdx.x == 0) s.counters[FP_CTR_CLOSES] = 0;
}

}  // namespace

int check_store(const fp_store* st) {
  FP_REQUIRE(st != nullptr, "store is null");
  FP_REQUIRE(st->counters && st->wslot && st->tags && st->free_stack && st->ovf_bits &&
                 st->claim_list && st->close_list && st->rec_addr && st->rec_len && st->fill &&
                 st->slot_owner && st->seen_list,
             "store has a null table");
  FP_REQUIRE(st->L > 0 && st->H > 0 && st->NB > 0 && st->cap >= 0 && st->S_p >= 0 && st->S_t >= 0 &&
                 st->ovf_words > 0,
             "bad store geometry");
  return FP_OK;
}

}  // namespace fpb

using namespace fpb;

extern "C" {

int fp_hbm_prepare(const fp_store* store, const int64_t* slot_mapping, int64_t num_tokens,
                   const int32_t* live, int64_t num_live, int32_t step, void* stream) {
  if (int rc = check_store(store)) return rc;
  FP_REQUIRE(num_tokens >= 0 && num_tokens <= store->cap, "block lists too small for %lld tokens",
             (long long)num_tokens);
  FP_REQUIRE(num_tokens == 0 || slot_mapping, "slot_mapping is null");
  FP_REQUIRE(num_live >= 0 && num_live < (1LL << 31) && (num_live == 0 || live),
             "live list is null");
  StoreView v{*store};
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t most = num_tokens > num_live ? num_tokens : num_live;
  if (most > 0) {
    prepare_scan_kernel<<<(unsigned)((most + kScanThreads - 1) / kScanThreads), kScanThreads, 0,
                          st>>>(v, slot_mapping, (int)num_tokens, live, (int)num_live, step);
    FP_LAUNCH_CHECK("prepare_scan_kernel");
  }
  prepare_assign_kernel<<<1, kAssignThreads, 0, st>>>(v, step);
  FP_LAUNCH_CHECK("prepare_assign_kernel");
  if (num_tokens > 0) {
    // At most one block opens per 128 tokens, plus one per request; the grid
    // strides over what the assign kernel actually claimed.
    const int64_t entries = (num_tokens / 128 + 64) * store->L * 2 * store->H;
    const int64_t want = (entries + 255) / 256, cap = 8LL * device_sms();
    prepare_repoint_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(v);
    FP_LAUNCH_CHECK("prepare_repoint_kernel");
  }
  return FP_OK;
}

int fp_hbm_commit(const fp_store* store, void* stream) {
  if (int rc = check_store(store)) return rc;
  StoreView v{*store};
  commit_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(v);
  FP_LAUNCH_CHECK("commit_kernel");
  return FP_OK;
}

}  // extern "C"
