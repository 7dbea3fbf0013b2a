// Split-KV decode attention over compressed KV records for sm_100a.
//
// Replaces plan_decode / decode_attn / combine of the reference
// (fragpack/ops/fused_attn_decode.cu:94-163, 214-404, 407-425).
//
// Shape of the kernel:
//  * persistent CTAs (two per SM), each walking a static list of work items
//    (unit, KV head); a unit is a chunk of `ppc` pages of one sequence;
//  * per CTA one producer warp streams the items' K and V records as ONE flat
//    sequence through a ring of shared-memory slots with cp.async.bulk + mbarrier
//    (full / empty barriers), so the HBM pipeline does not drain at item
//    boundaries;
//  * eight consumer warps rebuild K / V bit-exactly in registers as
//    mma.m16n8k16 A fragments (the record layout is that fragment order) and run
//    S^T = K Q^T and O^T += V^T P^T with an fp32 online softmax; P is rounded to
//    BF16 for the second product and the denominator stays fp32, as in the
//    reference (fused_attn_decode.cu:329-345);
//  * one consumer barrier per page: probabilities are formed against the
//    running maximum, and only a page that raises some head's maximum takes a
//    second barrier to rescale.
// The page loop is issue-bound and sits at the register limit of two CTAs per
// SM; its speed moves by 5-10 % with small changes around it, so changes here
// are re-measured on the steady-state case before they are kept.
// Every device-side wait is bounded: when it runs out the CTA sets
// FP_DECODE_WAIT_TIMEOUT in the status word, stops waiting and finishes its
// control flow, so the context stays usable.
#include <math.h>

#include "fp_api.h"
#include "fp_common.cuh"
#include "fp_pipe.cuh"

namespace fpb {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = 32 * kConsumerWarps;  // 256 = fragment owners
constexpr int kThreads = kConsumers + 32;        // + producer warp
// Ring slots of the plain comparison kernel (always two CTAs per SM).
constexpr int kSlots = 3;
// The fused kernel comes in two shapes, named by the CTAs that fit one SM.
// Two: a three-slot record ring, separate escape scratch for K and V records,
// 96 registers per thread.  Three: half as many warps again to hide the
// decode's latencies, paid for with a two-slot ring, one escape scratch for K
// and V (hence a barrier at the end of every page) and 72 registers.  The
// three-CTA shape wins where CTAs stream many pages each (long contexts, big
// batches); the two-CTA shape where a CTA sees only a handful of pages.
template <int kCtas>
struct Shape {
  static constexpr int kSlots = kCtas == 3 ? 2 : 3;
  static constexpr int kEscBuffers = kCtas == 3 ? 1 : 2;
};
constexpr int kSlotBytes = kCodedMax;            // raw records are read in place
constexpr int kPRow = 80;                        // bytes per (head, c) row of P, padded
constexpr int kPBytes = 32 * kPRow;
constexpr int kPlanThreads = 256;

struct SlotDesc {
  int64_t addr;  // global address of the record (used for raw records)
  int32_t vlen;  // rec_len: bytes past the dense part; > kVarCap marks raw
  // Dynamic schedule only: the work item the record belongs to (-1: no more
  // items for this CTA) as the producer resolved it, so that the consumers
  // need no dependent global loads of their own at the start of an item.
  int32_t item;
  int32_t seq_index, first_page, pages, seq_len;
};

template <int kCtas>
struct Smem {
  static constexpr int kSlots = Shape<kCtas>::kSlots;
  static constexpr int kEscBuffers = Shape<kCtas>::kEscBuffers;
  __align__(128) uint8_t slots[kSlots][kSlotBytes];
  // With two buffers K and V records expand their escapes apart: the V decode
  // of a page and the K decode of the next one run without a barrier between.
  __align__(16) uint8_t esc[kEscBuffers][kEscBytes];
  __align__(16) uint8_t p[2][kPBytes];
  __align__(16) float ref[2][kConsumerWarps][8];
  __align__(16) float lsum[kConsumerWarps][8];
  float mrow[8];
  // Per item: Q^T B fragments in lane order and the K / V decode tables.
  __align__(16) uint2 qfrag[8][32];
  __align__(16) HeadTables tabs[2];
  SlotDesc desc[kSlots];
  __align__(8) uint64_t full[kSlots];
  __align__(8) uint64_t empty[kSlots];
  WaitState wait;
};

// kCtas CTAs must fit one SM: 228 KB per SM, 1 KB reserved per CTA.
static_assert(sizeof(Smem<2>) <= (228 * 1024) / 2 - 1024, "Smem<2> too large for two CTAs per SM");
static_assert(sizeof(Smem<3>) <= (228 * 1024) / 3 - 1024, "Smem<3> too large for three CTAs per SM");

struct DecodeParams {
  const uint32_t* q;
  const int64_t* rec_addr;
  const int32_t* rec_len;
  const int32_t* plut;
  const uint8_t* slut;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const int32_t* plan;
  float* opart;
  float* ml;
  int32_t* status;
  int32_t* dyn;       // dynamic schedule words of the plan (see plan_words)
  int64_t q_stride;   // in 32-bit words
  int64_t bt_stride;  // in entries
  int kvh, group, units, batch;
  float scale_log2;
  PipeConsts k;
  long long wait_limit;   // cycle budget of every bounded wait
  long long skip_record;  // test hook: ordinal of a record the producer leaves out (-1: none)
};

// Plan (int32): [0] pages of the longest unit, [1] units in use, [2 + 2u]
// sequence and [3 + 2u] first page | pages << 16 of unit u (sequence -1:
// idle), [2 + 2 units + 2 b] first unit and [.. + 1] chunk count of sequence b,
// then one spare word and the
// status word, then the words of the dynamic item schedule (batches with more
// (sequence, head) pairs than resident CTAs): the number of attention CTAs
// started since the plan was made, and one item counter per attention launch
// since then.  The planner zeroes them; CTAs of one launch are all counted
// before any CTA of the next (a dependent grid launches only when every CTA of
// its predecessor has allowed it, which they do after being counted), so a
// CTA's arrival number divided by the grid size is its launch's index.
constexpr int kMaxPlanLaunches = 256;  // launches per plan that are scheduled dynamically
constexpr int kDynWords = 4 + kMaxPlanLaunches;
__host__ __device__ __forceinline__ int64_t status_index(int units) { return 2 + 4LL * units + 1; }
__host__ __device__ __forceinline__ int64_t dyn_index(int units) { return status_index(units) + 1; }
// Behind them, 16-byte aligned: one descriptor per unit in the order in which
// the schedules hand the units out (sequence, first page | pages << 16,
// sequence length, unit), so that an item's start costs one load.
__host__ __device__ __forceinline__ int64_t desc_index(int units) { return dyn_index(units) + kDynWords; }
__host__ __device__ __forceinline__ int64_t plan_words(int units) { return desc_index(units) + 4LL * units; }
static_assert((2 + 2 + kDynWords) % 4 == 0, "the unit descriptors must start on a 16-byte boundary");

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
}

// The consumer barrier combined with an OR over a predicate of every consumer.
__device__ __forceinline__ bool consumer_barrier_or(bool mine) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(any)
      : "r"((uint32_t)mine), "n"(kConsumers)
      : "memory");
  return any != 0;
}

// d += A B, one m16n8k16 BF16 tile with fp32 accumulation.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------
// Work items.  Both roles enumerate the same items in the same order.
// ---------------------------------------------------------------------------
struct Item {
  int unit, head, seq_index, first_page, pages, seq_len;
};

__device__ __forceinline__ bool load_item(const DecodeParams& p, int item, Item& it) {
  // Items walk the planner's list of units by decreasing length, heads innermost.
  const int place = item / p.kvh;
  it.head = item - place * p.kvh;
  const int4 d = reinterpret_cast<const int4*>(p.plan + desc_index(p.units))[place];
  it.seq_index = d.x;
  if (it.seq_index < 0) return false;
  it.first_page = d.y & 0xffff;
  it.seq_len = d.z;
  it.unit = d.w;
  const int total = (it.seq_len + 127) >> 7;
  it.pages = max(0, min(total - it.first_page, d.y >> 16));
  return it.pages > 0;
}

// ---------------------------------------------------------------------------
// Producer warp
// ---------------------------------------------------------------------------
// kDynamic: items beyond the CTA's first come first come, first served from
// the launch's counter in the plan (CTAs that share an SM, or that got shorter
// items, come back sooner) and every record's descriptor names its item.
template <bool kDynamic, int kCtas>
__device__ __forceinline__ void produce(const DecodeParams& p, Smem<kCtas>& sm) {
  constexpr int kSlots = Shape<kCtas>::kSlots;
  const int lane = threadIdx.x & 31;
  WaitState* const wait = &sm.wait;
  volatile int* abort = &sm.wait.abort;
  const int n_items = p.plan[1] * p.kvh;
  uint32_t r = 0;  // records issued so far
  // Under a programmatic dependent launch the preceding grid may still run.
  // Closed pages and their table entries are never written by a kernel that
  // can immediately precede this one, so they stream at once; a sequence's last
  // page (the open block the token writer and the encoder touch) waits.
  bool synced = false;
  // Dynamic schedule.  The CTA's first item is its block index; later ones come
  // from the counter of this launch, which the CTA's arrival number selects
  // (past kMaxPlanLaunches launches per plan the static stride takes over).
  // The arrival is counted before this warp allows dependent grids to launch,
  // so that every CTA of a launch is counted before a CTA of the next one is;
  // its result is first needed when the first record is on its way.  The next
  // item is requested just before this one's last record is issued: late enough
  // that a CTA does not hoard an item it will not reach for a while, early
  // enough that the atomic's round trip hides behind the records in the ring.
  int arrival = 0;
  if (kDynamic && lane == 0) arrival = atomicAdd(&p.dyn[0], 1);
  bool counted = false;
  int launch = -1, turn = 0;
  auto count_arrival = [&] {
    if (!kDynamic || counted) return;
    launch = __shfl_sync(0xffffffffu, arrival, 0) / (int)gridDim.x;
    if (launch >= kMaxPlanLaunches) launch = -1;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    counted = true;
  };
  auto take = [&]() -> int {
    count_arrival();
    ++turn;
    if (!kDynamic || launch < 0) return blockIdx.x + turn * gridDim.x;
    int item = 0;
    if (lane == 0) item = atomicAdd(p.dyn + 4 + launch, 1);
    return __shfl_sync(0xffffffffu, item, 0) + gridDim.x;
  };
  int upcoming = blockIdx.x;
  while (upcoming < n_items) {
    const int item = upcoming;
    if (!kDynamic) upcoming = take();
    Item it;
    if (!load_item(p, item, it)) {
      if (kDynamic) upcoming = take();
      continue;
    }
    const int32_t* bt = p.block_table + (int64_t)it.seq_index * p.bt_stride + it.first_page;
    const int last_page = ((it.seq_len + 127) >> 7) - 1;
    for (int base = 0; base < it.pages; base += 32) {
      if (!synced && it.first_page + base + 32 > last_page) {
        grid_dependency_wait();
        synced = true;
      }
      const int page = base + lane;
      int64_t addr_k = 0, addr_v = 0;
      int32_t len_k = 0, len_v = 0;
      if (page < it.pages) {
        const int64_t idx = ((int64_t)bt[page] * 2) * p.kvh + it.head;
        addr_k = p.rec_addr[idx];
        addr_v = p.rec_addr[idx + p.kvh];
        len_k = p.rec_len[idx];
        len_v = p.rec_len[idx + p.kvh];
      }
      const int count = min(32, it.pages - base);
      for (int j = 0; j < 2 * count; ++j) {
        if (kDynamic && base + 32 >= it.pages && j == 2 * count - 1) upcoming = take();
        const int src = j >> 1;
        const int64_t addr = __shfl_sync(0xffffffffu, (j & 1) ? addr_v : addr_k, src);
        const int32_t vlen = __shfl_sync(0xffffffffu, (j & 1) ? len_v : len_k, src);
        const uint32_t slot = r % kSlots, use = r / kSlots;
        if (lane == 0) {
          bool ok = true;
          if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1, wait);
          if (ok && (long long)r != p.skip_record) {
            sm.desc[slot].addr = addr;
            sm.desc[slot].vlen = vlen;
            if (kDynamic) {
              sm.desc[slot].item = it.unit * p.kvh + it.head;  // unit and head, not the place in the schedule
              sm.desc[slot].seq_index = it.seq_index;
              sm.desc[slot].first_page = it.first_page;
              sm.desc[slot].pages = it.pages;
              sm.desc[slot].seq_len = it.seq_len;
            }
            if (vlen > kVarCap || vlen < kHeaderBytes) {
              // Raw records are read in place by the consumers; warm the L2.
              prefetch_l2(reinterpret_cast<const void*>(addr), kRawRecord);
              mbar_arrive(&sm.full[slot]);
            } else {
              const uint32_t bytes = (uint32_t)(kDenseBytes + (vlen & ~15));
              mbar_expect_tx(&sm.full[slot], bytes);
              bulk_load(sm.slots[slot], reinterpret_cast<const void*>(addr), bytes,
                        &sm.full[slot]);
            }
          }
        }
        ++r;
        __syncwarp();
        if (*abort) return;  // uniform: lane 0's write is ordered by the warp sync
        count_arrival();     // first record on its way: the count has long returned
      }
    }
  }
  if (kDynamic) {
    count_arrival();
    // End marker: the consumers learn from the ring that nothing follows.
    if (lane == 0) {
      const uint32_t slot = r % kSlots, use = r / kSlots;
      bool ok = true;
      if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1, wait);
      if (ok) {
        sm.desc[slot].item = -1;
        mbar_arrive(&sm.full[slot]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Consumer warps
// ---------------------------------------------------------------------------
template <bool kDynamic, int kCtas>
__device__ __forceinline__ void consume(const DecodeParams& p, Smem<kCtas>& sm) {
  constexpr int kSlots = Shape<kCtas>::kSlots;
  constexpr int kEscBuffers = Shape<kCtas>::kEscBuffers;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  WaitState* const wait = &sm.wait;
  const int n_items = p.plan[1] * p.kvh;
  // Records consumed so far (matches the producer's count).  A page is a K and
  // a V record, so bit 1 alternates per page: it selects the P / ref buffers.
  uint32_t r = 0;
  bool synced = false;

  auto release = [&](uint32_t slot) {
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[slot]);
  };

  for (int item = blockIdx.x;; item += gridDim.x) {
    Item it;
    if (kDynamic) {
      // The first record of the next item (or the end marker) names the item.
      const uint32_t head_slot = r % kSlots;
      const bool landed = bounded_wait(&sm.full[head_slot], (r / kSlots) & 1, wait);
      const SlotDesc& d = sm.desc[head_slot];
      // All consumer warps leave together (a warp that left alone would hang
      // the others at their next barrier): after a wait that ran out in any
      // warp, or at the end marker, which every warp reads alike.
      if (consumer_barrier_or(!landed || d.item < 0)) break;
      it.unit = d.item / p.kvh;
      it.head = d.item - it.unit * p.kvh;
      it.seq_index = d.seq_index;
      it.first_page = d.first_page;
      it.pages = d.pages;
      it.seq_len = d.seq_len;
    } else {
      if (item >= n_items) break;
      if (!load_item(p, item, it)) continue;
    }
    if (!synced) {
      // Queries come from, and partial results may still be read by, the
      // preceding grids: wait for them here, after the plan lookup, while the
      // producer already streams records.
      grid_dependency_wait();
      synced = true;
    }
    // Stage this item's Q^T B fragments (head g, zero beyond the group; dims
    // 16 st + 2 c and + 8) and decode tables in shared memory.  The barrier
    // that closed the previous item ordered its last reads before these writes.
    {
      const uint32_t* q =
          p.q + (int64_t)it.seq_index * p.q_stride + (int64_t)(it.head * p.group + g) * 64;
      const int st = warp;
      sm.qfrag[st][lane] = g < p.group ? make_uint2(q[8 * st + c], q[8 * st + 4 + c])
                                        : make_uint2(0u, 0u);
      if (tid < 2) sm.tabs[tid] = load_tables(p.plut, p.slut, tid * p.kvh + it.head);
    }
    consumer_barrier();
    // Thread (g, c) of warp w holds S[head 2c+e][token 16w + 8jj + g] in
    // s[2jj+e] and O[head 2c+e][dim 16w + 8jj + g] in o[2jj+e].
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    // Few values stay live across the page loop: pages to go, the sequence's
    // tokens from the current page on, and the row of the partial result.
    const int row0 = (it.head * p.units + it.unit) * 8;
    int tok_left = it.seq_len - it.first_page * 128;

    for (int left = it.pages; left > 0; --left, tok_left -= 128) {
      const int buf = (r >> 1) & 1;
      // ---------------- K: S^T = K Q^T
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const uint32_t slot = r % kSlots;
        // A record whose wait ran out contributes nothing (the status word
        // marks the step invalid); its descriptor is not trusted either.
        const bool landed = bounded_wait(&sm.full[slot], (r / kSlots) & 1, wait);
        const int32_t vlen = sm.desc[slot].vlen;
        auto qk = [&](int st, const uint32_t (&w)[4]) {
          const uint2 qb = sm.qfrag[st][lane];
          mma_16816(s, w[0], w[2], w[1], w[3], qb.x, qb.y);
        };
        if (!landed) {
        } else if (vlen > kVarCap || vlen < kHeaderBytes) {
          const uint8_t* rec = reinterpret_cast<const uint8_t*>(sm.desc[slot].addr);
          release(slot);
          raw_record_words(rec, tid, qk);
        } else {
          coded_record_words(sm.slots[slot], vlen, sm.tabs[0], sm.esc[0], tid, p.k, [&] { release(slot); }, qk);
        }
        ++r;
      }
      // ---------------- softmax bookkeeping
#pragma unroll
      for (int x = 0; x < 4; ++x) s[x] *= p.scale_log2;
      if (tok_left < 128) {  // the sequence's last page: mask its tail
        const int tok = 16 * warp + g;
        if (tok >= tok_left) s[0] = s[1] = -INFINITY;
        if (tok + 8 >= tok_left) s[2] = s[3] = -INFINITY;
      }
      float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
      for (int x = 4; x < 32; x <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], x));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], x));
      }
      const bool raised = __any_sync(0xffffffffu, mx[0] > m_run[0] || mx[1] > m_run[1]);
      if (g == 0) *reinterpret_cast<float2*>(&sm.ref[buf][warp][2 * c]) = make_float2(mx[0], mx[1]);
      // P rows: (head, c') holds, for every k-step st, the two B words
      // (tokens 16 st + 2 c' + {0,1} and + 8) of the second product.
      uint8_t* prow = sm.p[buf];
      auto put_p = [&](const float (&pv)[4]) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int head = 2 * c + e;
            *reinterpret_cast<__nv_bfloat16*>(prow + (head * 4 + (g >> 1)) * kPRow +
                                              4 * (2 * warp + jj) + 2 * (g & 1)) =
                __float2bfloat16_rn(pv[2 * jj + e]);
          }
      };
      float pv[4];
      if (!raised) {
#pragma unroll
        for (int x = 0; x < 4; ++x) pv[x] = fast_exp2(s[x] - m_run[x & 1]);
        put_p(pv);
      }
      {
        // One barrier per page, carrying "some warp's maximum rose".
        if (consumer_barrier_or(raised)) {
          // Some head's maximum rose: rescale the state, redo P against it.
          float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) {
            const float2 t = *reinterpret_cast<const float2*>(&sm.ref[buf][w][2 * c]);
            m_new[0] = fmaxf(m_new[0], t.x);
            m_new[1] = fmaxf(m_new[1], t.y);
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            // A head with no valid token yet keeps -inf; use 0 as its reference.
            const float base = m_new[e] == -INFINITY ? 0.f : m_new[e];
            const float alpha = fast_exp2(m_run[e] - base);
            l_run[e] *= alpha;
            o[e] *= alpha;
            o[2 + e] *= alpha;
            pv[e] = fast_exp2(s[e] - base);
            pv[2 + e] = fast_exp2(s[2 + e] - base);
            m_run[e] = m_new[e];
          }
          put_p(pv);
          consumer_barrier();
        }
      }
      l_run[0] += pv[0] + pv[2];
      l_run[1] += pv[1] + pv[3];

      // ---------------- V: O^T += V^T P^T
      {
        const uint32_t slot = r % kSlots;
        const bool landed = bounded_wait(&sm.full[slot], (r / kSlots) & 1, wait);
        const int32_t vlen = sm.desc[slot].vlen;
        const uint4* pw = reinterpret_cast<const uint4*>(prow + (g * 4 + c) * kPRow);
        uint4 b;
        auto pv_word = [&](int st, const uint32_t (&w)[4]) {
          if ((st & 1) == 0) b = pw[st >> 1];
          mma_16816(o, w[0], w[2], w[1], w[3], (st & 1) ? b.z : b.x, (st & 1) ? b.w : b.y);
        };
        if (!landed) {
        } else if (vlen > kVarCap || vlen < kHeaderBytes) {
          const uint8_t* rec = reinterpret_cast<const uint8_t*>(sm.desc[slot].addr);
          release(slot);
          const int rem = tok_left;
          if (rem < 128) {
            // An open block (always a raw record) may hold stale bytes of the
            // slot's previous owner beyond its last token: force them to zero
            // so that no stale NaN / Inf can meet a zero probability.
            raw_record_words(rec, tid, [&](int st, const uint32_t (&w)[4]) {
              uint32_t a[4] = {w[0], w[1], w[2], w[3]};
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const int t0 = 16 * st + 8 * (x & 1) + 2 * c;
                if (t0 >= rem) a[x] = 0u;
                else if (t0 + 1 >= rem) a[x] &= 0xffffu;
              }
              pv_word(st, a);
            });
          } else {
            raw_record_words(rec, tid, pv_word);
          }
        } else {
          coded_record_words(sm.slots[slot], vlen, sm.tabs[1], sm.esc[kEscBuffers - 1], tid, p.k, [&] { release(slot); },
                             pv_word);
        }
        ++r;
      }
      // One escape scratch for K and V: the next page's K decode must not
      // start expanding into it while another warp still reads this page's V.
      if (kEscBuffers == 1) consumer_barrier();
    }

    // ---------------- partial result of this (unit, head)
#pragma unroll
    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        p.opart[(int64_t)(row0 + 2 * c + e) * 128 + 16 * warp + 8 * jj + g] = o[2 * jj + e];
    float l[2] = {l_run[0], l_run[1]};
#pragma unroll
    for (int x = 4; x < 32; x <<= 1) {
      l[0] += __shfl_xor_sync(0xffffffffu, l[0], x);
      l[1] += __shfl_xor_sync(0xffffffffu, l[1], x);
    }
    if (g == 0) *reinterpret_cast<float2*>(&sm.lsum[warp][2 * c]) = make_float2(l[0], l[1]);
    if (warp == 0 && g == 0)
      *reinterpret_cast<float2*>(&sm.mrow[2 * c]) = make_float2(m_run[0], m_run[1]);
    consumer_barrier();
    if (tid < 8) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) sum += sm.lsum[w][tid];
      p.ml[(int64_t)(row0 + tid) * 2] = sm.mrow[tid];
      p.ml[(int64_t)(row0 + tid) * 2 + 1] = sum;
    }
    // The next item's first page barrier orders these reads before the next
    // writes of lsum / mrow.
  }
}

template <bool kDynamic, int kCtas>
__global__ void __launch_bounds__(kThreads, kCtas) decode_attn_kernel(DecodeParams p) {
  constexpr int kSlots = Shape<kCtas>::kSlots;
  extern __shared__ __align__(128) uint8_t dyn[];
  Smem<kCtas>& sm = *reinterpret_cast<Smem<kCtas>*>(dyn);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kConsumerWarps);
    }
    sm.wait.abort = 0;
    sm.wait.status = p.status;
    sm.wait.limit = p.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Prologue done (barriers initialised).  Each role waits for the preceding
  // grid where it first needs it (see produce / consume).  The merge kernel may
  // become resident now; it waits for this grid to complete before it reads.
  // (With the dynamic schedule the producer warp allows it only after its
  // arrival has been counted, see produce.)
  if (threadIdx.x >= kConsumers) {
    if (!kDynamic) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    produce<kDynamic, kCtas>(p, sm);
  } else {
    // With the dynamic schedule the producer warp alone allows dependents,
    // after its arrival has been counted (the instruction takes effect with
    // the first thread of the CTA that issues it).
    if (!kDynamic) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    consume<kDynamic, kCtas>(p, sm);
  }
  // Nothing may still be writing this CTA's shared memory when it exits: on
  // the normal path every issued copy has been consumed; after a timeout give
  // the copies in flight a bounded chance to land.
  __syncthreads();
  if (sm.wait.abort && threadIdx.x == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 20000000LL) {
    }
  }
}

// ---------------------------------------------------------------------------
// Comparison arm: the same split-KV kernel over PLAIN BF16 records (32 KB each,
// fragment order, the layout of raw / open / overflow records) with no decode
// step.  Same planner, same ring, same softmax and merge; every record is
// staged whole through a ring of 32 KB slots.  It answers "what does a plain
// BF16 paged read of the same logical KV cost on this GPU"; a coded record met
// here contributes zeros and raises FP_DECODE_NOT_PLAIN in the status word.
// ---------------------------------------------------------------------------
struct PlainSmem {
  __align__(128) uint8_t slots[kSlots][kRawRecord];
  __align__(16) uint8_t p[2][kPBytes];
  __align__(16) float ref[2][kConsumerWarps][8];
  __align__(16) float lsum[kConsumerWarps][8];
  float mrow[8];
  __align__(16) uint2 qfrag[8][32];
  int raw[kSlots];
  SlotDesc desc[kSlots];  // the item fields only (dynamic schedule)
  __align__(8) uint64_t full[kSlots];
  __align__(8) uint64_t empty[kSlots];
  WaitState wait;
};
static_assert(sizeof(PlainSmem) <= (228 * 1024) / 2 - 1024, "PlainSmem too large for two CTAs per SM");

template <bool kDynamic>
__device__ __forceinline__ void plain_produce(const DecodeParams& p, PlainSmem& sm) {
  const int lane = threadIdx.x & 31;
  WaitState* const wait = &sm.wait;
  volatile int* abort = &sm.wait.abort;
  const int n_items = p.plan[1] * p.kvh;
  uint32_t r = 0;
  bool synced = false;  // see produce(), also for the dynamic schedule below
  int arrival = 0;
  if (kDynamic && lane == 0) arrival = atomicAdd(&p.dyn[0], 1);
  bool counted = false;
  int launch = -1, turn = 0;
  auto count_arrival = [&] {
    if (!kDynamic || counted) return;
    launch = __shfl_sync(0xffffffffu, arrival, 0) / (int)gridDim.x;
    if (launch >= kMaxPlanLaunches) launch = -1;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    counted = true;
  };
  auto take = [&]() -> int {
    count_arrival();
    ++turn;
    if (!kDynamic || launch < 0) return blockIdx.x + turn * gridDim.x;
    int item = 0;
    if (lane == 0) item = atomicAdd(p.dyn + 4 + launch, 1);
    return __shfl_sync(0xffffffffu, item, 0) + gridDim.x;
  };
  int upcoming = blockIdx.x;
  while (upcoming < n_items) {
    const int item = upcoming;
    if (!kDynamic) upcoming = take();
    Item it;
    if (!load_item(p, item, it)) {
      if (kDynamic) upcoming = take();
      continue;
    }
    const int32_t* bt = p.block_table + (int64_t)it.seq_index * p.bt_stride + it.first_page;
    const int last_page = ((it.seq_len + 127) >> 7) - 1;
    for (int base = 0; base < it.pages; base += 32) {
      if (!synced && it.first_page + base + 32 > last_page) {
        grid_dependency_wait();
        synced = true;
      }
      const int page = base + lane;
      int64_t addr_k = 0, addr_v = 0;
      int32_t len_k = 0, len_v = 0;
      if (page < it.pages) {
        const int64_t idx = ((int64_t)bt[page] * 2) * p.kvh + it.head;
        addr_k = p.rec_addr[idx];
        addr_v = p.rec_addr[idx + p.kvh];
        len_k = p.rec_len[idx];
        len_v = p.rec_len[idx + p.kvh];
      }
      const int count = min(32, it.pages - base);
      for (int j = 0; j < 2 * count; ++j) {
        if (kDynamic && base + 32 >= it.pages && j == 2 * count - 1) upcoming = take();
        const int src = j >> 1;
        const int64_t addr = __shfl_sync(0xffffffffu, (j & 1) ? addr_v : addr_k, src);
        const int32_t vlen = __shfl_sync(0xffffffffu, (j & 1) ? len_v : len_k, src);
        const uint32_t slot = r % kSlots, use = r / kSlots;
        if (lane == 0) {
          bool ok = true;
          if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1, wait);
          if (ok) {
            const bool raw = vlen > kVarCap;
            sm.raw[slot] = raw;
            if (kDynamic) {
              sm.desc[slot].item = it.unit * p.kvh + it.head;  // unit and head, not the place in the schedule
              sm.desc[slot].seq_index = it.seq_index;
              sm.desc[slot].first_page = it.first_page;
              sm.desc[slot].pages = it.pages;
              sm.desc[slot].seq_len = it.seq_len;
            }
            if (raw) {
              mbar_expect_tx(&sm.full[slot], kRawRecord);
              bulk_load(sm.slots[slot], reinterpret_cast<const void*>(addr), kRawRecord,
                        &sm.full[slot]);
            } else {
              atomicOr(p.status, FP_DECODE_NOT_PLAIN);
              mbar_arrive(&sm.full[slot]);
            }
          }
        }
        ++r;
        __syncwarp();
        if (*abort) return;
        count_arrival();
      }
    }
  }
  if (kDynamic) {
    count_arrival();
    if (lane == 0) {  // end marker
      const uint32_t slot = r % kSlots, use = r / kSlots;
      bool ok = true;
      if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1, wait);
      if (ok) {
        sm.desc[slot].item = -1;
        mbar_arrive(&sm.full[slot]);
      }
    }
  }
}


template <bool kDynamic>
__device__ __forceinline__ void plain_consume(const DecodeParams& p, PlainSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  WaitState* const wait = &sm.wait;
  const int n_items = p.plan[1] * p.kvh;
  uint32_t r = 0, pages = 0;
  bool synced = false;

  // Owner words of the record in `slot` (zeros for a record that is not plain),
  // in two halves of four 16-byte words to stay inside the register budget;
  // the slot goes back to the producer once the warp has read its last word.
  auto record_words = [&](uint32_t slot, bool landed, auto&& emit) {
    const uint4* src = reinterpret_cast<const uint4*>(sm.slots[slot]);
    const bool raw = landed && sm.raw[slot] != 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint4 v[4];
#pragma unroll
      for (int x = 0; x < 4; ++x)
        v[x] = raw ? src[(4 * half + x) * kOwners + tid] : make_uint4(0u, 0u, 0u, 0u);
      if (half == 1) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[slot]);
      }
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const uint32_t w[4] = {v[x].x, v[x].y, v[x].z, v[x].w};
        emit(4 * half + x, w);
      }
    }
  };

  for (int item = blockIdx.x;; item += gridDim.x) {
    Item it;
    if (kDynamic) {
      const uint32_t head_slot = r % kSlots;
      const bool landed = bounded_wait(&sm.full[head_slot], (r / kSlots) & 1, wait);
      const SlotDesc& d = sm.desc[head_slot];
      // All consumer warps leave together (a warp that left alone would hang
      // the others at their next barrier): after a wait that ran out in any
      // warp, or at the end marker, which every warp reads alike.
      if (consumer_barrier_or(!landed || d.item < 0)) break;
      it.unit = d.item / p.kvh;
      it.head = d.item - it.unit * p.kvh;
      it.seq_index = d.seq_index;
      it.first_page = d.first_page;
      it.pages = d.pages;
      it.seq_len = d.seq_len;
    } else {
      if (item >= n_items) break;
      if (!load_item(p, item, it)) continue;
    }
    if (!synced) {
      grid_dependency_wait();
      synced = true;
    }
    {
      const uint32_t* q =
          p.q + (int64_t)it.seq_index * p.q_stride + (int64_t)(it.head * p.group + g) * 64;
      const int st = warp;
      sm.qfrag[st][lane] = g < p.group ? make_uint2(q[8 * st + c], q[8 * st + 4 + c])
                                        : make_uint2(0u, 0u);
    }
    consumer_barrier();
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[4] = {0.f, 0.f, 0.f, 0.f};

    for (int i = 0; i < it.pages; ++i, ++pages) {
      const int buf = pages & 1;
      const int page_tok0 = (it.first_page + i) * 128;
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const uint32_t slot = r % kSlots;
        const bool landed = bounded_wait(&sm.full[slot], (r / kSlots) & 1, wait);
        record_words(slot, landed, [&](int st, const uint32_t (&w)[4]) {
          const uint2 qb = sm.qfrag[st][lane];
          mma_16816(s, w[0], w[2], w[1], w[3], qb.x, qb.y);
        });
        ++r;
      }
#pragma unroll
      for (int x = 0; x < 4; ++x) s[x] *= p.scale_log2;
      if (page_tok0 + 128 > it.seq_len) {  // the sequence's last page: mask its tail
        const int tok = page_tok0 + 16 * warp + g;
        if (tok >= it.seq_len) s[0] = s[1] = -INFINITY;
        if (tok + 8 >= it.seq_len) s[2] = s[3] = -INFINITY;
      }
      float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
      for (int x = 4; x < 32; x <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], x));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], x));
      }
      const bool raised = __any_sync(0xffffffffu, mx[0] > m_run[0] || mx[1] > m_run[1]);
      if (g == 0) *reinterpret_cast<float2*>(&sm.ref[buf][warp][2 * c]) = make_float2(mx[0], mx[1]);
      uint8_t* prow = sm.p[buf];
      auto put_p = [&](const float (&pv)[4]) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int head = 2 * c + e;
            *reinterpret_cast<__nv_bfloat16*>(prow + (head * 4 + (g >> 1)) * kPRow +
                                              4 * (2 * warp + jj) + 2 * (g & 1)) =
                __float2bfloat16_rn(pv[2 * jj + e]);
          }
      };
      float pv[4];
      if (!raised) {
#pragma unroll
        for (int x = 0; x < 4; ++x) pv[x] = fast_exp2(s[x] - m_run[x & 1]);
        put_p(pv);
      }
      {
        // One barrier per page, carrying "some warp's maximum rose".
        if (consumer_barrier_or(raised)) {
          float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) {
            const float2 t = *reinterpret_cast<const float2*>(&sm.ref[buf][w][2 * c]);
            m_new[0] = fmaxf(m_new[0], t.x);
            m_new[1] = fmaxf(m_new[1], t.y);
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float base = m_new[e] == -INFINITY ? 0.f : m_new[e];
            const float alpha = fast_exp2(m_run[e] - base);
            l_run[e] *= alpha;
            o[e] *= alpha;
            o[2 + e] *= alpha;
            pv[e] = fast_exp2(s[e] - base);
            pv[2 + e] = fast_exp2(s[2 + e] - base);
            m_run[e] = m_new[e];
          }
          put_p(pv);
          consumer_barrier();
        }
      }
      l_run[0] += pv[0] + pv[2];
      l_run[1] += pv[1] + pv[3];
      {
        const uint32_t slot = r % kSlots;
        const bool landed = bounded_wait(&sm.full[slot], (r / kSlots) & 1, wait);
        const uint4* pw = reinterpret_cast<const uint4*>(prow + (g * 4 + c) * kPRow);
        const int rem = it.seq_len - page_tok0;
        uint4 b;
        record_words(slot, landed, [&](int st, const uint32_t (&w)[4]) {
          uint32_t a[4] = {w[0], w[1], w[2], w[3]};
          if (rem < 128) {
            // Stale bytes beyond the last token of an open block must not meet
            // a zero probability as NaN / Inf.
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const int t0 = 16 * st + 8 * (x & 1) + 2 * c;
              if (t0 >= rem) a[x] = 0u;
              else if (t0 + 1 >= rem) a[x] &= 0xffffu;
            }
          }
          if ((st & 1) == 0) b = pw[st >> 1];
          mma_16816(o, a[0], a[2], a[1], a[3], (st & 1) ? b.z : b.x, (st & 1) ? b.w : b.y);
        });
        ++r;
      }
    }

    const int64_t row0 = ((int64_t)it.head * p.units + it.unit) * 8;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        p.opart[(row0 + 2 * c + e) * 128 + 16 * warp + 8 * jj + g] = o[2 * jj + e];
    float l[2] = {l_run[0], l_run[1]};
#pragma unroll
    for (int x = 4; x < 32; x <<= 1) {
      l[0] += __shfl_xor_sync(0xffffffffu, l[0], x);
      l[1] += __shfl_xor_sync(0xffffffffu, l[1], x);
    }
    if (g == 0) *reinterpret_cast<float2*>(&sm.lsum[warp][2 * c]) = make_float2(l[0], l[1]);
    if (warp == 0 && g == 0)
      *reinterpret_cast<float2*>(&sm.mrow[2 * c]) = make_float2(m_run[0], m_run[1]);
    consumer_barrier();
    if (tid < 8) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) sum += sm.lsum[w][tid];
      p.ml[(row0 + tid) * 2] = sm.mrow[tid];
      p.ml[(row0 + tid) * 2 + 1] = sum;
    }
  }
}

template <bool kDynamic>
__global__ void __launch_bounds__(kThreads, 2) plain_attn_kernel(DecodeParams p) {
  extern __shared__ __align__(128) uint8_t dyn[];
  PlainSmem& sm = *reinterpret_cast<PlainSmem*>(dyn);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kConsumerWarps);
    }
    sm.wait.abort = 0;
    sm.wait.status = p.status;
    sm.wait.limit = p.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x >= kConsumers) {
    if (!kDynamic) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    plain_produce<kDynamic>(p, sm);
  } else {
    if (!kDynamic) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    plain_consume<kDynamic>(p, sm);
  }
  __syncthreads();
  if (sm.wait.abort && threadIdx.x == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 20000000LL) {
    }
  }
}

// Merges the chunk partials of every sequence into BF16 out[B, H * group, 128]:
// grid (B, H), one warp per query head, four dims per lane.  Rows without
// context (CUDA-graph padding) become zeros.  A separate launch on purpose:
// merging inside the attention kernel needs a device-wide fence per item, which
// was measured to cost several microseconds each under load.  The launch is
// programmatically dependent on the attention kernel, so its blocks are already
// resident (and past their index arithmetic) when the last partial lands.
// The kernel is a chain of dependent memory round trips (plan, then partials),
// so it keeps that chain short: every lane reads the same (max, sum) pairs and
// needs no shuffle, and sixteen chunks are in flight per round with an online
// rescale between rounds instead of a separate pass for the maximum.
constexpr int kMergeRound = 16;

// Destinations of the merged rows in a tensor-parallel group (world == 0: the
// caller's own `out` only) and the flags of the arrival protocol.
struct PeerOut {
  __nv_bfloat16* out[FP_MAX_PEERS];
  int64_t offset;  // elements: copy `buffer` and this rank's first head
  int world;
};
struct PeerFlags {
  int32_t* flag[FP_MAX_PEERS];
  int32_t* epoch;
  int32_t* status;
  int world, rank;
};

__global__ void __launch_bounds__(256)
combine_kernel(const float* opart, const float* ml, const int32_t* plan, __nv_bfloat16* out,
               int64_t out_stride, int units, int group, PeerOut dests) {
  const int b = blockIdx.x, kv_head = blockIdx.y;
  const int head = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Let the next grid in the stream start its prologue now; it waits for this
  // grid before it touches anything this grid reads or writes.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The plan was complete before the attention grid started, so the sequence's
  // chunk list is read while that grid may still be running: one dependent
  // round trip less after it finishes.
  const int2 seq = *reinterpret_cast<const int2*>(plan + 2 + 2 * units + 2 * b);
  const int first = seq.x, chunks = seq.y;
  const int64_t base = ((int64_t)kv_head * units + first) * 8 + head;
  // The partial results read below are written by the attention grid: wait for it.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (head >= group) return;
  float top = -INFINITY, den = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < chunks; s0 += kMergeRound) {
    float2 mlv[kMergeRound];
    float4 part[kMergeRound];
#pragma unroll
    for (int k = 0; k < kMergeRound; ++k) {
      const int64_t row = base + 8LL * min(s0 + k, chunks - 1);
      mlv[k] = *reinterpret_cast<const float2*>(ml + row * 2);
      part[k] = reinterpret_cast<const float4*>(opart + row * 128)[lane];
    }
    float round_top = top;
#pragma unroll
    for (int k = 0; k < kMergeRound; ++k)
      if (s0 + k < chunks) round_top = fmaxf(round_top, mlv[k].x);
    if (round_top == -INFINITY) continue;  // only chunks without a valid token so far
    const float keep = exp2f(top - round_top);  // 0 while top is still -inf
    den *= keep;
    acc.x *= keep;
    acc.y *= keep;
    acc.z *= keep;
    acc.w *= keep;
    top = round_top;
#pragma unroll
    for (int k = 0; k < kMergeRound; ++k) {
      const float wgt = s0 + k < chunks ? exp2f(mlv[k].x - top) : 0.f;
      den += wgt * mlv[k].y;
      acc.x += wgt * part[k].x;
      acc.y += wgt * part[k].y;
      acc.z += wgt * part[k].z;
      acc.w += wgt * part[k].w;
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  const int64_t at = (int64_t)b * out_stride + ((int64_t)kv_head * group + head) * 128 + 4 * lane;
  if (dests.world == 0) {
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + at);
    dst[0] = lo;
    dst[1] = hi;
  } else {
    // One 8-byte store per destination rank: 256 contiguous bytes per warp,
    // through the peer mapping for the other ranks.
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&lo);
    v.y = *reinterpret_cast<const uint32_t*>(&hi);
#pragma unroll
    for (int r = 0; r < FP_MAX_PEERS; ++r)  // constant indices keep the pointers in registers
      if (r < dests.world) *reinterpret_cast<uint2*>(dests.out[r] + dests.offset + at) = v;
  }
}

// Arrival of this rank's merged rows at every rank: runs after the merge kernel
// (stream order), so the fence below covers every row it stored.  Lane r tells
// rank r; lane 0 advances the local call counter.
__global__ void peer_signal_kernel(PeerFlags f) {
  const int r = threadIdx.x;
  const int arrived = *f.epoch + 1;
  __syncwarp();
  __threadfence_system();
  int32_t* mine = nullptr;
#pragma unroll
  for (int x = 0; x < FP_MAX_PEERS; ++x)
    if (x == r) mine = f.flag[x];
  if (r < f.world) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(mine + f.rank), "r"(arrived)
                 : "memory");
  }
  if (r == 0) *f.epoch = arrived;
}

// Waits (bounded) until every rank has arrived `*epoch` times.  Runs after
// peer_signal_kernel of the same call, so *epoch is this call's number.
__global__ void peer_wait_kernel(PeerFlags f) {
  const int r = threadIdx.x;
  if (r >= f.world) return;
  const int want = *f.epoch;
  const int32_t* word = nullptr;
#pragma unroll
  for (int x = 0; x < FP_MAX_PEERS; ++x)
    if (x == f.rank) word = f.flag[x] + r;
  const long long t0 = clock64();
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
    if (seen - want >= 0) return;
    if (clock64() - t0 > kWaitCycles) {
      atomicOr(f.status, FP_PEER_WAIT_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}

// ---------------------------------------------------------------------------
// Planner: one CTA, once per step.  Cuts the sequences into units (chunks of
// consecutive pages), lists the units by decreasing length and maps them to
// (sequence, first page, pages).  Both schedules walk that list, so a CTA's
// items are one long, one medium, one short instead of whatever the sequence
// order deals; and since the block scheduler deals CTAs breadth first (one per
// SM per pass: CTA i, i + SMs, i + 2 SMs meet on one SM), so are an SM's.
//
// Sequences of one length (the usual padded decode batch): a candidate shares
// t * SMs items out over the sequences - some get one chunk more than the
// others - or gives every sequence k chunks, and cuts every sequence into
// equal chunks (a page apart at most).
// There are at most four chunk lengths, so the makespan of the static walk is
// known exactly: the first CTA takes the longest item of every round, the
// first SM the longest of every pass; the cost is the larger of the two (an
// SM's CTAs share its decode throughput), an item costing its pages plus about
// three quarters of a page of start-up.
//
// Ragged batches: candidate k cuts the longest sequence into k chunks of ppc
// pages and every sequence into chunks of at most ppc; rounds of the longest
// item, or, first come first served, the even share plus one item.
//
// Plan words: [0] longest unit in pages, [1] units in use, then per unit
// (sequence or -1, first page | pages << 16), then per sequence (first unit,
// units); behind the status and schedule words the units again, by decreasing
// length, as (sequence, first page | pages << 16, sequence length, unit).
// ---------------------------------------------------------------------------
__device__ __forceinline__ int block_reduce_sum(int v, int* scratch) {
#pragma unroll
  for (int x = 16; x; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < kPlanThreads / 32; ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ int block_reduce_max(int v, int* scratch) {
#pragma unroll
  for (int x = 16; x; x >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, x));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < kPlanThreads / 32; ++w) t = max(t, scratch[w]);
  return t;
}

// Exclusive prefix of `v` over the block; `total` receives the block's sum.
__device__ __forceinline__ int block_exclusive_sum(int v, int* warp_total, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int before = warp_exclusive_sum(v, lane);
  __syncthreads();
  if (lane == 31) warp_total[warp] = before + v;
  __syncthreads();
  int first = before;
  total = 0;
#pragma unroll
  for (int w = 0; w < kPlanThreads / 32; ++w) {
    if (w < warp) first += warp_total[w];
    total += warp_total[w];
  }
  return first;
}

// Units are sorted by length up to this many pages (131,072 tokens); longer
// ones - contexts beyond what the reference's tests reach - share the last bin.
constexpr int kMaxUnitPages = 1024;

// A batch of `active` sequences of `n` pages cut into `target` units: `more`
// sequences (the first ones) get `fewest + 1` chunks, the others `fewest`.
struct EvenCut {
  int fewest, more;
};
__device__ __forceinline__ EvenCut even_cut(int target, int active, int n) {
  EvenCut c;
  c.fewest = target / active;
  c.more = target - c.fewest * active;
  if (c.fewest >= n) {  // cannot cut finer than pages
    c.fewest = n;
    c.more = 0;
  }
  return c;
}

// Sum of the item costs (4 pages + 3) at ranks 0, bins, 2 bins, .. of the
// items listed by decreasing length; `pages[x]` (decreasing) occurs `count[x]` times.
__device__ __forceinline__ long long first_of_every_round(const int (&pages)[4], const long long (&count)[4],
                                                          long long bins) {
  long long sum = 0, start = 0;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const long long end = start + count[x];
    // multiples of `bins` in [start, end)
    const long long hits = (end + bins - 1) / bins - (start + bins - 1) / bins;
    sum += hits * (4LL * pages[x] + 3);
    start = end;
  }
  return sum;
}

__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const int32_t* seq_lens, int32_t* plan, int batch, int units, int kvh, int slots, int sms,
            int dynamic) {
  __shared__ int scratch[kPlanThreads / 32];
  __shared__ int warp_total[kPlanThreads / 32];
  __shared__ unsigned long long best;
  __shared__ int bins[kMaxUnitPages + 1];
  const int tid = threadIdx.x;
  int total = 0, longest = 0, active = 0;
  int short_gap = 0;  // (1 << 30) - pages of the shortest sequence with context (0: none yet)
  for (int b = tid; b < batch; b += kPlanThreads) {
    const int n = (seq_lens[b] + 127) >> 7;
    total += n;
    longest = max(longest, n);
    if (n > 0) short_gap = max(short_gap, (1 << 30) - n);
    active += n > 0;
  }
  total = block_reduce_sum(total, scratch);
  longest = block_reduce_max(longest, scratch);
  short_gap = block_reduce_max(short_gap, scratch);
  active = block_reduce_sum(active, scratch);
  const bool ragged = short_gap > 0 && (1 << 30) - short_gap != longest;
  // Each padding row gives back the unit reserved for it.
  const int capacity = max(1, units - batch + active);
  if (tid == 0) best = ~0ull;
  for (int i = tid; i <= kMaxUnitPages; i += kPlanThreads) bins[i] = 0;
  __syncthreads();

  if (active > 0 && !ragged) {
    // Candidates: t * SMs items (threads 1 .. 127) and k chunks per sequence
    // (threads 128 ..; k = 1 is the coarsest cut).
    const long long target = tid < kPlanThreads / 2 ? (long long)tid * sms / kvh
                                                    : (long long)(tid - kPlanThreads / 2 + 1) * active;
    if (target >= active && target <= min(capacity, 0xfffff)) {
      const int n = longest;
      const EvenCut cut = even_cut((int)target, active, n);
      // Chunk lengths, decreasing: sequences with `fewest` chunks have the
      // longer ones; within a sequence `n mod chunks` chunks have a page more.
      int pages[4];
      long long count[4];
      const int few = cut.fewest, many = min(cut.fewest + 1, n);
      pages[1] = n / few;
      pages[0] = pages[1] + 1;
      count[0] = (long long)(active - cut.more) * (n - pages[1] * few) * kvh;
      count[1] = (long long)(active - cut.more) * few * kvh - count[0];
      pages[3] = n / many;
      pages[2] = pages[3] + 1;
      count[2] = (long long)cut.more * (n - pages[3] * many) * kvh;
      count[3] = (long long)cut.more * many * kvh - count[2];
      if (pages[2] > pages[1]) {  // n / many + 1 may exceed n / few only when they are equal
        const int p = pages[1];
        const long long c = count[1];
        pages[1] = pages[2];
        count[1] = count[2];
        pages[2] = p;
        count[2] = c;
      }
      const long long per_sm = slots / sms;
      const unsigned long long cost =
          (unsigned long long)max(first_of_every_round(pages, count, slots) * per_sm,
                                  first_of_every_round(pages, count, sms));
      // Ties go to the coarser cut (fewer partial results).
      atomicMin(&best, (cost << 20) | (unsigned long long)target);
    }
  } else if (active > 0) {
    // Candidate k cuts the longest sequence into k chunks.
    const int ppc = max(1, (longest + tid) / (tid + 1));
    const float inv = 1.0f / (float)ppc;
    int chunks = 0;
    for (int b = 0; b < batch; ++b) {
      // ceil(pages / ppc) without an integer division: estimate, then correct.
      const int up = ((seq_lens[b] + 127) >> 7) + ppc - 1;
      int q = (int)((float)up * inv);
      if (q * ppc > up) --q;
      if ((q + 1) * ppc <= up) ++q;
      chunks += q;
    }
    if (chunks <= capacity) {
      // Costs in quarter pages.  A static schedule: every CTA runs `rounds`
      // items.  Ragged items taken first come, first served: the step ends
      // within one item of the even share.
      const long long items = (long long)chunks * kvh;
      const long long rounds = max(1LL, (items + slots - 1) / slots);
      const long long one = 4LL * ppc + 3;
      const long long share = (4LL * total * kvh + 3 * items + slots - 1) / slots;
      const unsigned long long cost =
          (unsigned long long)(dynamic && items > slots ? share + one : rounds * one);
      // Ties go to the longer chunk (fewer partial results).
      atomicMin(&best, (cost << 20) | (unsigned long long)(0xfffff - ppc));
    }
  }
  __syncthreads();
  const int choice = (int)(best & 0xfffff);
  const int ppc = 0xfffff - choice;  // ragged batches
  const EvenCut cut = even_cut(!ragged && active > 0 ? choice : 1, max(active, 1), max(longest, 1));

  // Units, sequence by sequence; a sequence's chunks are consecutive units.
  int32_t* seq_plan = plan + 2 + 2 * units;
  int used = 0, seen = 0, top = 0;
  for (int base = 0; base < batch; base += kPlanThreads) {
    const int b = base + tid;
    const int n = b < batch ? (seq_lens[b] + 127) >> 7 : 0;
    int tile_active;
    const int rank = seen + block_exclusive_sum(n > 0, warp_total, tile_active);  // among the active sequences
    int chunks = 0;
    if (n > 0) chunks = ragged ? (n + ppc - 1) / ppc : min(cut.fewest + (rank < cut.more), n);
    int tile_units;
    const int first = used + block_exclusive_sum(chunks, warp_total, tile_units);
    if (b < batch) {
      seq_plan[2 * b] = first;
      seq_plan[2 * b + 1] = chunks;
      if (chunks > 0) {
        // Ragged: chunks of ppc pages and a remainder.  Else equal chunks, the
        // first `extra` of them a page longer.
        const int small = ragged ? ppc : n / chunks;
        const int extra = ragged ? 0 : n - small * chunks;
        int page = 0;
        for (int s = 0; s < chunks; ++s) {
          const int pages = min(small + (s < extra), n - page);
          plan[2 + 2 * (first + s)] = b;
          plan[3 + 2 * (first + s)] = page | (pages << 16);
          atomicAdd(&bins[min(pages, kMaxUnitPages)], 1);
          top = max(top, pages);
          page += pages;
        }
      }
    }
    used += tile_units;
    seen += tile_active;
  }
  for (int u = used + tid; u < units; u += kPlanThreads) plan[2 + 2 * u] = -1;
  top = block_reduce_max(top, scratch);

  // The units by decreasing length: bins[p] -> place of the first unit of p
  // pages; thread t scans the four lengths 1024 - 4 t .. 1021 - 4 t.
  static_assert(kMaxUnitPages == 4 * kPlanThreads, "one thread scans four bins");
  __syncthreads();
  {
    int count[4], mine = 0;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      count[x] = bins[kMaxUnitPages - (4 * tid + x)];
      mine += count[x];
    }
    int all;
    int at = block_exclusive_sum(mine, warp_total, all);
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      bins[kMaxUnitPages - (4 * tid + x)] = at;
      at += count[x];
    }
  }
  __syncthreads();
  int4* desc = reinterpret_cast<int4*>(plan + desc_index(units));
  for (int u = tid; u < used; u += kPlanThreads) {
    const int b = plan[2 + 2 * u], where = plan[3 + 2 * u];
    desc[atomicAdd(&bins[min(where >> 16, kMaxUnitPages)], 1)] = make_int4(b, where, seq_lens[b], u);
  }
  for (int u = used + tid; u < units; u += kPlanThreads) desc[u] = make_int4(-1, 0, 0, 0);
  if (tid == 0) {
    plan[0] = top;
    plan[1] = used;
    plan[status_index(units) - 1] = 0;
    plan[status_index(units)] = 0;
  }
  for (int i = tid; i < kDynWords; i += kPlanThreads) plan[dyn_index(units) + i] = 0;
}

}  // namespace

int device_sms() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace fpb

using namespace fpb;

namespace {

// Shared body of fp_fused_decode and fp_plain_decode: argument checks, planner,
// attention kernel (`plain` selects the comparison arm), merge kernel.
int launch_decode(bool plain, const fp_peers* peers, int buffer, const void* q, int64_t q_stride,
                  const int64_t* rec_addr,
                  const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                  const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                  float* opart, int64_t opart_elems, float* ml, int64_t ml_elems, int32_t* plan,
                  int64_t plan_elems, void* out, int64_t out_stride, int32_t batch,
                  int32_t kv_heads, int32_t group, int32_t units, int32_t replan, float scale,
                  int32_t num_sms, void* stream) {
  if (batch == 0) return FP_OK;
  FP_REQUIRE(batch > 0 && kv_heads > 0, "bad batch %d / kv_heads %d", batch, kv_heads);
  FP_REQUIRE(group == 1 || group == 2 || group == 4 || group == 8,
             "query group %d must be 1, 2, 4 or 8", group);
  FP_REQUIRE(units >= batch, "decode needs at least one unit per sequence");
  // A unit's first page and page count are packed into 16 bits each in the plan.
  FP_REQUIRE(bt_stride <= 32767, "block tables of more than 32767 pages per sequence are not supported");
  FP_REQUIRE((int64_t)kv_heads * units * 8 < (1LL << 31), "kv_heads * units too large");
  FP_REQUIRE(q && rec_addr && rec_len && (plain || (plut && slut)) && block_table && seq_lens &&
                 opart && ml && plan && (out || peers),
             "null decode argument");
  PeerOut dests = {};
  PeerFlags flags = {};
  if (peers) {
    FP_REQUIRE(peers->world >= 1 && peers->world <= FP_MAX_PEERS && peers->rank >= 0 &&
                   peers->rank < peers->world && (buffer == 0 || buffer == 1) && peers->epoch &&
                   peers->status,
               "bad peer group (world %d, rank %d, buffer %d)", peers->world, peers->rank, buffer);
    const int64_t row = (int64_t)peers->world * kv_heads * group * 128;
    FP_REQUIRE(out_stride >= row, "gathered rows hold %lld elements, stride is %lld",
               (long long)row, (long long)out_stride);
    for (int r = 0; r < peers->world; ++r) {
      FP_REQUIRE(peers->out[r] && peers->flag[r] &&
                     reinterpret_cast<uintptr_t>(peers->out[r]) % 8 == 0,
                 "peer %d has no buffer", r);
      dests.out[r] = static_cast<__nv_bfloat16*>(peers->out[r]);
      flags.flag[r] = peers->flag[r];
    }
    dests.offset = (int64_t)buffer * batch * out_stride + (int64_t)peers->rank * kv_heads * group * 128;
    dests.world = peers->world;
    flags.epoch = peers->epoch;
    flags.status = peers->status;
    flags.world = peers->world;
    flags.rank = peers->rank;
  }
  FP_REQUIRE(q_stride % 2 == 0 && reinterpret_cast<uintptr_t>(q) % 4 == 0,
             "q rows must be 4-byte aligned");
  FP_REQUIRE(plain || reinterpret_cast<uintptr_t>(slut) % 16 == 0, "slut must be 16-byte aligned");
  FP_REQUIRE(opart_elems >= (int64_t)kv_heads * units * 8 * 128 &&
                 ml_elems >= (int64_t)kv_heads * units * 16,
             "decode workspace too small");
  FP_REQUIRE(plan_elems >= plan_words(units), "decode plan must hold %lld int32",
             (long long)plan_words(units));
  FP_REQUIRE(reinterpret_cast<uintptr_t>(plan) % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(opart) % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(ml) % 8 == 0,
             "decode workspace must be 16-byte aligned");
  FP_REQUIRE(out_stride % 4 == 0 || (!peers && out_stride % 2 == 0),
             "out rows must be 4-byte aligned (8-byte in a peer group)");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(out) % 4 == 0, "out rows must be 4-byte aligned");
  const int sms = num_sms > 0 ? num_sms : device_sms();
  // The fused kernel's shape (see Shape): three CTAs per SM when the CTAs will
  // stream many pages each.  The rule reads the call's shape only - sequence x
  // head pairs times the block-table width (an upper bound of the pages of a
  // sequence), per CTA of the two-CTA grid - so every layer of a step, and
  // every replay of a captured graph, takes the same kernel.
  const long long pages_bound = (long long)batch * kv_heads * (bt_stride > 0 ? bt_stride : 1);
  const bool three = !plain && pages_bound >= 24LL * 2 * sms;
  const int slots = (three ? 3 : 2) * sms;
  cudaStream_t st = (cudaStream_t)stream;
  // More (sequence, head) pairs than resident CTAs: CTAs run several items, of
  // ragged sizes in a ragged batch, and taking them first come, first served
  // pays; with fewer pairs every CTA has at most one item either way.  The rule
  // depends on the call's shape only, so all layers of a step agree.
  const bool dynamic = (long long)batch * kv_heads > slots;
  if (replan) {
    plan_kernel<<<1, kPlanThreads, 0, st>>>(seq_lens, plan, batch, units, kv_heads, slots, sms,
                                            dynamic ? 1 : 0);
    FP_LAUNCH_CHECK("plan_kernel");
  }
  DecodeParams p;
  p.q = static_cast<const uint32_t*>(q);
  p.rec_addr = rec_addr;
  p.rec_len = rec_len;
  p.plut = plut;
  p.slut = slut;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.plan = plan;
  p.opart = opart;
  p.ml = ml;
  p.status = plan + status_index(units);
  p.dyn = plan + dyn_index(units);
  p.q_stride = q_stride / 2;
  p.bt_stride = bt_stride;
  p.kvh = kv_heads;
  p.group = group;
  p.units = units;
  p.batch = batch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.k = pipe_consts();
  p.wait_limit = wait_debug().limit;
  p.skip_record = wait_debug().skip_record;
  void (*kernel)(DecodeParams) =
      plain ? (dynamic ? plain_attn_kernel<true> : plain_attn_kernel<false>)
      : three ? (dynamic ? decode_attn_kernel<true, 3> : decode_attn_kernel<false, 3>)
              : (dynamic ? decode_attn_kernel<true, 2> : decode_attn_kernel<false, 2>);
  const char* name = plain ? "plain_attn_kernel" : "decode_attn_kernel";
  const int smem = plain ? (int)sizeof(PlainSmem)
                         : three ? (int)sizeof(Smem<3>) : (int)sizeof(Smem<2>);
  // The shared memory limit is set once per device and kernel, not per call.
  static std::atomic<uint64_t> smem_allowed[6];
  if (int rc = allow_dynamic_smem(kernel, smem,
                                  smem_allowed[(plain ? 4 : three ? 2 : 0) + (dynamic ? 1 : 0)]))
    return rc;
  const long long max_items = (long long)units * kv_heads;
  const int grid = (int)(max_items < slots ? max_items : slots);
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (int rc = cuda_status(cudaLaunchKernelEx(&cfg, kernel, p), name)) return rc;
  }
  {
    // Programmatic dependent launch: the merge may be scheduled while the
    // attention grid drains; it waits for that grid inside the kernel.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(batch, kv_heads);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* opart_c = opart;
    const float* ml_c = ml;
    const int32_t* plan_c = plan;
    __nv_bfloat16* out_c = static_cast<__nv_bfloat16*>(out);
    if (int rc = cuda_status(cudaLaunchKernelEx(&cfg, combine_kernel, opart_c, ml_c, plan_c, out_c,
                                                out_stride, (int)units, (int)group, dests),
                             "combine_kernel"))
      return rc;
  }
  FP_LAUNCH_CHECK("combine_kernel");
  if (peers) {
    // Plain launches: each starts when the kernel before it has completed.
    peer_signal_kernel<<<1, 32, 0, st>>>(flags);
    FP_LAUNCH_CHECK("peer_signal_kernel");
    peer_wait_kernel<<<1, 32, 0, st>>>(flags);
    FP_LAUNCH_CHECK("peer_wait_kernel");
  }
  return FP_OK;
}

}  // namespace

extern "C" {

int fp_decode_workspace(int32_t kv_heads, int32_t units, int64_t* opart_elems, int64_t* ml_elems,
                        int64_t* plan_elems) {
  FP_REQUIRE(kv_heads > 0 && units > 0, "bad workspace geometry");
  const int64_t rows = (int64_t)kv_heads * units * 8;
  if (opart_elems) *opart_elems = rows * 128;
  if (ml_elems) *ml_elems = rows * 2;
  if (plan_elems) *plan_elems = plan_words(units);
  return FP_OK;
}

int fp_fused_decode(const void* q, int64_t q_stride, const int64_t* rec_addr,
                    const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                    float* opart, int64_t opart_elems, float* ml, int64_t ml_elems, int32_t* plan,
                    int64_t plan_elems, void* out, int64_t out_stride, int32_t batch,
                    int32_t kv_heads, int32_t group, int32_t units, int32_t replan, float scale,
                    int32_t num_sms, void* stream) {
  return launch_decode(false, nullptr, 0, q, q_stride, rec_addr, rec_len, plut, slut, block_table,
                       bt_stride, seq_lens, opart, opart_elems, ml, ml_elems, plan, plan_elems, out,
                       out_stride, batch, kv_heads, group, units, replan, scale, num_sms, stream);
}

int fp_fused_decode_peers(const void* q, int64_t q_stride, const int64_t* rec_addr,
                          const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                          const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                          float* opart, int64_t opart_elems, float* ml, int64_t ml_elems,
                          int32_t* plan, int64_t plan_elems, const fp_peers* peers,
                          int32_t buffer, int64_t out_stride, int32_t batch, int32_t kv_heads,
                          int32_t group, int32_t units, int32_t replan, float scale,
                          int32_t num_sms, void* stream) {
  FP_REQUIRE(peers, "null peer group");
  return launch_decode(false, peers, buffer, q, q_stride, rec_addr, rec_len, plut, slut,
                       block_table, bt_stride, seq_lens, opart, opart_elems, ml, ml_elems, plan,
                       plan_elems, nullptr, out_stride, batch, kv_heads, group, units, replan,
                       scale, num_sms, stream);
}

int fp_plain_decode(const void* q, int64_t q_stride, const int64_t* rec_addr,
                    const int32_t* rec_len, const int32_t* block_table, int64_t bt_stride,
                    const int32_t* seq_lens, float* opart, int64_t opart_elems, float* ml,
                    int64_t ml_elems, int32_t* plan, int64_t plan_elems, void* out,
                    int64_t out_stride, int32_t batch, int32_t kv_heads, int32_t group,
                    int32_t units, int32_t replan, float scale, int32_t num_sms, void* stream) {
  return launch_decode(true, nullptr, 0, q, q_stride, rec_addr, rec_len, nullptr, nullptr, block_table,
                       bt_stride, seq_lens, opart, opart_elems, ml, ml_elems, plan, plan_elems,
                       out, out_stride, batch, kv_heads, group, units, replan, scale, num_sms,
                       stream);
}

/*
 * Decode attention for callers that may not allocate device memory.
 *
 * Some hosts of this library hand it a CUDA context in which they own every
 * allocation: an engine that carved the whole device into its own pools at
 * start-up, a plugin running inside someone else's memory planner, a worker
 * whose allocator is locked once serving begins.  Such callers cannot provide
 * (or grow) the opart / ml / plan workspace that fp_fused_decode needs.  This
 * variant keeps that workspace in one fixed array inside the library image, so
 * the caller passes only inputs and outputs.
 *
 * The array is part of every process image that loads the library: each GPU
 * the process touches holds kStaticScratchBytes of it until the process exits.
 */
namespace {

constexpr int kStaticUnitHeads = 4096;  // largest kv_heads * units served
constexpr int kStaticUnits = 4096;      // largest units served
constexpr size_t kStaticOpartBytes = (size_t)kStaticUnitHeads * 8 * 128 * sizeof(float);
constexpr size_t kStaticMlBytes = (size_t)kStaticUnitHeads * 8 * 2 * sizeof(float);
constexpr size_t kStaticPlanBytes =
    ((2 + 4 * (size_t)kStaticUnits + 2 + kDynWords + 4 * (size_t)kStaticUnits) * sizeof(int32_t) + 255) / 256 * 256;
constexpr size_t kStaticScratchBytes = kStaticOpartBytes + kStaticMlBytes + kStaticPlanBytes;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not
// a device address and must never be passed to a kernel as one.
static __device__ __align__(256) uint8_t g_decode_scratch[kStaticScratchBytes];

// Device address of g_decode_scratch on the current device, looked up once per
// device (with that device current) and cached.
int static_scratch(uint8_t** base) {
  static std::atomic<uint8_t*> cached[64];
  int dev = 0;
  if (int rc = cuda_status(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return fail(FP_ERR_ARGUMENT, "device index %d not supported", dev);
  uint8_t* known = cached[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    void* ptr = nullptr;
    if (int rc = cuda_status(cudaGetSymbolAddress(&ptr, g_decode_scratch),
                             "cudaGetSymbolAddress(g_decode_scratch)"))
      return rc;
    if (ptr == nullptr) return fail(FP_ERR_CUDA, "static decode scratch has no device address");
    known = static_cast<uint8_t*>(ptr);
    cached[dev].store(known, std::memory_order_release);
  }
  *base = known;
  return FP_OK;
}

}  // namespace

int fp_fused_decode_noalloc(const void* q, int64_t q_stride, const int64_t* rec_addr,
                            const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* seq_lens, void* out, int64_t out_stride, int32_t batch,
                            int32_t kv_heads, int32_t group, int32_t units, int32_t replan,
                            float scale, int32_t num_sms, void* stream) {
  if (batch == 0) return FP_OK;
  FP_REQUIRE(kv_heads > 0 && units > 0, "bad kv_heads %d / units %d", kv_heads, units);
  FP_REQUIRE(units <= kStaticUnits && (int64_t)kv_heads * units <= kStaticUnitHeads,
             "the built-in decode scratch serves kv_heads * units <= %d and units <= %d; got "
             "kv_heads %d, units %d (pass fewer units, or use fp_fused_decode with a workspace)",
             kStaticUnitHeads, kStaticUnits, kv_heads, units);
  uint8_t* base = nullptr;
  if (int rc = static_scratch(&base)) return rc;
  float* opart = reinterpret_cast<float*>(base);
  float* ml = reinterpret_cast<float*>(base + kStaticOpartBytes);
  int32_t* plan = reinterpret_cast<int32_t*>(base + kStaticOpartBytes + kStaticMlBytes);
  // Nothing in the scratch has to start at zero: the planner rewrites the plan
  // and its status word whenever `replan` is set, and every partial result is
  // written by the attention kernel before the merge reads it.
  return fp_fused_decode(q, q_stride, rec_addr, rec_len, plut, slut, block_table, bt_stride,
                         seq_lens, opart, (int64_t)(kStaticOpartBytes / sizeof(float)), ml,
                         (int64_t)(kStaticMlBytes / sizeof(float)), plan, plan_words(units), out,
                         out_stride, batch, kv_heads, group, units, replan, scale, num_sms, stream);
}

}  // extern "C"
