// Causal prefill attention directly over compressed KV records, for sm_100a.
//
// The reference's prefill path first decompresses a request's cached blocks
// into a BF16 workspace and then runs FlashAttention over it
// (fragpack/integrations/vllm/backend.py:560-575: store.gather, then
// flash_attn_varlen_func with causal=True and a paged workspace).  This kernel
// does both in one pass and never writes the decompressed KV to HBM: a CTA
// takes two tiles of 128 query rows (128 / G tokens x the G query heads of one
// KV head each; a decoded record serves both), walks the request's pages,
// decodes each K and V record straight into shared-memory tiles laid out as
// tensor-core operands, and runs both products on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in tensor memory), per query tile:
//
//   S = Q K^T      A = Q tile [128 rows, 128 dims], B = K tile [128 tokens, 128 dims]
//   O += P V       A = P [128 rows, 128 tokens] in tensor memory, B = V tile [128 dims, 128 tokens]
//
// The three shared-memory tiles are K-major with the 128-byte swizzle (eight 16-byte chunks
// of a row XOR-ed with the row index modulo 8), which is also what stmatrix
// can write from the record decoder's mma fragments: a K record yields rows =
// tokens, a V record rows = dims, with the same store.  The two S tiles live in
// tensor memory columns 0..255, the two O tiles in columns 256..511; each
// warpgroup (four warps) owns one query tile and reads its S with tcgen05.ld,
// one thread per query row (no shuffles in the softmax), writes P as BF16 over
// the first half of its S columns (two values per 32-bit cell: the A operand of
// the O product is read from tensor memory), and rescales its O in tensor
// memory when a row's maximum rose.  P is rounded to BF16 and the denominator sums the unrounded
// values, as in decode attention.
//
// The CTA is specialised by warp, and the phases of successive pages overlap:
//   warps 0-7   decode K records (the decoder's 256 owners): K of page p + 1 as
//               soon as the S products of page p have read the K tile;
//   warps 8-15  decode V records, side by side with the K team: V of page p + 1
//               as soon as the O products of page p have read the V tile;
//   warps 16-19 softmax of query tile 0, warps 20-23 of query tile 1 (a warp
//               reaches the tensor-memory lanes 32 (warp % 4) ..), running while
//               the next page's records are decoded;
//   warp 24     one lane issues every tcgen05.mma: O_t(p) and then S_t(p + 1) as
//               soon as tile t's probabilities of page p are written (in this
//               order, so that S_t(p + 1) overwrites P_t(p) after it was used);
//   warp 25     streams the coded records into the two teams' slots of shared
//               memory with bulk copies, 32 table look-ups at a time (raw
//               records, the open tails, are read in place).
// They meet only through mbarriers (ring slot full / empty, K / V tile written,
// K / V tile read, S_t ready, O_t done, P_t written); every wait is bounded and reports through the
// status word.  Nothing here uses thread-block clusters or multicast.
#include <math.h>

#include "fp_api.h"
#include "fp_common.cuh"
#include "fp_pipe.cuh"

namespace fpb {
namespace {

constexpr int kTeamThreads = 256;  // one decoder team: the record decoder's 256 owners
constexpr int kDecoderThreads = 2 * kTeamThreads;  // warps 0-7 decode K records, warps 8-15 V records
constexpr int kSoftmaxThreads = 256;  // warps 16-23: one warpgroup per query tile, thread = row
constexpr int kIssuerThread = kDecoderThreads + kSoftmaxThreads;  // lane 0 of warp 24
constexpr int kProducerWarp = 25;
constexpr int kPrefillThreads = kDecoderThreads + kSoftmaxThreads + 64;
constexpr int kRingSlots = 2;  // records alternate K, V: slot 0 serves the K team, slot 1 the V team
// How far (log2 units) a row's maximum may rise above the reference point of
// its exponentials before the reference follows.  0: the reference is the
// running maximum, as in decode attention.  A lag would spare most rescales
// of O (6 % of the kernel's time at 8), but the error against fp32 attention
// grew with it in measurement (mean-abs 1.84e-4 at 0, 1.93e-4 at 1, 2.18e-4
// at 8; max-abs 0.0045, 0.0056, 0.0084), so it is not used.
constexpr float kRescaleSlack = 0.f;
constexpr int kTile = 128;
constexpr int kQTiles = 2;                     // query tiles per CTA, one per warpgroup
constexpr int kTileBytes = kTile * kTile * 2;  // 32 KB: one operand tile
constexpr int kHalfTile = kTileBytes / 2;      // one 64-column (128-byte) swizzle atom column
constexpr uint32_t kTmemColumns = 512;         // S tiles: 0..255, O tiles: 256..511

struct PrefillSmem {
  __align__(1024) uint8_t q[kQTiles][kTileBytes];
  __align__(1024) uint8_t k[kTileBytes];
  __align__(1024) uint8_t v[kTileBytes];
  __align__(128) uint8_t ring[kRingSlots][kCodedMax];  // coded records, as stored
  __align__(16) uint8_t esc[2][kEscBytes];  // escape scratch of the K team and of the V team
  int64_t addr[kRingSlots];  // where the slot's record lives (raw records are read there)
  int32_t vlen[kRingSlots];
  // Phase p of every barrier belongs to page p.
  __align__(8) uint64_t k_ready, v_ready;      // decoder team (256 arrivals): tile written
  uint64_t k_free, v_free;                     // products that read the tile are complete
  uint64_t s_ready[kQTiles], o_done[kQTiles];  // tile t's S / O products are complete
  uint64_t p_ready[kQTiles];                   // tile t's softmax threads (128 arrivals): P written, S read
  uint64_t drained;                            // every product issued by this CTA is complete
  uint64_t full[kRingSlots], empty[kRingSlots];  // ring: copy landed / the team's 8 warps are done
  uint32_t tmem_base;
  WaitState wait;
};

struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int64_t* rec_addr;
  const int32_t* rec_len;
  const int32_t* plut;
  const uint8_t* slut;
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* ctx_len;
  int32_t* status;
  int64_t q_stride, out_stride, bt_stride;
  int kvh, group;
  float scale_log2;
  PipeConsts k;
  long long wait_limit;
  int skip_page;  // test hook: the decoders do not report this page's K tile (-1: none)
};

// Byte offset of the 16-byte chunk holding (row, col .. col + 7) of a K-major
// 128 x 128 BF16 operand tile with the 128-byte swizzle: two column halves of
// 64 elements, each a stack of 8-row groups of 1024 bytes.
__device__ __forceinline__ uint32_t tile_chunk(int row, int col) {
  return (uint32_t)((col >> 6) * kHalfTile + (row >> 3) * 1024 + (row & 7) * 128 +
                    ((((col & 63) >> 3) ^ (row & 7)) << 4));
}

// Shared-memory matrix descriptor of an operand tile starting at `addr`
// (K-major, 128-byte swizzle: 8-row groups 1024 bytes apart).
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: BF16 x BF16 -> FP32, both operands K-major, M = N = 128.
constexpr uint32_t kInstrDesc =
    (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTile >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"((uint32_t)accumulate)
      : "memory");
}

// The same with the A operand in tensor memory: 128 rows on the 128 lanes, two
// BF16 values per 32-bit column, so a K = 16 step spans eight columns.
__device__ __forceinline__ void umma_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(kInstrDesc), "r"((uint32_t)accumulate)
      : "memory");
}

// D (+)= A B over the tiles' 128-deep contraction: eight K = 16 steps, each
// 32 bytes further along the row (four per swizzle atom column).
__device__ __forceinline__ void tile_product(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr,
                                             bool accumulate) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t step = (uint32_t)((j >> 2) * kHalfTile + (j & 3) * 32);
    umma(d_tmem, tile_desc(a_addr + step), tile_desc(b_addr + step), accumulate || j > 0);
  }
}

__device__ __forceinline__ void tile_product_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr,
                                                    bool accumulate) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t step = (uint32_t)((j >> 2) * kHalfTile + (j & 3) * 32);
    umma_tmem_a(d_tmem, a_tmem + 8u * (uint32_t)j, tile_desc(b_addr + step), accumulate || j > 0);
  }
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_addr(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// The same load without the wait: the caller overlaps it with arithmetic on
// an earlier chunk and calls tmem_wait_loads() before it reads `r`.
__device__ __forceinline__ void tmem_load32_async(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_loads() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_stores() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n\t"
      "tcgen05.wait::st.sync.aligned;"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// No wait inside: the caller calls tmem_wait_stores() once after its last store.
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Decodes one record into an operand tile.  Owner (w, g, c) holds, for word
// st, the four 8 x 8 pieces (j, f) of rows 16 w + 8 j + 0..7 and columns
// 16 st + 8 f + 0..7: for a K record rows are tokens and columns dims, for a V
// record rows are dims and columns tokens - in both cases the tile's row is
// the fragment's row, so one stmatrix per word stores all four pieces; lane
// 8 m + r supplies the address of row r of piece m = 2 j + f.  `valid_cols`
// clears the columns (tokens of a V record) past the end of an open block, so
// that stale bytes there cannot meet a zero probability as NaN.  A coded
// record is read from its ring slot `staged`, a raw one in place; `released`
// is called once the slot is no longer needed.
template <typename Released>
__device__ __forceinline__ void record_to_tile(const uint8_t* staged, int64_t in_place, int vlen,
                                               const HeadTables& tab, uint8_t* tile, uint8_t* esc,
                                               int tid, const PipeConsts& k, int valid_cols,
                                               Released&& released) {
  const int lane = tid & 31, warp = tid >> 5;
  const int r = lane & 7, j = (lane >> 4) & 1, f = (lane >> 3) & 1, c = lane & 3;
  const uint32_t base = smem_addr(tile);
  auto emit = [&](int st, const uint32_t (&w)[4]) {
    uint32_t a[4] = {w[0], w[1], w[2], w[3]};
    if (valid_cols < kTile) {
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int col = 16 * st + 8 * (x & 1) + 2 * c;
        if (col >= valid_cols) a[x] = 0u;
        else if (col + 1 >= valid_cols) a[x] &= 0xffffu;
      }
    }
    const uint32_t at = base + tile_chunk(16 * warp + 8 * j + r, 16 * st + 8 * f);
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(at),
                 "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3])
                 : "memory");
  };
  if (vlen > kVarCap || vlen < kHeaderBytes) {
    released();
    raw_record_words(reinterpret_cast<const uint8_t*>(in_place), tid, emit);
  } else {
    // Low bytes up front, so that the slot is free for the next record's copy
    // while this one is still being assembled.
    coded_record_words<true>(staged, vlen, tab, esc, tid, k, released, emit);
  }
}

// What every role needs to know about the CTA's work.
struct PrefillWork {
  int req, head, q0, n_q, ctx, first_pos, cta_tok0, rows_tokens;
  int tile_last[kQTiles];  // last page query tile t needs; -1: the tile has no queries
  int last_page;
};

// Producer warp: the records of the CTA's pages, K then V, into the ring.
// Lane L resolves the L-th of the next 32 records (block table -> record
// address and length), lane 0 then issues them in order.
__device__ __forceinline__ void prefill_produce(const PrefillParams& p, PrefillSmem& sm,
                                                const PrefillWork& w, int lane) {
  const int32_t* bt = p.block_table + (int64_t)w.req * p.bt_stride;
  const int records = 2 * (w.last_page + 1);
  volatile int* abort = &sm.wait.abort;
  for (int base = 0; base < records; base += 32) {
    const int n = base + lane;
    int64_t addr = 0;
    int32_t vlen = 0;
    if (n < records) {
      const int64_t at = (int64_t)bt[n >> 1] * 2 * p.kvh + w.head + (n & 1) * p.kvh;
      addr = p.rec_addr[at];
      vlen = p.rec_len[at];
    }
    const int count = min(32, records - base);
    for (int j = 0; j < count; ++j) {
      const int64_t a = __shfl_sync(0xffffffffu, addr, j);
      const int32_t v = __shfl_sync(0xffffffffu, vlen, j);
      const uint32_t r = (uint32_t)(base + j), slot = r % kRingSlots, use = r / kRingSlots;
      if (lane == 0) {
        bool ok = true;
        if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1u, &sm.wait);
        if (ok) {
          sm.addr[slot] = a;
          sm.vlen[slot] = v;
          if (v > kVarCap || v < kHeaderBytes) {
            prefetch_l2(reinterpret_cast<const void*>(a), kRawRecord);
            mbar_arrive(&sm.full[slot]);
          } else {
            const uint32_t bytes = (uint32_t)(kDenseBytes + (v & ~15));
            mbar_expect_tx(&sm.full[slot], bytes);
            bulk_load(sm.ring[slot], reinterpret_cast<const void*>(a), bytes, &sm.full[slot]);
          }
        }
      }
      __syncwarp();
      if (*abort) return;
    }
  }
}

// A decoder team (kv = 0: K records, 1: V records; `tid` within the team):
// its record of every page out of its ring slot into its operand tile.  The two
// teams run side by side, so a page costs one record's decode time, not two.
__device__ __forceinline__ void prefill_decode(const PrefillParams& p, PrefillSmem& sm,
                                               const PrefillWork& w, int kv, int tid) {
  const HeadTables tab = load_tables(p.plut, p.slut, kv * p.kvh + w.head);
  const int lane = tid & 31;
  uint64_t* const full = &sm.full[kv];
  uint64_t* const tile_free = kv == 0 ? &sm.k_free : &sm.v_free;
  uint64_t* const tile_ready = kv == 0 ? &sm.k_ready : &sm.v_ready;
  uint8_t* const tile = kv == 0 ? sm.k : sm.v;
  const auto released = [&] {
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[kv]);
  };
  for (int page = 0; page <= w.last_page; ++page) {
    // A record whose wait ran out is not decoded (the status word marks the call invalid).
    const bool landed = bounded_wait(full, (uint32_t)page & 1u, &sm.wait);
    // The tile's readers are the S (K tile) / O (V tile) products of the page before.
    if (page > 0) bounded_wait(tile_free, (uint32_t)(page - 1) & 1u, &sm.wait);
    if (landed) {
      // Columns (tokens) of a V tile past the end of an open block are cleared.
      record_to_tile(sm.ring[kv], sm.addr[kv], sm.vlen[kv], tab, tile, sm.esc[kv], tid, p.k,
                     kv == 0 ? kTile : w.ctx - page * kTile, released);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (kv == 1 || page != p.skip_page) mbar_arrive(tile_ready);
    // The team's escape scratch is reused by its next record: all owners are done with it.
    if (kv == 0)
      asm volatile("bar.sync 1, %0;" ::"n"(kTeamThreads) : "memory");
    else
      asm volatile("bar.sync 2, %0;" ::"n"(kTeamThreads) : "memory");
  }
}

// The thread that issues the products.  Order: S_t(0); then per page p and
// tile t: O_t(p), S_t(p + 1) - the tensor pipe runs them in this order, so the
// next page's scores are not held up behind the other tile's O product for
// longer than one product.
__device__ __forceinline__ void prefill_issue(PrefillSmem& sm, const PrefillWork& w, uint32_t tmem) {
  const uint32_t q_addr[kQTiles] = {smem_addr(sm.q[0]), smem_addr(sm.q[1])};
  const uint32_t k_addr = smem_addr(sm.k), v_addr = smem_addr(sm.v);
  const auto last_tile = [&](int page) { return page <= w.tile_last[kQTiles - 1] ? kQTiles - 1 : 0; };
  bounded_wait(&sm.k_ready, 0u, &sm.wait);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
  for (int t = 0; t < kQTiles; ++t)
    if (0 <= w.tile_last[t]) {
      tile_product(tmem + (uint32_t)(t * kTile), q_addr[t], k_addr, false);
      umma_commit(&sm.s_ready[t]);
    }
  umma_commit(&sm.k_free);
  for (int page = 0; page <= w.last_page; ++page) {
    const uint32_t parity = (uint32_t)page & 1u;
    bool v_seen = false, k_seen = false;
#pragma unroll
    for (int t = 0; t < kQTiles; ++t) {
      if (page <= w.tile_last[t]) {
        bounded_wait(&sm.p_ready[t], parity, &sm.wait);
        if (!v_seen) bounded_wait(&sm.v_ready, parity, &sm.wait);
        v_seen = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // P_t sits in the first half of S_t's columns.
        tile_product_tmem_a(tmem + (uint32_t)((kQTiles + t) * kTile), tmem + (uint32_t)(t * kTile),
                            v_addr, page > 0);
        umma_commit(&sm.o_done[t]);
        if (t == last_tile(page)) umma_commit(&sm.v_free);
      }
      if (page + 1 <= w.tile_last[t]) {
        if (!k_seen) bounded_wait(&sm.k_ready, parity ^ 1u, &sm.wait);
        k_seen = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tile_product(tmem + (uint32_t)(t * kTile), q_addr[t], k_addr, false);
        umma_commit(&sm.s_ready[t]);
        if (t == last_tile(page + 1)) umma_commit(&sm.k_free);
      }
    }
  }
  // Tensor memory is given back at the end of the kernel: nothing may still be
  // running there, also when a wait above gave up and the roles ran ahead.
  umma_commit(&sm.drained);
#pragma unroll 1
  for (int tries = 0; tries < (1 << 20); ++tries)
    if (mbar_try(&sm.drained, 0u, 1000u)) break;
}

// Largest of 32 raw scores, columns first .. first + 31 of the page; kMasked:
// only the columns up to `visible` count.
template <bool kMasked>
__device__ __forceinline__ float chunk_max(const uint32_t (&s)[32], int first, int visible, float m) {
#pragma unroll
  for (int x = 0; x < 32; x += 2) {
    float a = __uint_as_float(s[x]), b = __uint_as_float(s[x + 1]);
    if (kMasked && first + x > visible) a = -INFINITY;
    if (kMasked && first + x + 1 > visible) b = -INFINITY;
    m = fmaxf(m, fmaxf(a, b));
  }
  return m;
}

// exp2(score * scale - ref) of 32 scores as 16 BF16 pairs; returns their sum
// (of the unrounded values).
template <bool kMasked>
__device__ __forceinline__ float chunk_probabilities(const uint32_t (&s)[32], int first, int visible,
                                                     float scale, float ref,
                                                     uint32_t (&packed)[16]) {
  float sum = 0.f;
#pragma unroll
  for (int x = 0; x < 32; x += 2) {
    float a = ex2(fmaf(__uint_as_float(s[x]), scale, -ref));
    float b = ex2(fmaf(__uint_as_float(s[x + 1]), scale, -ref));
    if (kMasked && first + x > visible) a = 0.f;
    if (kMasked && first + x + 1 > visible) b = 0.f;
    sum += a + b;
    const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
    packed[x >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
  }
  return sum;
}

// Softmax warpgroup of query tile `mine`: thread = query row.
__device__ __forceinline__ void prefill_softmax(const PrefillParams& p, PrefillSmem& sm,
                                                const PrefillWork& w, uint32_t tmem, int mine,
                                                int row, int warp) {
  const int my_last = w.tile_last[mine];
  if (my_last < 0) return;
  const int tok0 = w.cta_tok0 + mine * w.rows_tokens;
  // Key positions <= row_pos are visible (rows past the request's queries
  // compute like its last token and are not stored).
  const int row_pos = min(w.first_pos + tok0 + row / p.group, w.ctx - 1);
  float row_max = -INFINITY, row_sum = 0.f;
  const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;  // this warp's tensor-memory lanes
  const uint32_t tmem_s = tmem + (uint32_t)(mine * kTile);
  const uint32_t tmem_o = tmem + (uint32_t)((kQTiles + mine) * kTile);
  uint32_t s[32], s2[32];
  for (int page = 0; page <= my_last; ++page) {
    const uint32_t parity = (uint32_t)page & 1u;
    bounded_wait(&sm.s_ready[mine], parity, &sm.wait);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int visible = row_pos - page * kTile;  // columns 0..visible of this page count
    // Only the pages on the diagonal need the causal mask (uniform over the warp).
    const bool masked = __any_sync(0xffffffffu, visible < kTile - 1);
    // Two chunks of 32 scores in flight: the load of the next overlaps the
    // arithmetic on this one.  The scale is positive, so the largest raw score
    // gives the largest scaled one.
    float raw_max = -INFINITY;
    tmem_load32_async(tmem_s + lane_base, s);
    tmem_wait_loads();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t(&cur)[32] = (c & 1) ? s2 : s;
      uint32_t(&nxt)[32] = (c & 1) ? s : s2;
      if (c < 3) tmem_load32_async(tmem_s + lane_base + (uint32_t)(32 * (c + 1)), nxt);
      raw_max = masked ? chunk_max<true>(cur, 32 * c, visible, raw_max)
                       : chunk_max<false>(cur, 32 * c, visible, raw_max);
      tmem_wait_loads();
    }
    const float page_max = raw_max * p.scale_log2;
    // The reference point of the exponentials follows the running maximum
    // (kRescaleSlack = 0; see there).
    const bool rise = page_max > row_max + kRescaleSlack;  // row_max is -inf until a key is seen
    const float new_max = rise ? page_max : row_max;
    // A row that sees no key yet keeps -inf; use 0 as its reference point.
    const float ref = new_max == -INFINITY ? 0.f : new_max;
    const float keep = rise ? ex2(row_max - ref) : 1.f;  // 0 while row_max is still -inf
    // The O product of the page before writes O (and read P, which the S
    // product of this page has since overwritten).
    if (page > 0) {
      bounded_wait(&sm.o_done[mine], parity ^ 1u, &sm.wait);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (__any_sync(0xffffffffu, rise)) {
#pragma unroll 1
        for (int c0 = 0; c0 < kTile; c0 += 32) {
          tmem_load32(tmem_o + lane_base + (uint32_t)c0, s);
#pragma unroll
          for (int x = 0; x < 32; ++x) s[x] = __float_as_uint(__uint_as_float(s[x]) * keep);
          tmem_store32(tmem_o + lane_base + (uint32_t)c0, s);
        }
      }
    }
    row_sum *= keep;
    row_max = new_max;
    // P over the S columns already read: chunk c of 32 scores becomes 16 cells
    // at columns 16 c .., always behind the read position.
    tmem_load32_async(tmem_s + lane_base, s);
    tmem_wait_loads();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t(&cur)[32] = (c & 1) ? s2 : s;
      uint32_t(&nxt)[32] = (c & 1) ? s : s2;
      if (c < 3) tmem_load32_async(tmem_s + lane_base + (uint32_t)(32 * (c + 1)), nxt);
      uint32_t packed[16];
      row_sum += masked ? chunk_probabilities<true>(cur, 32 * c, visible, p.scale_log2, ref, packed)
                        : chunk_probabilities<false>(cur, 32 * c, visible, p.scale_log2, ref, packed);
      tmem_wait_loads();
      tmem_store16(tmem_s + lane_base + (uint32_t)(16 * c), packed);
    }
    tmem_wait_stores();
    // P written, S read, O rescaled: the issuing thread may go on.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    mbar_arrive(&sm.p_ready[mine]);
  }

  // ---- epilogue: O / row_sum -> BF16 rows of `out`.
  bounded_wait(&sm.o_done[mine], (uint32_t)my_last & 1u, &sm.wait);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int tok = tok0 + row / p.group, g = row % p.group;
  const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
  __nv_bfloat16* dst =
      p.out + (int64_t)(w.q0 + tok) * p.out_stride + (int64_t)(w.head * p.group + g) * 128;
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    tmem_load32(tmem_o + lane_base + (uint32_t)c0, s);
    if (tok < w.n_q) {
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const __nv_bfloat162 pair =
              __floats2bfloat162_rn(__uint_as_float(s[8 * ch + 2 * x]) * inv,
                                    __uint_as_float(s[8 * ch + 2 * x + 1]) * inv);
          o[x] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(dst + c0 + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__global__ void __launch_bounds__(kPrefillThreads, 1) prefill_attn_kernel(PrefillParams p) {
  // The operand tiles must start on 1024-byte boundaries (the swizzle is a
  // function of the address); the launch reserves the slack for this.
  extern __shared__ uint8_t dyn[];
  PrefillSmem& sm =
      *reinterpret_cast<PrefillSmem*>(dyn + ((1024u - (smem_addr(dyn) & 1023u)) & 1023u));
  const int tid = threadIdx.x, warp = tid >> 5;
  PrefillWork w;
  w.req = blockIdx.z;
  w.head = blockIdx.y;
  w.rows_tokens = kTile / p.group;  // query tokens per tile
  w.q0 = p.q_start[w.req];
  w.n_q = p.q_start[w.req + 1] - w.q0;
  w.cta_tok0 = blockIdx.x * kQTiles * w.rows_tokens;
  if (w.cta_tok0 >= w.n_q) return;  // uniform over the CTA, before anything is allocated
  w.ctx = p.ctx_len[w.req];
  w.first_pos = w.ctx - w.n_q;  // position of the request's first query token
#pragma unroll
  for (int t = 0; t < kQTiles; ++t) {
    const int t0 = w.cta_tok0 + t * w.rows_tokens;
    w.tile_last[t] = t0 < w.n_q ? (w.first_pos + min(t0 + w.rows_tokens, w.n_q) - 1) >> 7 : -1;
  }
  w.last_page = max(w.tile_last[0], w.tile_last[kQTiles - 1]);

  if (tid == 0) {
    mbar_init(&sm.k_ready, kTeamThreads);
    mbar_init(&sm.v_ready, kTeamThreads);
    mbar_init(&sm.k_free, 1);
    mbar_init(&sm.v_free, 1);
    mbar_init(&sm.drained, 1);
#pragma unroll
    for (int i = 0; i < kRingSlots; ++i) {
      mbar_init(&sm.full[i], 1);
      mbar_init(&sm.empty[i], kTeamThreads / 32);
    }
#pragma unroll
    for (int t = 0; t < kQTiles; ++t) {
      mbar_init(&sm.s_ready[t], 1);
      mbar_init(&sm.o_done[t], 1);
      mbar_init(&sm.p_ready[t], kSoftmaxThreads / kQTiles);
    }
    sm.wait.abort = 0;
    sm.wait.status = p.status;
    sm.wait.limit = p.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_addr(&sm.tmem_base)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Q tiles: row = token * G + head of the group, zero rows past the request's queries.
  for (int x = tid; x < kQTiles * kTile * 16; x += kPrefillThreads) {
    const int t = x / (kTile * 16), row = (x >> 4) & (kTile - 1), col = (x & 15) * 8;
    const int tok = w.cta_tok0 + t * w.rows_tokens + row / p.group, g = row % p.group;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (tok < w.n_q)
      val = *reinterpret_cast<const uint4*>(p.q + (int64_t)(w.q0 + tok) * p.q_stride +
                                            (int64_t)(w.head * p.group + g) * 128 + col);
    *reinterpret_cast<uint4*>(sm.q[t] + tile_chunk(row, col)) = val;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  if (tid < kDecoderThreads) {
    prefill_decode(p, sm, w, tid / kTeamThreads, tid % kTeamThreads);
  } else if (tid < kDecoderThreads + kSoftmaxThreads) {
    const int row = (tid - kDecoderThreads) & (kTile - 1);
    prefill_softmax(p, sm, w, tmem, (tid - kDecoderThreads) / kTile, row, warp);
  } else if (tid == kIssuerThread) {
    prefill_issue(sm, w, tmem);
  } else if (warp == kProducerWarp) {
    prefill_produce(p, sm, w, tid & 31);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(kTmemColumns)
                 : "memory");
  }
}

}  // namespace
}  // namespace fpb

using namespace fpb;

extern "C" {

int fp_prefill_attention(const void* q, int64_t q_stride, const int64_t* rec_addr,
                         const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                         const int32_t* block_table, int64_t bt_stride, const int32_t* q_start,
                         const int32_t* ctx_len, void* out, int64_t out_stride, int32_t num_requests,
                         int32_t max_query_tokens, int32_t kv_heads, int32_t group, float scale,
                         int32_t* status, void* stream) {
  if (num_requests == 0 || max_query_tokens == 0) return FP_OK;
  FP_REQUIRE(num_requests > 0 && num_requests <= 65535 && max_query_tokens > 0 && kv_heads > 0 &&
                 kv_heads <= 65535,
             "bad prefill geometry (%d requests, %d query tokens, %d KV heads)", num_requests,
             max_query_tokens, kv_heads);
  FP_REQUIRE(scale > 0.f, "the softmax scale must be positive");
  FP_REQUIRE(group == 1 || group == 2 || group == 4 || group == 8,
             "query group %d must be 1, 2, 4 or 8", group);
  FP_REQUIRE(q && rec_addr && rec_len && plut && slut && block_table && q_start && ctx_len && out &&
                 status,
             "null prefill attention argument");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                 q_stride % 8 == 0 && out_stride % 8 == 0,
             "q / out rows must be 16-byte aligned");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(slut) % 16 == 0, "slut must be 16-byte aligned");
  static std::atomic<uint64_t> smem_allowed;
  const int smem = (int)sizeof(PrefillSmem) + 1024;  // room to align the tiles to 1024 bytes
  if (int rc = allow_dynamic_smem(prefill_attn_kernel, smem, smem_allowed)) return rc;
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.rec_addr = rec_addr;
  p.rec_len = rec_len;
  p.plut = plut;
  p.slut = slut;
  p.block_table = block_table;
  p.q_start = q_start;
  p.ctx_len = ctx_len;
  p.status = status;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.bt_stride = bt_stride;
  p.kvh = kv_heads;
  p.group = group;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.k = pipe_consts();
  p.wait_limit = wait_debug().limit;
  p.skip_page = (int)std::max<long long>(-1, std::min<long long>(wait_debug().skip_record, 1 << 20));
  const int cta_tokens = kQTiles * (kTile / group);  // query tokens per CTA
  const dim3 grid((unsigned)((max_query_tokens + cta_tokens - 1) / cta_tokens), (unsigned)kv_heads,
                  (unsigned)num_requests);
  prefill_attn_kernel<<<grid, kPrefillThreads, smem, (cudaStream_t)stream>>>(p);
  FP_LAUNCH_CHECK("prefill_attn_kernel");
  return FP_OK;
}

}  // extern "C"
