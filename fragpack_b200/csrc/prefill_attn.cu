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
//   O += P V       A = P tile [128 rows, 128 tokens], B = V tile [128 dims, 128 tokens]
//
// All four tiles are K-major with the 128-byte swizzle (eight 16-byte chunks
// of a row XOR-ed with the row index modulo 8), which is also what stmatrix
// can write from the record decoder's mma fragments: a K record yields rows =
// tokens, a V record rows = dims, with the same store.  The two S tiles live in
// tensor memory columns 0..255, the two O tiles in columns 256..511; each
// warpgroup (four warps) owns one query tile and reads its S with tcgen05.ld,
// one thread per query row (no shuffles in the softmax), writes P as BF16 into
// its operand tile, and rescales its O in tensor memory when a row's maximum
// rose.  P is rounded to BF16 and the denominator sums the unrounded
// values, as in decode attention.
//
// This first version runs its phases one after another (decode K, S product,
// decode V beside it, softmax, O product); every wait is bounded and reports
// through the status word.  Nothing here uses thread-block clusters or
// multicast.
#include <math.h>

#include "fp_api.h"
#include "fp_common.cuh"
#include "fp_pipe.cuh"

namespace fpb {
namespace {

constexpr int kPrefillThreads = 256;  // eight warps decode; each warpgroup runs one tile's softmax
constexpr int kTile = 128;
constexpr int kQTiles = 2;                     // query tiles per CTA, one per warpgroup
constexpr int kTileBytes = kTile * kTile * 2;  // 32 KB: one operand tile
constexpr int kHalfTile = kTileBytes / 2;      // one 64-column (128-byte) swizzle atom column
constexpr uint32_t kTmemColumns = 512;         // S tiles: 0..255, O tiles: 256..511

struct PrefillSmem {
  __align__(1024) uint8_t q[kQTiles][kTileBytes];
  __align__(1024) uint8_t k[kTileBytes];
  __align__(1024) uint8_t v[kTileBytes];
  __align__(1024) uint8_t p[kQTiles][kTileBytes];
  __align__(16) uint8_t esc[kEscBytes];
  __align__(8) uint64_t bar_s;  // S product complete
  __align__(8) uint64_t bar_o;  // O product complete
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
// that stale bytes there cannot meet a zero probability as NaN.
__device__ __forceinline__ void record_to_tile(const uint8_t* rec, int vlen, const HeadTables& tab,
                                               uint8_t* tile, uint8_t* esc, int tid,
                                               const PipeConsts& k, int valid_cols) {
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
  if (vlen > kVarCap || vlen < kHeaderBytes)
    raw_record_words(rec, tid, emit);
  else
    coded_record_words<true>(rec, vlen, tab, esc, tid, k, [] {}, emit);
}

__global__ void __launch_bounds__(kPrefillThreads, 1) prefill_attn_kernel(PrefillParams p) {
  // The operand tiles must start on 1024-byte boundaries (the swizzle is a
  // function of the address); the launch reserves the slack for this.
  extern __shared__ uint8_t dyn[];
  PrefillSmem& sm =
      *reinterpret_cast<PrefillSmem*>(dyn + ((1024u - (smem_addr(dyn) & 1023u)) & 1023u));
  const int tid = threadIdx.x, warp = tid >> 5;
  const int req = blockIdx.z, head = blockIdx.y;
  const int rows_tokens = kTile / p.group;  // query tokens per tile
  const int q0 = p.q_start[req], n_q = p.q_start[req + 1] - q0;
  const int cta_tok0 = blockIdx.x * kQTiles * rows_tokens;
  if (cta_tok0 >= n_q) return;  // uniform over the CTA, before anything is allocated
  const int ctx = p.ctx_len[req];
  const int first_pos = ctx - n_q;  // position of the request's first query token
  // Last page each query tile needs (-1: the tile lies past the request's
  // queries); the CTA walks the pages of its last tile.
  int tile_last[kQTiles];
#pragma unroll
  for (int t = 0; t < kQTiles; ++t) {
    const int t0 = cta_tok0 + t * rows_tokens;
    tile_last[t] = t0 < n_q ? (first_pos + min(t0 + rows_tokens, n_q) - 1) >> 7 : -1;
  }
  const int last_page = max(tile_last[0], tile_last[kQTiles - 1]);

  if (tid == 0) {
    mbar_init(&sm.bar_s, 1);
    mbar_init(&sm.bar_o, 1);
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
    const int tok = cta_tok0 + t * rows_tokens + row / p.group, g = row % p.group;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (tok < n_q)
      val = *reinterpret_cast<const uint4*>(p.q + (int64_t)(q0 + tok) * p.q_stride +
                                            (int64_t)(head * p.group + g) * 128 + col);
    *reinterpret_cast<uint4*>(sm.q[t] + tile_chunk(row, col)) = val;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;
  const HeadTables tab_k = load_tables(p.plut, p.slut, head);
  const HeadTables tab_v = load_tables(p.plut, p.slut, p.kvh + head);
  const int32_t* bt = p.block_table + (int64_t)req * p.bt_stride;

  // Softmax state of this thread's query row: warpgroup `mine` owns query tile
  // `mine`, thread = row.  Key positions <= row_pos are visible (rows past the
  // request's queries compute like its last token and are not stored).
  const int mine = warp >> 2, row = tid & (kTile - 1);
  const int tok0 = cta_tok0 + mine * rows_tokens;
  const int my_last = mine == 0 ? tile_last[0] : tile_last[kQTiles - 1];
  const int row_pos = min(first_pos + tok0 + row / p.group, ctx - 1);
  float row_max = -INFINITY, row_sum = 0.f;
  const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;  // this warp's tensor-memory lanes
  const uint32_t tmem_s = tmem + (uint32_t)(mine * kTile);
  const uint32_t tmem_o = tmem + (uint32_t)((kQTiles + mine) * kTile);
  uint8_t* p_tile = sm.p[mine];

  for (int page = 0; page <= last_page; ++page) {
    const uint32_t parity = (uint32_t)page & 1u;
    const int64_t idx = (int64_t)bt[page] * 2 * p.kvh + head;
    const int open_cols = ctx - page * kTile;  // tokens of this block that exist
    if (tid < 2 && page < last_page) {
      // The records are decoded straight from global memory: ask the L2 for the
      // next page's K (thread 0) and V (thread 1) record while this page is worked on.
      const int64_t next = (int64_t)bt[page + 1] * 2 * p.kvh + head + tid * p.kvh;
      const int32_t n = p.rec_len[next];
      prefetch_l2(reinterpret_cast<const void*>(p.rec_addr[next]),
                  n > kVarCap || n < kHeaderBytes ? (uint32_t)kRawRecord
                                                  : (uint32_t)(kDenseBytes + (n & ~15)));
    }
    // ---- K record -> K tile (its previous readers, the S products of the page
    // before, finished before that page's softmax began).
    record_to_tile(reinterpret_cast<const uint8_t*>(p.rec_addr[idx]), p.rec_len[idx], tab_k, sm.k,
                   sm.esc, tid, p.k, kTile);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int t = 0; t < kQTiles; ++t)
        if (page <= tile_last[t])
          tile_product(tmem + (uint32_t)(t * kTile), smem_addr(sm.q[t]), smem_addr(sm.k), false);
      umma_commit(&sm.bar_s);
    }
    // ---- V record -> V tile while the S products run; the O products of the
    // page before must be done with the V and P tiles (and with O) first.
    if (page > 0) bounded_wait(&sm.bar_o, parity ^ 1u, &sm.wait);
    record_to_tile(reinterpret_cast<const uint8_t*>(p.rec_addr[idx + p.kvh]),
                   p.rec_len[idx + p.kvh], tab_v, sm.v, sm.esc, tid, p.k, open_cols);
    // ---- softmax: one thread per query row of the warpgroup's tile (a tile
    // whose queries all lie before this page has nothing to add).
    if (page <= my_last) {
      bounded_wait(&sm.bar_s, parity, &sm.wait);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int visible = row_pos - page * kTile;  // columns 0..visible of this page count
      float page_max = -INFINITY;
      uint32_t s[32];
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        tmem_load32(tmem_s + lane_base + (uint32_t)c0, s);
#pragma unroll
        for (int x = 0; x < 32; ++x)
          if (c0 + x <= visible) page_max = fmaxf(page_max, __uint_as_float(s[x]) * p.scale_log2);
      }
      const float new_max = fmaxf(row_max, page_max);
      // A row that sees no key yet keeps -inf; use 0 as its reference point.
      const float ref = new_max == -INFINITY ? 0.f : new_max;
      const float keep = ex2(row_max - ref);  // 0 while row_max is still -inf
      // O rows are rescaled in tensor memory when some row of the warp's 32 rose.
      if (page > 0 && __any_sync(0xffffffffu, new_max > row_max)) {
#pragma unroll 1
        for (int c0 = 0; c0 < kTile; c0 += 32) {
          tmem_load32(tmem_o + lane_base + (uint32_t)c0, s);
#pragma unroll
          for (int x = 0; x < 32; ++x) s[x] = __float_as_uint(__uint_as_float(s[x]) * keep);
          tmem_store32(tmem_o + lane_base + (uint32_t)c0, s);
        }
      }
      row_sum *= keep;
      row_max = new_max;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        tmem_load32(tmem_s + lane_base + (uint32_t)c0, s);
        uint32_t packed[16];
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float a = c0 + x <= visible ? ex2(__uint_as_float(s[x]) * p.scale_log2 - ref) : 0.f;
          const float b =
              c0 + x + 1 <= visible ? ex2(__uint_as_float(s[x + 1]) * p.scale_log2 - ref) : 0.f;
          row_sum += a + b;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
          packed[x >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(p_tile + tile_chunk(row, c0 + 8 * ch)) =
              make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();  // V and P tiles complete, S read, O rescaled
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int t = 0; t < kQTiles; ++t)
        if (page <= tile_last[t])
          tile_product(tmem + (uint32_t)((kQTiles + t) * kTile), smem_addr(sm.p[t]), smem_addr(sm.v),
                       page > 0);
      umma_commit(&sm.bar_o);
    }
  }

  // ---- epilogue: O / row_sum -> BF16 rows of `out`.
  if (my_last >= 0) {
    bounded_wait(&sm.bar_o, (uint32_t)last_page & 1u, &sm.wait);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int tok = tok0 + row / p.group, g = row % p.group;
    const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
    __nv_bfloat16* dst =
        p.out + (int64_t)(q0 + tok) * p.out_stride + (int64_t)(head * p.group + g) * 128;
    uint32_t o[32];
#pragma unroll 1
    for (int c0 = 0; c0 < kTile; c0 += 32) {
      tmem_load32(tmem_o + lane_base + (uint32_t)c0, o);
      if (tok < n_q) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const __nv_bfloat162 pair =
                __floats2bfloat162_rn(__uint_as_float(o[8 * ch + 2 * x]) * inv,
                                      __uint_as_float(o[8 * ch + 2 * x + 1]) * inv);
            w[x] = *reinterpret_cast<const uint32_t*>(&pair);
          }
          *reinterpret_cast<uint4*>(dst + c0 + 8 * ch) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
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
  const int cta_tokens = kQTiles * (kTile / group);  // query tokens per CTA
  const dim3 grid((unsigned)((max_query_tokens + cta_tokens - 1) / cta_tokens), (unsigned)kv_heads,
                  (unsigned)num_requests);
  prefill_attn_kernel<<<grid, kPrefillThreads, smem, (cudaStream_t)stream>>>(p);
  FP_LAUNCH_CHECK("prefill_attn_kernel");
  return FP_OK;
}

}  // extern "C"
