// Record constants and the in-register record decoder shared by the decode
// attention kernel, the prefill decompressor and the standalone codec entry
// points.  Record format: fragpack/compression/attn_page.py:1-44 (reference).
//
// A record is 128 tokens x 128 dims of BF16 split over 256 "fragment owners":
// owner t (warp w = t / 32, g = (t / 4) % 8, c = t % 4) holds 64 scalars, as
// eight 8-scalar words.  Word st is one m16n8k16 A fragment (a0, a2, a1, a3):
//   K: token 16 w + 8 j + g,        dim 16 st + 8 f + 2 c + e
//   V: token 16 st + 8 f + 2 c + e, dim 16 w + 8 j + g
// with scalar index s = 8 st + 4 j + 2 f + e inside the owner.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fpb {

constexpr int kOwners = 256;            // fragment owners (threads) per record
constexpr int kLowBytes = 16384;        // one low byte per scalar
constexpr int kSymBytes = 6144;         // 3 bits per scalar
constexpr int kDenseBytes = kLowBytes + kSymBytes;
constexpr int kVarCap = 2048;           // largest variable region of a coded record
constexpr int kCodedMax = kDenseBytes + kVarCap;  // 24576
constexpr int kRawRecord = 32768;
constexpr int kRawVarLen = kRawRecord - kDenseBytes;  // rec_len of a raw record
constexpr int kHeaderBytes = 48;
constexpr int kPrimaryDirect = 7;
constexpr int kTableEntries = 22;
constexpr int kMaxWarpRaw = 32;
// Expanded escapes of one record.  Escape ordinal x of warp w owns the 4-byte
// window (escape bytes x .. x + 3) at byte kEscPad + 64 w + 4 x, so a word reads
// its next eight escape bytes as the two aligned windows x and x + 4.  The
// 64-byte shift per warp keeps the 8-window groups that neighbouring warps
// write at their range boundaries disjoint; the front pad takes the raw patches
// that reach three windows back.  Ordinals are clamped to kEscOrdinalCap, so a
// malformed record cannot leave the buffer.
// A coded record holds at most (2048 - 48) * 2 = 4000 escapes.
constexpr int kEscOrdinalCap = 4000;
constexpr int kEscPad = 16;
constexpr int kEscBytes = kEscPad + 64 * 7 + 4 * (kEscOrdinalCap + 8) + 32;  // 16528

// Multipliers that are only known at run time, so that adds written as integer
// multiply-adds issue on the multiply pipe instead of the half-rate ALU pipe.
// (Right shifts as high multiplies were measured and dropped: they cost two
// dispatch slots each.)
struct PipeConsts {
  uint32_t one, four, two16, two29, two30, two31;
};
__host__ __device__ inline PipeConsts pipe_consts() {
  return PipeConsts{1u, 4u, 1u << 16, 1u << 29, 1u << 30, 1u << 31};
}

__device__ __forceinline__ uint32_t mul_hi(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.hi.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t mad_hi(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t mad_lo(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// a + b, on the multiply pipe (a * 1 + b with a run-time 1) unless the named
// experiment switch asks for the ALU pipe.
__device__ __forceinline__ uint32_t add_fma(uint32_t a, uint32_t b, const PipeConsts& k) {
  return mad_lo(a, k.one, b);
}

// x >> 16.  With FPB_SHIFT_MULHI the shift is a high multiply by 2^16 on the
// multiply pipe instead of a funnel shift on the ALU pipe.
__device__ __forceinline__ uint32_t shift_right_16(uint32_t x, const PipeConsts& k) {
#ifdef FPB_SHIFT_MULHI
  return mul_hi(x, k.two16);
#else
  (void)k;
  return x >> 16;
#endif
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// PTX prmt with the selector used as is: callers keep bit 3 of every used
// selector nibble clear (it would request sign replication).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// Exclusive prefix sum over the warp.  shfl.up reports whether the source lane
// exists, so each step is one shuffle and one predicated add.
__device__ __forceinline__ int warp_exclusive_sum(int v, int /*lane*/) {
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    asm("{\n\t.reg .pred p;\n\t.reg .s32 t;\n\t"
        "shfl.sync.up.b32 t|p, %0, %1, 0, 0xffffffff;\n\t"
        "@p add.s32 %0, %0, t;\n\t}"
        : "+r"(inc)
        : "r"(d));
  }
  return inc - v;
}

// Four escape nibbles (low 16 bits of n) -> their four extended-table bytes.
__device__ __forceinline__ uint32_t extended_bytes(const uint4& slut, uint32_t n) {
  const uint32_t low3 = n & 0x7777u;
  const uint32_t first = prmt(slut.x, slut.y, low3);   // entries 0..7
  const uint32_t second = prmt(slut.z, slut.w, low3);  // entries 8..15
  return prmt(first, second, 0x3210u | ((n >> 1) & 0x4444u));
}

// The two primary prmt words and the 16-byte extended table of one
// (layer, kv, head): attn_tables.py:96-124.
struct HeadTables {
  uint32_t p0, p1;
  uint4 ext;
};

__device__ __forceinline__ HeadTables load_tables(const int32_t* plut, const uint8_t* slut,
                                                  int table_index) {
  HeadTables t;
  t.p0 = static_cast<uint32_t>(plut[2 * table_index]);
  // Entry 7 is the escape code: the decoder relies on it reading as 0x00.
  t.p1 = static_cast<uint32_t>(plut[2 * table_index + 1]) & 0x00ffffffu;
  t.ext = *reinterpret_cast<const uint4*>(slut + 16 * table_index);
  return t;
}

// Raw record: owner t's word st is the 16 bytes at 16 (256 st + t)
// (attn_page.py:36-40, 279-282).
template <typename Emit>
__device__ __forceinline__ void raw_record_words(const uint8_t* rec, int tid, Emit&& emit) {
  const uint4* src = reinterpret_cast<const uint4*>(rec);
  uint4 v[8];
#pragma unroll
  for (int st = 0; st < 8; ++st) v[st] = src[st * kOwners + tid];
#pragma unroll
  for (int st = 0; st < 8; ++st) {
    const uint32_t w[4] = {v[st].x, v[st].y, v[st].z, v[st].w};
    emit(st, w);
  }
}

// Decodes owner `tid`'s 64 scalars of a CODED record and calls emit(st, w)
// for st = 0..7 where w[0..3] are the BF16 pairs (j0 f0, j0 f1, j1 f0, j1 f1).
//
// `rec` may be shared or global memory.  `esc` is a kEscBytes scratch in
// shared memory.  `released()` is called after the last read of `rec` by this
// warp: at the end, or with kEagerLow before the words are assembled.  Within one record each warp touches only its own part of `esc`,
// so only warp-level synchronisation happens in here; but the parts move with
// the record's escape prefixes, so two records may share one scratch only if a
// block-wide barrier separates their decodes.
//
// Phases: (1) the warp expands its escape nibbles through the extended table
// into sliding windows and patches raw scalars; (2) every owner counts its
// escapes and a warp scan gives its first ordinal; (3) per word: primary codes
// through prmt over the 8-byte table (an escape code selects the table's zero
// byte), escape bytes picked from two windows by exclusive rank, masked to the
// escape positions and OR-ed in, low and high bytes interleaved.
// The scheme is the one the format was laid out for
// (fragpack/ops/fragpack_common.cuh:92-186).
//
// The integer (ALU) pipe is the busiest unit of every kernel that runs this,
// so whatever has an equivalent on another pipe is written that way: adds as
// multiply-adds (k.one, k.four are run-time multipliers), the per-owner escape
// count as eight population counts, the scan's adds as predicated multiply-adds.
// kEagerLow: fetch all low bytes up front (records read straight from global
// memory, where four serialised fetches inside the word loop would each expose
// the memory latency) instead of on demand (records staged in shared memory,
// where the sixteen live registers cost more than the late fetches).
template <bool kEagerLow = false, typename Released, typename Emit>
__device__ __forceinline__ void coded_record_words(const uint8_t* rec, int vlen,
                                                   const HeadTables& tab, uint8_t* esc, int tid,
                                                   const PipeConsts& k, Released&& released,
                                                   Emit&& emit) {
  const int lane = tid & 31, warp = tid >> 5;
  uint2 sym[3];
#pragma unroll
  for (int m = 0; m < 3; ++m)
    sym[m] = reinterpret_cast<const uint2*>(rec + kLowBytes)[m * kOwners + tid];
  uint4 low[kEagerLow ? 4 : 1];
  if (kEagerLow) {
#pragma unroll
    for (int j = 0; j < 4; ++j) low[j] = reinterpret_cast<const uint4*>(rec)[j * kOwners + tid];
  }

  const uint8_t* var = rec + kDenseBytes;
  const uint16_t* h16 = reinterpret_cast<const uint16_t*>(var);
  const uint32_t* h32 = reinterpret_cast<const uint32_t*>(var);
  uint8_t* mine = esc + kEscPad + 64 * warp;
  // The header holds exclusive per-warp prefixes; the last warp's range ends at
  // the record's totals, whose low halves are h16[0] (escapes) and h16[2] (raw).
  const int first_esc = min((int)h16[8 + warp], kEscOrdinalCap);
  {
    const int end_esc = min((int)h16[warp < 7 ? 9 + warp : 0], kEscOrdinalCap);
    const uint32_t* nibbles = reinterpret_cast<const uint32_t*>(var + kHeaderBytes);
    const uint4 ext = tab.ext;
    __syncwarp();  // the previous record's readers of `mine` are done
    // 31 groups of eight escapes per round: lane L expands group g8 and takes
    // the first bytes of the next group from lane L + 1 (lane 31 only feeds).
    // end_esc <= kEscOrdinalCap keeps every nibble word inside the 2048-byte
    // variable region of a staged record; a record read in place from global
    // memory may end sooner, so there the index is clamped to the record.
    for (int base = first_esc >> 3; 8 * base < end_esc; base += 31) {
      int g8 = base + lane;
      if (kEagerLow) g8 = min(g8, max(0, (vlen - kHeaderBytes - 4) >> 2));
      const uint32_t n0 = nibbles[g8];
      const uint32_t b0 = extended_bytes(ext, n0), b1 = extended_bytes(ext, n0 >> 16);
      const uint32_t b2 = __shfl_down_sync(0xffffffffu, b0, 1);
#ifdef FPB_EXPAND_BRANCH
      if (lane < 31 && 8 * (base + lane) < end_esc) {
        uint4* dst = reinterpret_cast<uint4*>(mine + 32 * (base + lane));
        dst[0] = make_uint4(b0, __funnelshift_r(b0, b1, 8), __funnelshift_r(b0, b1, 16),
                            __funnelshift_r(b0, b1, 24));
        dst[1] = make_uint4(b1, __funnelshift_r(b1, b2, 8), __funnelshift_r(b1, b2, 16),
                            __funnelshift_r(b1, b2, 24));
      }
#else
      {
        // Lanes with nothing to store (the feeding lane 31, groups past the
        // warp's range) store to the spare 32 bytes at the end of the scratch
        // instead of branching around the stores.
        const bool live = lane < 31 && 8 * (base + lane) < end_esc;
        uint4* dst = reinterpret_cast<uint4*>(live ? mine + 32 * (base + lane)
                                                   : esc + kEscBytes - 32);
        dst[0] = make_uint4(b0, __funnelshift_r(b0, b1, 8), __funnelshift_r(b0, b1, 16),
                            __funnelshift_r(b0, b1, 24));
        dst[1] = make_uint4(b1, __funnelshift_r(b1, b2, 8), __funnelshift_r(b1, b2, 16),
                            __funnelshift_r(b1, b2, 24));
      }
#endif
    }
    // Raw scalars are rare: at most kMaxWarpRaw per warp, one patch per lane.
    const int first_raw = h16[16 + warp];
    const int n_raw = min((int)h16[warp < 7 ? 17 + warp : 2] - first_raw, kMaxWarpRaw);
    if (n_raw > 0) {  // uniform over the warp
      uint32_t patch = 0;
      if (lane < n_raw) {
        // Clamped so that a malformed header cannot read past the variable region.
        const uint32_t at =
            min(h32[2] + 4u * (uint32_t)(first_raw + lane), (uint32_t)max(vlen - 4, 0));
        patch = *reinterpret_cast<const uint32_t*>(var + (at & ~3u));
      }
      __syncwarp();
      if (lane < n_raw) {
        // The raw byte of ordinal x is byte j of window x - j.
        const int x = min((int)(patch & 0xffffu), kEscOrdinalCap);
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[4 * (x - j) + j] = (uint8_t)(patch >> 16);
      }
    }
  }

  if (kEagerLow) {
    // Symbols and low bytes are in registers, escapes in the scratch: the
    // record itself is no longer needed.
    __syncwarp();
    released();
  }

  // Selector words (3-bit codes, bit 3 clear) of the eight words; escapes are
  // the nibbles equal to 7, flagged in bit 3 of `flag`.
  uint32_t sel[8], flag[8];
#pragma unroll
  for (int gi = 0; gi < 2; ++gi) {
    const uint32_t w0 = gi == 0 ? sym[0].x : sym[1].y;
    const uint32_t w1 = gi == 0 ? sym[0].y : sym[2].x;
    const uint32_t w2 = gi == 0 ? sym[1].x : sym[2].y;
    sel[4 * gi + 0] = w0 & 0x77777777u;
    sel[4 * gi + 1] = w1 & 0x77777777u;
    sel[4 * gi + 2] = w2 & 0x77777777u;
    // Bit 3 of the three stored words carries the fourth word, one bit each.
    sel[4 * gi + 3] =
        ((w0 >> 3) & 0x11111111u) | ((w1 >> 2) & 0x22222222u) | ((w2 >> 1) & 0x44444444u);
#pragma unroll
    for (int x = 0; x < 3; ++x)
#ifdef FPB_FLAG_ALU
      flag[4 * gi + x] = (sel[4 * gi + x] + 0x11111111u) & 0x88888888u;
#else
      flag[4 * gi + x] = mad_lo(sel[4 * gi + x], k.one, 0x11111111u) & 0x88888888u;
#endif
    // The fourth word's code is 7 where all three carried bits are set.
    flag[4 * gi + 3] = w0 & w1 & w2 & 0x88888888u;
  }
  // Escapes of this owner: population counts go to their own unit, the adds to
  // the multiply pipe.
#if defined(FPB_COUNT_PACKED)
  // The flags of four words sit on distinct bits once shifted by 0..3.
  uint32_t count = 0;
#pragma unroll
  for (int gi = 0; gi < 2; ++gi)
    count += __popc(flag[4 * gi] | (flag[4 * gi + 1] >> 1) | (flag[4 * gi + 2] >> 2) |
                    (flag[4 * gi + 3] >> 3));
#elif defined(FPB_COUNT_ALU)
  uint32_t count = (uint32_t)__popc(flag[0]);
#pragma unroll
  for (int st = 1; st < 8; ++st) count += (uint32_t)__popc(flag[st]);
#else
  uint32_t count = (uint32_t)__popc(flag[0]);
#pragma unroll
  for (int st = 1; st < 8; ++st) count = mad_lo((uint32_t)__popc(flag[st]), k.one, count);
#endif
  // Inclusive warp scan; shfl.up reports whether the source lane exists.
  uint32_t inclusive = count;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
#ifdef FPB_SCAN_ALU
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t"
        "shfl.sync.up.b32 t|p, %0, %1, 0, 0xffffffff;\n\t"
        "@p add.u32 %0, %0, t;\n\t}"
        : "+r"(inclusive)
        : "r"(d));
#else
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t"
        "shfl.sync.up.b32 t|p, %0, %1, 0, 0xffffffff;\n\t"
        "@p mad.lo.u32 %0, t, %2, %0;\n\t}"
        : "+r"(inclusive)
        : "r"(d), "r"(k.one));
#endif
  }
  // A thread consumes at most 64 escapes: clamping its first ordinal bounds
  // every window read below.
  const int ordinal = min(first_esc + (int)(inclusive - count), kEscOrdinalCap - 64);
  __syncwarp();  // expansion and patches visible to the whole warp

  uint32_t window = smem_addr(mine) + 4u * (uint32_t)ordinal;
  uint4 lw;
#pragma unroll
  for (int st = 0; st < 8; ++st) {
    const uint32_t s = sel[st], f = flag[st];
    const uint32_t s_hi = shift_right_16(s, k);
    uint32_t ha = prmt(tab.p0, tab.p1, s);
    uint32_t hb = prmt(tab.p0, tab.p1, s_hi);
    // The next eight escape bytes are windows x and x + 4; the second one is
    // only fetched by the (rare) owners with more than four escapes in this word.
    const uint32_t n_here = (uint32_t)__popc(f);
    uint32_t e0, e1 = 0;
    asm("ld.shared.u32 %0, [%1];" : "=r"(e0) : "r"(window) : "memory");
#ifdef FPB_E1_ALWAYS
    asm("ld.shared.u32 %0, [%1+16];" : "=r"(e1) : "r"(window) : "memory");
#elif defined(FPB_E1_BRANCH)
    if (n_here > 4) asm("ld.shared.u32 %0, [%1+16];" : "=r"(e1) : "r"(window) : "memory");
#else
    // Predicated inside the statement: an `if` around it becomes a divergent
    // branch with its convergence bookkeeping, eight times per record.
    asm("{\n\t.reg .pred p;\n\tsetp.gt.u32 p, %2, 4;\n\t@p ld.shared.u32 %0, [%1+16];\n\t}"
        : "+r"(e1)
        : "r"(window), "r"(n_here)
        : "memory");
#endif
#ifdef FPB_WINDOW_ALU
    window += 4u * n_here;
#else
    window = mad_lo(n_here, k.four, window);
#endif
    // Nibble n of `rank` = escapes among the nibbles below n: the selector that
    // brings every position the escape byte it would take.
#ifdef FPB_RANK_SHIFTS
    // The same exclusive ranks by shifts and adds on the ALU pipe.
    uint32_t rank = f >> 3;
    rank += rank << 4;
    rank += rank << 8;
    rank = (rank + (rank << 16)) << 4;
#else
    const uint32_t rank = f * 0x02222222u;
#endif
#ifdef FPB_PICK_MERGE
    // Selector nibble n: n keeps the table byte, 4 + n takes the escape byte.
    const uint32_t pick = (f >> 1) + 0x32103210u;
    ha = prmt(ha, prmt(e0, e1, rank), pick);
    hb = prmt(hb, prmt(e0, e1, shift_right_16(rank, k)), pick >> 16);
#else
    // Byte masks of the escape positions (code 7 selects the 0xff byte); the
    // table gave those positions 0x00, so the escape bytes are OR-ed in.
    ha |= prmt(e0, e1, rank) & prmt(0u, 0xff000000u, s);
    hb |= prmt(e0, e1, shift_right_16(rank, k)) & prmt(0u, 0xff000000u, s_hi);
#endif
    // Low bytes are fetched as they are needed (two words per 16-byte chunk):
    // holding all sixteen registers across the loop cost more in lost
    // instruction-level parallelism than the later release of the record costs.
    if ((st & 1) == 0)
      lw = kEagerLow ? low[kEagerLow ? st >> 1 : 0]
                     : reinterpret_cast<const uint4*>(rec)[(st >> 1) * kOwners + tid];
    const uint32_t la = (st & 1) ? lw.z : lw.x;
    const uint32_t lb = (st & 1) ? lw.w : lw.y;
    const uint32_t w[4] = {__byte_perm(la, ha, 0x5140), __byte_perm(la, ha, 0x7362),
                           __byte_perm(lb, hb, 0x5140), __byte_perm(lb, hb, 0x7362)};
    emit(st, w);
  }
  if (!kEagerLow) {
    __syncwarp();
    released();
  }
}

// One owner's view of where its word scalars live in a token-major tile.
// For word st and pair index i = 2 j + f: (token, dim) of the first scalar.
struct OwnerCoords {
  int warp, g, c;
  __device__ __forceinline__ explicit OwnerCoords(int tid)
      : warp(tid >> 5), g((tid >> 2) & 7), c(tid & 3) {}
  __device__ __forceinline__ int row(int j) const { return 16 * warp + 8 * j + g; }
  __device__ __forceinline__ int col(int st, int f) const { return 16 * st + 8 * f + 2 * c; }
};

// Token-major 128 x 128 BF16 tile in shared memory: 256-byte rows of sixteen
// 16-byte chunks, chunk index XORed with (token & 7) so that both the
// fragment-order accesses and row-wise 16-byte accesses spread over the banks.
__device__ __forceinline__ uint8_t* tile_at(uint8_t* tile, int tok, int dim) {
  return tile + tok * 256 + ((((dim >> 3) ^ tok) & 15) << 4) + 2 * (dim & 7);
}

}  // namespace fpb
