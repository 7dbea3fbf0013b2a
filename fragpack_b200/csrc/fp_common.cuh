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
// Expanded escape bytes of one record: warp w keeps escape ordinal x at byte
// 32 w + x.  The 32-byte shift keeps the 8-byte groups that neighbouring warps
// write at their range boundaries disjoint.  Ordinals are clamped to
// kEscOrdinalCap when they are written, and readers reach at most 2048 + 12
// bytes further, so a malformed record cannot leave the buffer.
constexpr int kEscOrdinalCap = 4096;
constexpr int kEscBytes = 32 * 7 + kEscOrdinalCap + 2048 + 32;  // 6400

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

__device__ __forceinline__ int warp_exclusive_sum(int v, int lane) {
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += up;
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
  t.p1 = static_cast<uint32_t>(plut[2 * table_index + 1]);
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
// shared memory; each warp touches only its own part of it, so only warp-level
// synchronisation happens in here.  `released()` is called once every read of
// `rec` by this warp has been made (dense part held in registers, escapes
// expanded), so the caller may hand the record's buffer back to a producer.
//
// Follows the decoder the format was designed for
// (fragpack/ops/fragpack_common.cuh:92-186) with a byte-per-escape scratch
// instead of sliding windows.
template <typename Released, typename Emit>
__device__ __forceinline__ void coded_record_words(const uint8_t* rec, const HeadTables& tab,
                                                   uint8_t* esc, int tid, Released&& released,
                                                   Emit&& emit) {
  const int lane = tid & 31, warp = tid >> 5;
  uint4 low[4];
  uint2 sym[3];
#pragma unroll
  for (int j = 0; j < 4; ++j) low[j] = reinterpret_cast<const uint4*>(rec)[j * kOwners + tid];
#pragma unroll
  for (int m = 0; m < 3; ++m)
    sym[m] = reinterpret_cast<const uint2*>(rec + kLowBytes)[m * kOwners + tid];

  const uint8_t* var = rec + kDenseBytes;
  const uint16_t* h16 = reinterpret_cast<const uint16_t*>(var);
  const uint32_t* h32 = reinterpret_cast<const uint32_t*>(var);
  uint8_t* mine = esc + 32 * warp;
  const int first_esc = min((int)h16[8 + warp], kEscOrdinalCap);
  {
    const int end_esc = min(warp < 7 ? (int)h16[9 + warp] : (int)h32[0], kEscOrdinalCap);
    const uint32_t* nibbles = reinterpret_cast<const uint32_t*>(var + kHeaderBytes);
    __syncwarp();  // the previous record's readers of `mine` are done
    for (int k = (first_esc >> 3) + lane; 8 * k < end_esc; k += 32) {
      const uint32_t n = nibbles[k];
      *reinterpret_cast<uint2*>(mine + 8 * k) =
          make_uint2(extended_bytes(tab.ext, n), extended_bytes(tab.ext, n >> 16));
    }
    // At most kMaxWarpRaw raw scalars per warp: one patch per lane.
    const int first_raw = h16[16 + warp];
    const int n_raw = min((warp < 7 ? (int)h16[17 + warp] : (int)h32[1]) - first_raw, kMaxWarpRaw);
    uint32_t patch = 0;
    if (lane < n_raw) {
      // Clamped so that a malformed header cannot read past the variable region.
      const uint32_t at = min(h32[2] + 4u * (uint32_t)(first_raw + lane), (uint32_t)(kVarCap - 4));
      patch = *reinterpret_cast<const uint32_t*>(var + (at & ~3u));
    }
    __syncwarp();
    released();
    if (lane < n_raw) mine[min(patch & 0xffffu, (uint32_t)kEscOrdinalCap)] = (uint8_t)(patch >> 16);
  }

  // Escape flags (bit 3 of each nibble) of the eight words and their count.
  uint32_t sel[8];
  int count = 0;
#pragma unroll
  for (int gi = 0; gi < 2; ++gi) {
    const uint32_t w0 = gi == 0 ? sym[0].x : sym[1].y;
    const uint32_t w1 = gi == 0 ? sym[0].y : sym[2].x;
    const uint32_t w2 = gi == 0 ? sym[1].x : sym[2].y;
    sel[4 * gi + 0] = w0 & 0x77777777u;
    sel[4 * gi + 1] = w1 & 0x77777777u;
    sel[4 * gi + 2] = w2 & 0x77777777u;
    sel[4 * gi + 3] =
        ((w0 >> 3) & 0x11111111u) | ((w1 >> 2) & 0x22222222u) | ((w2 >> 1) & 0x44444444u);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      count += __popc((sel[4 * gi + k] + 0x11111111u) & 0x88888888u);
  }
  int ordinal = first_esc + warp_exclusive_sum(count, lane);
  __syncwarp();  // expansion and patches visible to the whole warp

  const uint32_t* mine32 = reinterpret_cast<const uint32_t*>(mine);
#pragma unroll
  for (int st = 0; st < 8; ++st) {
    const uint32_t s = sel[st], f = (s + 0x11111111u) & 0x88888888u;
    uint32_t ha = prmt(tab.p0, tab.p1, s);
    uint32_t hb = prmt(tab.p0, tab.p1, s >> 16);
    {
      // The next eight escape bytes from `ordinal` on, unaligned.
      const uint32_t* at = mine32 + (ordinal >> 2);
      const uint32_t shift = (ordinal & 3) * 8;
      const uint32_t a = at[0], b = at[1], c = at[2];
      const uint32_t e0 = __funnelshift_r(a, b, shift), e1 = __funnelshift_r(b, c, shift);
      ordinal += __popc(f);
      // Nibble n of `rank` = escapes among nibbles below n.
      const uint32_t rank = f * 0x02222222u;
      ha = prmt(ha, prmt(e0, e1, rank), (f >> 1) + 0x3210u);
      hb = prmt(hb, prmt(e0, e1, rank >> 16), (f >> 17) + 0x3210u);
    }
    const uint4& lw = low[st >> 1];
    const uint32_t la = (st & 1) ? lw.z : lw.x;
    const uint32_t lb = (st & 1) ? lw.w : lw.y;
    const uint32_t w[4] = {__byte_perm(la, ha, 0x5140), __byte_perm(la, ha, 0x7362),
                           __byte_perm(lb, hb, 0x5140), __byte_perm(lb, hb, 0x7362)};
    emit(st, w);
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
