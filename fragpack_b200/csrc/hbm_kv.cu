// HBM KV store kernels for sm_100a: the token writer, the block encoder, the
// prefill decompressor and the batch codec entry points (the step lifecycle
// lives in lifecycle.cu).  What they compute follows fragpack/ops/hbm_kv.cu of
// the reference (cited per kernel); the byte format is attn_page.py's.
#include <stdarg.h>
#include <stdio.h>

#include "fp_api.h"
#include "fp_common.cuh"
#include "fp_pipe.cuh"
#include "fp_store.cuh"

namespace fpb {

namespace {
thread_local char g_error[512] = "";
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

int cuda_status(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return FP_OK;
  return fail(FP_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

const char* last_error() { return g_error; }

namespace {
std::atomic<long long> g_wait_limit{kWaitCycles};
std::atomic<long long> g_skip_record{-1};
}  // namespace

WaitDebug wait_debug() {
  return WaitDebug{g_wait_limit.load(std::memory_order_relaxed),
                   g_skip_record.load(std::memory_order_relaxed)};
}

namespace {

// ---------------------------------------------------------------------------
// Token writer (replaces write_kernel, hbm_kv.cu:221-255): scatters tokens'
// K and V rows into the fragment order of their block's staging record (see
// fp_common.cuh for the owner layout).
//
// Sixteen tokens at offsets 16 i .. 16 i + 15 of one block are a complete
// piece of the record: for K the 32 owners of row group i (512 contiguous
// bytes in each of the eight word planes), for V the whole word plane i (4 KB
// contiguous).  A CTA looks at sixteen consecutive input tokens and handles
//  * every such group that STARTS at one of them and is complete and
//    contiguous in the input (the bulk of a prefill): rows are staged in shared
//    memory and written with 16-byte coalesced stores;
//  * every token of its sixteen that no complete group covers (sequence ends,
//    decode steps): 4-byte / 2-byte scattered stores.
// grid = (ceil(tokens / 16), ceil(H / kWriteHeads)).
// ---------------------------------------------------------------------------
constexpr int kWriteHeads = 4;          // KV heads per CTA
constexpr int kWriteRow = 272;          // bytes per staged token row (256 + pad)

// The general path: one token's K and V rows of one head go to their places in
// the record, one warp per (token, head), lane l carrying dims 4 l .. 4 l + 3
// (one 8-byte load of each row).  A K token is a row of the A fragment: its
// dims are spread over all eight word planes, two neighbouring owners per
// lane, as 4-byte pairs.  A V token is a column: every dim lands in another
// owner's word as a single scalar.
__device__ __forceinline__ void scatter_token_row(uint8_t* k_rec, uint8_t* v_rec,
                                                  const uint16_t* k_row, const uint16_t* v_row,
                                                  int off, int lane) {
  // Rows are only known to be 4-byte aligned: two 4-byte loads each.
  const uint32_t* k32 = reinterpret_cast<const uint32_t*>(k_row) + 2 * lane;
  const uint32_t* v32 = reinterpret_cast<const uint32_t*>(v_row) + 2 * lane;
  const uint2 kk = make_uint2(k32[0], k32[1]), vv = make_uint2(v32[0], v32[1]);
  {
    // dims 4 l .. 4 l + 3 = pairs 2 l and 2 l + 1 of word st = l / 4; inside the
    // word they are owner columns c = 2 (l & 1) and + 1 of half f = (l / 2) & 1.
    const int st = lane >> 2, f = (lane >> 1) & 1, c = 2 * (lane & 1);
    const int owner = 32 * (off >> 4) + 4 * (off & 7) + c;
    uint8_t* at = k_rec + 16 * (kOwners * st + owner) + 4 * (2 * ((off >> 3) & 1) + f);
    *reinterpret_cast<uint32_t*>(at) = kk.x;
    *reinterpret_cast<uint32_t*>(at + 16) = kk.y;
  }
  {
    // Token `off` is scalar e = off & 1 of pair c = (off / 2) & 3, half
    // f = (off / 8) & 1 of word st = off / 16, in the owners of its dims.
    const int st = off >> 4, within = 2 * ((off >> 3) & 1) + (off & 1), c = (off >> 1) & 3;
    const uint32_t vals[4] = {vv.x & 0xffffu, vv.x >> 16, vv.y & 0xffffu, vv.y >> 16};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int d = 4 * lane + x;
      const int owner = 32 * (d >> 4) + 4 * (d & 7) + c;
      // j = (d / 8) & 1 selects the register pair of the owner's word.
      uint8_t* at = v_rec + 16 * (kOwners * st + owner) + 2 * (4 * ((d >> 3) & 1) + within);
      *reinterpret_cast<uint16_t*>(at) = (uint16_t)vals[x];
    }
  }
}

// 16 bytes global -> shared without a register in between.
__device__ __forceinline__ void async_copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(256)
write_kernel(StoreView v, const uint16_t* key, const uint16_t* value, int64_t ks0, int64_t ks1,
             int64_t vs0, int64_t vs1, const int64_t* slots, int64_t n_tokens, int layer,
             int vector_ok) {
  const fp_store& s = v.s;
  __shared__ __align__(16) uint8_t tile[kWriteHeads][2][16][kWriteRow];
  __shared__ int tok_slot[16];   // staging slot of each token, -1: skip the token
  __shared__ int tok_off[16];    // offset of each token in its block
  __shared__ int tok_flags[16];  // bit 0: covered by a complete group, bit 1: starts one
  const int tid = threadIdx.x;
  const int64_t t0 = (int64_t)blockIdx.x * 16;
  const int head0 = blockIdx.y * kWriteHeads;
  const int heads = min(kWriteHeads, s.H - head0);

  if (tid < 16) {
    const int64_t t = t0 + tid;
    int w = -1, off = 0, flags = 0;
    if (t < n_tokens) {
      const int64_t slot = slots[t];
      if (slot >= 0 && (slot >> 7) < s.NB) {
        off = (int)(slot & 127);
        w = s.wslot[slot >> 7];
        // The group of this token: offsets (off & ~15) .. + 15 of its block,
        // complete and contiguous iff the sixteen inputs from `first` map to them.
        const int64_t first = t - (off & 15), base = slot - (off & 15);
        if (vector_ok && w >= 0 && first >= 0 && first + 16 <= n_tokens) {
          bool whole = true;
          for (int k = 0; k < 16; ++k) whole &= slots[first + k] == base + k;
          if (whole) flags = 1 | ((off & 15) == 0 ? 2 : 0);
        }
      }
    }
    tok_slot[tid] = w;
    tok_off[tid] = off;
    tok_flags[tid] = flags;
  }
  __syncthreads();

  // Tokens outside every complete group: one warp per (token, head).
  for (int x = tid >> 5; x < 16 * heads; x += 8) {
    const int k = x / heads, head = head0 + x % heads;
    if (tok_slot[k] < 0 || (tok_flags[k] & 1)) continue;
    scatter_token_row(v.staging(tok_slot[k], layer, head), v.staging(tok_slot[k], layer, s.H + head),
                      key + (t0 + k) * ks0 + head * ks1, value + (t0 + k) * vs0 + head * vs1,
                      tok_off[k], tid & 31);
  }

  // Complete groups that start here (their later tokens may belong to the next CTA's sixteen).
  for (int k = 0; k < 16; ++k) {
    if (!(tok_flags[k] & 2)) continue;
    const int w = tok_slot[k], group = tok_off[k] >> 4;
    const int64_t first = t0 + k;
    // All of the CTA's heads are copied into shared memory before the first is
    // transposed, asynchronously and without passing through registers: the
    // loads of four heads (64 KB per CTA) are in flight together, the CTA meets
    // at two barriers per group, and the kernel stays small in registers.
    const int row = tid >> 4, col = tid & 15;  // 16 tokens x 16 chunks of 16 bytes
    __syncthreads();  // the previous group's tiles have been read
#pragma unroll
    for (int h = 0; h < kWriteHeads; ++h)
      if (h < heads) {
        const int head = head0 + h;
        async_copy16(&tile[h][0][row][16 * col], key + (first + row) * ks0 + head * ks1 + 8 * col);
        async_copy16(&tile[h][1][row][16 * col], value + (first + row) * vs0 + head * vs1 + 8 * col);
      }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kWriteHeads; ++h) {
      if (h >= heads) break;
      const int head = head0 + h;
      {
        // K: thread (st, g, c) owns word st of owner 32 group + 4 g + c: tokens g
        // and g + 8, dim pairs 16 st + 2 c and + 8.
        const int st = tid >> 5, g = (tid >> 2) & 7, c = tid & 3;
        uint4 out;
        out.x = *reinterpret_cast<const uint32_t*>(&tile[h][0][g][2 * (16 * st + 2 * c)]);
        out.y = *reinterpret_cast<const uint32_t*>(&tile[h][0][g][2 * (16 * st + 8 + 2 * c)]);
        out.z = *reinterpret_cast<const uint32_t*>(&tile[h][0][g + 8][2 * (16 * st + 2 * c)]);
        out.w = *reinterpret_cast<const uint32_t*>(&tile[h][0][g + 8][2 * (16 * st + 8 + 2 * c)]);
        uint8_t* rec = v.staging(w, layer, head);
        *reinterpret_cast<uint4*>(rec + 16 * (kOwners * st + 32 * group + (tid & 31))) = out;
      }
      {
        // V: thread = owner (dw, dg, vc) of word plane `group`: dims 16 dw + dg
        // and + 8, tokens 2 vc, 2 vc + 1 and + 8.
        const int dw = tid >> 5, dg = (tid >> 2) & 7, vc = tid & 3;
        uint32_t out[4];
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int f = 0; f < 2; ++f) {
            const int dim = 16 * dw + 8 * b + dg, tok = 8 * f + 2 * vc;
            const uint32_t lo = *reinterpret_cast<const uint16_t*>(&tile[h][1][tok][2 * dim]);
            const uint32_t hi = *reinterpret_cast<const uint16_t*>(&tile[h][1][tok + 1][2 * dim]);
            out[2 * b + f] = lo | (hi << 16);
          }
        uint8_t* rec = v.staging(w, layer, s.H + head);
        *reinterpret_cast<uint4*>(rec + 16 * (kOwners * group + tid)) =
            make_uint4(out[0], out[1], out[2], out[3]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Block encoder core: attn_page.py:146-209 on one CTA of 256 owners, each
// holding its eight fragment words.  Bit-exact with the reference encoder.
// ---------------------------------------------------------------------------
struct EncodeShared {
  __align__(16) uint8_t var[kVarCap];
  // Per byte position k of a packed word and per high byte: .x = the 3-bit
  // primary code (7 = escape) already at nibble k, plus an escape flag at bit
  // 16 + k and a flag for a byte outside the table at bit 24 + k; .y = the
  // escape nibble (rank - 7, or 15 for a byte outside the table) already at
  // byte k.  Four look-ups OR into the packed codes, the
  // escape mask and the escape bytes of four scalars with no shifting or
  // repacking afterwards.
  __align__(16) uint2 classes[4][256];
  // Per 8-bit escape mask: byte selectors (prmt nibbles) listing the flagged
  // positions in ascending order; unused selectors are 8, which makes prmt
  // replicate the sign bit of an escape byte (always clear): a zero byte.
  uint32_t compact[256];
  // The owners' low bytes, packed in store order, wait here from the
  // classification to the final stores (sixteen registers less per thread).
  __align__(16) uint4 park_low[4][kOwners];
  int warp_sum[2][8];
  uint8_t* dst;
  int raw;
};

// The class tables are indexed by the high byte rotated left by one bit: the
// sign moves to bit 0, so +x and -x, and neighbouring exponents, are
// neighbours.  Real KV uses a handful of exponents with both signs; unrotated,
// +x and -x sit 128 entries apart - same banks, different words - and the
// look-ups of a warp replay on bank conflicts.
__device__ __forceinline__ uint32_t table_slot(uint32_t high) {
  return ((high << 1) | (high >> 7)) & 0xffu;
}

// Class-table entries of high byte `tid`, whose rank in the table is `r`.
__device__ __forceinline__ void store_classes(EncodeShared& sh, uint32_t r, int tid) {
  const uint32_t code = min(r, (uint32_t)kPrimaryDirect);
  const uint32_t nib = r < kPrimaryDirect ? 0u : (r < kTableEntries ? r - kPrimaryDirect : 15u);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    sh.classes[k][table_slot((uint32_t)tid)] =
        make_uint2((code << (4 * k)) | ((uint32_t)(r >= kPrimaryDirect) << (16 + k)) |
                       ((uint32_t)(r >= kTableEntries) << (24 + k)),
                   nib << (8 * k));
}

// Selector-table entry of escape mask `tid`.
__device__ __forceinline__ void store_selectors(EncodeShared& sh, int tid) {
  uint32_t pick = 0x88888888u;
  int n = 0;
  for (int pos = 0; pos < 8; ++pos)
    if ((tid >> pos) & 1) {
      pick ^= (8u ^ (uint32_t)pos) << (4 * n);
      ++n;
    }
  sh.compact[tid] = pick;
}

// Fills the class tables from `rank_of` and the selector table (one entry of
// each per thread).
__device__ __forceinline__ void load_classes(EncodeShared& sh, const uint8_t* rank_of, int tid) {
  store_classes(sh, rank_of[tid], tid);
  store_selectors(sh, tid);
}

struct EncodePlan {
  int var_len;   // variable-region bytes if coded
  bool codes;    // false: raw fallback (attn_page.py:200-202)
};

// Classes of the four high bytes packed in `hi`: .x = their primary codes as
// four nibbles, .y = their escape nibbles as four bytes.
__device__ __forceinline__ uint2 classes4(const EncodeShared& sh, uint32_t hi, const PipeConsts& k) {
  // All four bytes rotated at once (see table_slot).
  const uint32_t at = ((hi << 1) & 0xfefefefeu) | ((hi >> 7) & 0x01010101u);
  const uint2 c0 = sh.classes[0][at & 0xffu], c1 = sh.classes[1][(at >> 8) & 0xffu];
  const uint2 c2 = sh.classes[2][(at >> 16) & 0xffu], c3 = sh.classes[3][at >> 24];
  // The four entries occupy disjoint bits, so their OR is their sum: written
  // as multiply-adds, it issues on the multiply pipe instead of the half-rate
  // integer pipe that the rest of the classification keeps busy.
  return make_uint2(add_fma(add_fma(c0.x, c1.x, k), add_fma(c2.x, c3.x, k), k),
                    add_fma(add_fma(c0.y, c1.y, k), add_fma(c2.y, c3.y, k), k));
}

// What classification leaves in an owner's registers.
struct OwnerCodes {
  uint32_t sym[6];    // symbol words
  uint64_t queue;     // first 16 escape nibbles
  // Bit 8 st + e of esc / raw: scalar e of word st escapes / is outside the table.
  uint32_t esc[2], raw[2];
  int n_esc, n_raw;
};

// Classifies the 64 scalars of an owner four at a time: primary codes as
// nibble words, escape nibbles appended to a queue (the first 16; longer runs
// are redone by build_variable_region).  `wd` is dead afterwards: the low bytes
// are set aside in packed form as each word is consumed, so the 32 registers of
// the record do not stay live to the end.  Scalars outside the table (raw
// entries) are only marked while the words go by; build_variable_region makes
// their entries, after the barrier at which the record's size becomes known,
// so that the loop over them (lanes differ in how many they have, and each
// fetches a high byte again) runs beside the placement's atomic instead of
// holding every warp of the CTA up in front of that barrier.
__device__ __forceinline__ void classify(const uint4 (&wd)[8], EncodeShared& sh, int tid,
                                         const PipeConsts& k, OwnerCodes& o) {
  uint32_t codes[8], marks[4], low[4];
  o.queue = 0;
  int n_esc = 0;
#pragma unroll
  for (int st = 0; st < 8; ++st) {
    const uint32_t hi_a = __byte_perm(wd[st].x, wd[st].y, 0x7531);
    const uint32_t hi_b = __byte_perm(wd[st].z, wd[st].w, 0x7531);
    low[2 * (st & 1)] = __byte_perm(wd[st].x, wd[st].y, 0x6420);
    low[2 * (st & 1) + 1] = __byte_perm(wd[st].z, wd[st].w, 0x6420);
    if (st & 1) sh.park_low[st >> 1][tid] = make_uint4(low[0], low[1], low[2], low[3]);
    const uint2 ca = classes4(sh, hi_a, k), cb = classes4(sh, hi_b, k);
    codes[st] = prmt(ca.x, cb.x, 0x5410u);
    // Byte 0: which of the eight scalars escape; byte 1: which are outside the table.
    const uint32_t flags = (ca.x >> 16) | ((cb.x >> 16) << 4);
    if (st & 1)
      marks[st >> 1] = prmt(marks[st >> 1], flags, 0x5410u);
    else
      marks[st >> 1] = flags;
    // This word's escape nibbles, in order, without a loop over them (lanes
    // differ in how many they have; a loop runs as long as the worst lane).
    const uint32_t mask8 = flags & 0xffu;
    const uint32_t pick = sh.compact[mask8];  // byte selectors that move flagged bytes to the front
    const uint32_t front_lo = prmt(ca.y, cb.y, pick), front_hi = prmt(ca.y, cb.y, pick >> 16);
    // Eight bytes holding one nibble each -> eight adjacent nibbles: OR-ing a
    // word with itself shifted by four pairs the nibbles up in bytes 0 and 2.
    const uint32_t pair_lo = front_lo | (front_lo >> 4), pair_hi = front_hi | (front_hi >> 4);
    const uint32_t packed = prmt(pair_lo, pair_hi, 0x6420u);
    if (n_esc < 16) o.queue |= (uint64_t)packed << (4 * n_esc);
    n_esc += __popc(mask8);
  }
  o.esc[0] = prmt(marks[0], marks[1], 0x6420u);
  o.esc[1] = prmt(marks[2], marks[3], 0x6420u);
  o.raw[0] = prmt(marks[0], marks[1], 0x7531u);
  o.raw[1] = prmt(marks[2], marks[3], 0x7531u);
  const int n_raw = __popc(o.raw[0]) + __popc(o.raw[1]);
  o.n_esc = n_esc;
  o.n_raw = n_raw;
  // Symbol words: per 32-scalar group three words; bit 3 of word b's nibble j
  // is bit b of the code of scalar 24 + j (attn_page.py:174-181).
#pragma unroll
  for (int gi = 0; gi < 2; ++gi)
#pragma unroll
    for (int b = 0; b < 3; ++b)
      o.sym[3 * gi + b] = codes[4 * gi + b] | (((codes[4 * gi + 3] >> b) & 0x11111111u) << 3);
}

// Where an owner's escapes and raw entries go, and the record's plan.
struct OwnerLayout {
  int esc_at, raw_at, esc_total, raw_total, raw_offset;
  EncodePlan plan;
};

// Ordinals of the owner's escapes and raw entries within the record (two warp
// scans and one pass over the warps' sums; one barrier).
__device__ __forceinline__ OwnerLayout record_layout(EncodeShared& sh, int n_esc, int n_raw, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
  const int esc_before = warp_exclusive_sum(n_esc, lane);
  const int raw_before = warp_exclusive_sum(n_raw, lane);
  if (lane == 31) {
    sh.warp_sum[0][warp] = esc_before + n_esc;
    sh.warp_sum[1][warp] = raw_before + n_raw;
  }
  __syncthreads();
  OwnerLayout at;
  at.esc_at = esc_before;
  at.raw_at = raw_before;
  at.esc_total = at.raw_total = 0;
  int raw_worst = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int ew = sh.warp_sum[0][w], rw = sh.warp_sum[1][w];
    if (w < warp) {
      at.esc_at += ew;
      at.raw_at += rw;
    }
    at.esc_total += ew;
    at.raw_total += rw;
    raw_worst = max(raw_worst, rw);
  }
  at.raw_offset = (kHeaderBytes + ((at.esc_total + 1) >> 1) + 3) & ~3;
  at.plan.var_len = (at.raw_offset + 4 * at.raw_total + 15) & ~15;
  at.plan.codes = at.plan.var_len <= kVarCap && raw_worst <= kMaxWarpRaw;
  return at;
}

// Builds the variable region in `sh.var` (zero beforehand, with a barrier in
// between).  `reload(st)` fetches word st of the owner's record again for the
// rare owner with more escapes or raw scalars than the queues hold.
template <typename Reload>
__device__ __forceinline__ void build_variable_region(EncodeShared& sh, const OwnerCodes& o,
                                                      const OwnerLayout& at, int tid,
                                                      Reload&& reload) {
  if (!at.plan.codes) return;  // the record is stored raw
  uint32_t* var32 = reinterpret_cast<uint32_t*>(sh.var);
  if (o.n_esc > 0 && o.n_esc <= 16) {
    // This owner's nibbles are consecutive from nibble `esc_at` of the stream
    // that starts at byte 48 (word 12).
    const int word = (kHeaderBytes >> 2) + (at.esc_at >> 3), shift = 4 * (at.esc_at & 7);
    const uint64_t lo = o.queue << shift;
    const uint32_t hi = shift ? (uint32_t)(o.queue >> (64 - shift)) : 0u;
    if ((uint32_t)lo) atomicOr(&var32[word], (uint32_t)lo);
    if ((uint32_t)(lo >> 32)) atomicOr(&var32[word + 1], (uint32_t)(lo >> 32));
    if (hi) atomicOr(&var32[word + 2], hi);
  }
  if (o.n_raw > 0 && o.n_raw <= 4 && o.n_esc <= 16) {
    // Raw entries `ordinal | high << 16` (attn_page.py:188-191): the ordinal
    // from the masks, the high byte from the record's word again.
    uint32_t left[2] = {o.raw[0], o.raw[1]};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      if (x < o.n_raw) {
        const int half = left[0] ? 0 : 1;
        const uint32_t m = left[half];
        const int bit = __ffs(m) - 1;
        left[half] = m & (m - 1);
        const uint32_t below = (1u << bit) - 1u;
        const int ordinal =
            half ? __popc(o.esc[0]) + __popc(o.esc[1] & below) : __popc(o.esc[0] & below);
        const uint4 w = reload(4 * half + (bit >> 3));
        const int e = bit & 7;
        const uint32_t pair = e < 4 ? (e < 2 ? w.x : w.y) : (e < 6 ? w.z : w.w);
        const uint32_t high = (pair >> (8 + 16 * (e & 1))) & 0xffu;
        var32[(at.raw_offset >> 2) + at.raw_at + x] = (uint32_t)(at.esc_at + ordinal) | (high << 16);
      }
    }
  }
  if (o.n_esc > 16 || o.n_raw > 4) {
    // Rare: walk the scalars again.
    int ordinal = at.esc_at, raw_at = at.raw_at;
#pragma unroll 1
    for (int st = 0; st < 8; ++st) {
      const uint4 w = reload(st);
      const uint32_t highs[2] = {__byte_perm(w.x, w.y, 0x7531), __byte_perm(w.z, w.w, 0x7531)};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t high = (highs[e >> 2] >> (8 * (e & 3))) & 0xffu;
        const uint2 c = sh.classes[0][table_slot(high)];
        if ((c.x & 0xfu) == (uint32_t)kPrimaryDirect) {
          const uint32_t nib = c.y;
          if (o.n_esc > 16) {
            const int bit = 8 * kHeaderBytes + 4 * ordinal;
            atomicOr(&var32[bit >> 5], nib << (bit & 31));
          }
          if (nib == 15u) var32[(at.raw_offset >> 2) + raw_at++] = (uint32_t)ordinal | (high << 16);
          ++ordinal;
        }
      }
    }
  }
  if (tid == 0) {
    var32[0] = at.esc_total;
    var32[1] = at.raw_total;
    var32[2] = at.raw_offset;
    var32[3] = 0;
    uint16_t* h16 = reinterpret_cast<uint16_t*>(sh.var);
    int e = 0, r = 0;
    for (int w = 0; w < 8; ++w) {
      h16[8 + w] = (uint16_t)e;
      h16[16 + w] = (uint16_t)r;
      e += sh.warp_sum[0][w];
      r += sh.warp_sum[1][w];
    }
  }
}

// Dense part of a coded record: low bytes in four 16-byte chunks, symbols in
// three 8-byte chunks, both chunk-major (attn_page.py:272-276).
__device__ __forceinline__ void store_dense(uint8_t* dst, const uint4 (&low)[4], const uint2 (&sym)[3],
                                            int tid) {
#pragma unroll
  for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j * kOwners + tid] = low[j];
#pragma unroll
  for (int m = 0; m < 3; ++m) reinterpret_cast<uint2*>(dst + kLowBytes)[m * kOwners + tid] = sym[m];
}

// One record on one CTA of 256 owners, start to end.  `place(plan, raw)` is
// called by all lanes of warp 0 together and returns, in every lane, where the
// record goes; it sets `raw` when the record must be stored raw; a null
// destination drops the record.
template <typename Reload, typename Place>
__device__ __forceinline__ void encode_cta(const uint4 (&wd)[8], EncodeShared& sh, int tid,
                                           const PipeConsts& k, Reload&& reload, Place&& place) {
  for (int i = tid; i < kVarCap / 16; i += kOwners)
    reinterpret_cast<uint4*>(sh.var)[i] = make_uint4(0, 0, 0, 0);
  OwnerCodes o;
  classify(wd, sh, tid, k, o);
  const OwnerLayout at = record_layout(sh, o.n_esc, o.n_raw, tid);
  if (tid < 32) {
    bool raw = !at.plan.codes;
    uint8_t* dst = place(at.plan, raw);
    if (tid == 0) {
      sh.dst = dst;
      sh.raw = raw;
    }
  }
  build_variable_region(sh, o, at, tid, reload);
  __syncthreads();  // placement known, variable region complete
  uint8_t* dst = sh.dst;
  if (dst == nullptr) return;
  if (sh.raw) {
#pragma unroll
    for (int st = 0; st < 8; ++st) reinterpret_cast<uint4*>(dst)[st * kOwners + tid] = reload(st);
    return;
  }
  const uint4 low[4] = {sh.park_low[0][tid], sh.park_low[1][tid], sh.park_low[2][tid],
                        sh.park_low[3][tid]};
  const uint2 sym[3] = {make_uint2(o.sym[0], o.sym[1]), make_uint2(o.sym[2], o.sym[3]),
                        make_uint2(o.sym[4], o.sym[5])};
  store_dense(dst, low, sym, tid);
  for (int i = tid; i < at.plan.var_len / 16; i += kOwners)
    reinterpret_cast<uint4*>(dst + kDenseBytes)[i] = reinterpret_cast<const uint4*>(sh.var)[i];
}

// grid (max_close, 2 H): CTA (i, rec) encodes record `rec` of close_list[i]
// at `layer` from staging.  hbm_kv.cu:257-429.
// Five CTAs per SM (48 registers; the low bytes wait in shared memory instead
// of sixteen registers): the kernel's stalls are the loads at a CTA's start
// and the placement's atomic at its end, which only other resident CTAs cover.
// A fourth CTA measured 12 % faster than three, the fifth 8 % faster again; a
// sixth (40 registers, spills) is slower.
__global__ void __launch_bounds__(kOwners, 5)
encode_kernel(StoreView v, int layer, uint8_t* arena, int64_t page_bytes, const uint8_t* rank_of,
              PipeConsts k) {
  __shared__ EncodeShared sh;
  const fp_store& s = v.s;
  const int rec = blockIdx.y, tid = threadIdx.x;
  // counters -> close_list -> wslot -> record would be four dependent round
  // trips before the first scalar can be classified.  The first two are
  // independent loads, and the record is fetched before the count is checked
  // (a stale list entry is clamped into range, so the fetch is always legal).
  const int closes = s.counters[FP_CTR_CLOSES];
  const int listed = s.close_list[blockIdx.x];
  const uint32_t rank = rank_of[((int64_t)layer * 2 * s.H + rec) * 256 + tid];
  const int block = min(max(listed, 0), s.NB - 1);
  const int slot = min(max(s.wslot[block], 0), s.S_p + s.S_t - 1);
  uint8_t* src = v.staging(slot, layer, rec);
  uint4 wd[8];
#pragma unroll
  for (int st = 0; st < 8; ++st) wd[st] = reinterpret_cast<const uint4*>(src)[st * kOwners + tid];
  if ((int)blockIdx.x >= closes) return;
  const int64_t idx = v.table_index(layer, block, rec);
  store_classes(sh, rank, tid);
  store_selectors(sh, tid);
  __syncthreads();
  const auto reload = [&](int st) { return reinterpret_cast<const uint4*>(src)[st * kOwners + tid]; };
  encode_cta(wd, sh, tid, k, reload, [&](const EncodePlan& plan, bool& raw) -> uint8_t* {
    const int lane = tid & 31;
    int at = -1;
    if (lane == 0) {
      if (plan.codes) {
        // Claim page bytes.  Fast path: one fetch-add (the records of a page are
        // encoded at the same time, and a compare-and-swap loop on one word
        // serialises them with retries).  A claim that would overshoot the page
        // is undone at once, and a compare-and-swap loop then decides, so that a
        // record too large for what is left does not block the block's smaller
        // records.  While some sibling's overshoot is still outstanding the
        // fill word reads above the page size (a record needs between 22,576
        // and 24,576 bytes, so honest claims never pass the page size): the
        // loop waits that out, bounded, before it judges, so a record spills
        // only when the page really has no room for it.
        int32_t* fill = s.fill + (int64_t)layer * s.NB + block;
        const int need = kDenseBytes + plan.var_len;
        const int got = atomicAdd(fill, need);
        if ((int64_t)got + need <= page_bytes) {
          at = got;
        } else {
          atomicSub(fill, need);
          for (int tries = 0; tries < 4096; ++tries) {
            const int seen = *reinterpret_cast<volatile int32_t*>(fill);
            if (seen > page_bytes) continue;  // an overshoot about to be undone
            if ((int64_t)seen + need > page_bytes) break;
            if (atomicCAS(fill, seen, seen + need) == seen) {
              at = seen;
              break;
            }
          }
        }
        if (at < 0) atomicAdd(&s.counters[FP_CTR_SPILLS], 1);
      }
      // One add per closed block-layer (by its first record) instead of one per
      // record: tens of thousands of adds to one address serialise in the L2.
      if (rec == 0) atomicAdd(&s.counters[FP_CTR_ENCODED], 2 * s.H);
    }
    at = __shfl_sync(0xffffffffu, at, 0);
    if (at >= 0) {
      uint8_t* dst = arena + (int64_t)block * page_bytes + at;
      if (lane == 0) {
        s.rec_addr[idx] = reinterpret_cast<int64_t>(dst);
        s.rec_len[idx] = plan.var_len;
      }
      raw = false;
      return dst;
    }
    raw = true;
    const int slot = v.overflow_take_warp((uint32_t)(block * 2 * s.H + rec));
    if (lane == 0) {
      atomicAdd(&s.counters[FP_CTR_FALLBACKS], 1);
      if (slot < 0) atomicAdd(&s.counters[FP_CTR_ERR_OVERFLOW], 1);
    }
    if (slot < 0) return nullptr;
    uint8_t* dst = s.overflow + (int64_t)slot * kRawRecord;
    if (lane == 0) {
      s.rec_addr[idx] = reinterpret_cast<int64_t>(dst);
      s.rec_len[idx] = kRawVarLen;
    }
    return dst;
  });
  // A closing block that donates its slot: the heir's transient record moves
  // in and the heir's table entry follows it.  Every owner overwrites only the
  // words it alone read (and may have read again just above), so no barrier is
  // needed; attention has already read the transient copy.
  const int heir = s.close_list[s.cap + blockIdx.x];
  if (heir >= 0) {
    const uint4* from = reinterpret_cast<const uint4*>(v.staging(s.wslot[heir], layer, rec));
#pragma unroll
    for (int st = 0; st < 8; ++st)
      reinterpret_cast<uint4*>(src)[st * kOwners + tid] = from[st * kOwners + tid];
    if (tid == 0) s.rec_addr[v.table_index(layer, heir, rec)] = reinterpret_cast<int64_t>(src);
  }
}

// Loads a token-major [128,128] BF16 tile (row stride `row_bytes`) into the
// swizzled shared tile with coalesced 16-byte accesses.
__device__ __forceinline__ void tile_load(uint8_t* tile, const uint8_t* src, int64_t row_bytes,
                                          int tid) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int x = q * kOwners + tid, r = x >> 4, ch = x & 15;
    *reinterpret_cast<uint4*>(tile + r * 256 + (((ch ^ r) & 15) << 4)) =
        *reinterpret_cast<const uint4*>(src + r * row_bytes + ch * 16);
  }
}

__device__ __forceinline__ void tile_store(const uint8_t* tile, uint8_t* dst, int64_t row_bytes,
                                           int tid) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int x = q * kOwners + tid, r = x >> 4, ch = x & 15;
    *reinterpret_cast<uint4*>(dst + r * row_bytes + ch * 16) =
        *reinterpret_cast<const uint4*>(tile + r * 256 + (((ch ^ r) & 15) << 4));
  }
}

// Fragment word `st` of owner `o` out of a token-major shared tile.
__device__ __forceinline__ uint4 tile_word(uint8_t* tile, int kv, const OwnerCoords& o, int st) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int j = i >> 1, f = i & 1;
    if (kv == 0) {
      w[i] = *reinterpret_cast<const uint32_t*>(tile_at(tile, o.row(j), o.col(st, f)));
    } else {
      const int tok = o.col(st, f), dim = o.row(j);
      w[i] = (uint32_t)*reinterpret_cast<const uint16_t*>(tile_at(tile, tok, dim)) |
             ((uint32_t)*reinterpret_cast<const uint16_t*>(tile_at(tile, tok + 1, dim)) << 16);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void word_to_tile(uint8_t* tile, int kv, const OwnerCoords& o, int st,
                                             const uint32_t (&w)[4]) {
  // The four registers of word st are the four 8 x 8 pieces (j, f) of an
  // m16n8k16 A fragment, which is also stmatrix's register layout: one
  // instruction stores all four, K pieces as they are (rows = tokens) and V
  // pieces transposed (the fragment's rows are dims).  Lane 8 m + r supplies
  // the address of row r of piece m = 2 j + f: eight scalars, 16 bytes.
  const int lane = (o.g << 2) | o.c;
  const int r = lane & 7, j = (lane >> 4) & 1, f = (lane >> 3) & 1;
  if (kv == 0) {
    const uint32_t at = smem_addr(tile_at(tile, 16 * o.warp + 8 * j + r, 16 * st + 8 * f));
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(at),
                 "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
  } else {
    const uint32_t at = smem_addr(tile_at(tile, 16 * st + 8 * f + r, 16 * o.warp + 8 * j));
    asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(at),
                 "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
  }
}

constexpr int kTileBytes = 128 * 256;

// Batch encoder over token-major records: grid = records.
__global__ void __launch_bounds__(kOwners, 3)
encode_records_kernel(const uint8_t* raw, const uint8_t* rank_of, const int32_t* table_index,
                      const int32_t* kv, uint8_t* out, int64_t out_stride, int32_t* out_len,
                      PipeConsts k) {
  extern __shared__ __align__(16) uint8_t dyn[];
  uint8_t* tile = dyn;
  EncodeShared& sh = *reinterpret_cast<EncodeShared*>(dyn + kTileBytes);
  const int64_t i = blockIdx.x;
  const int tid = threadIdx.x;
  const int which = kv[i];
  load_classes(sh, rank_of + (int64_t)(table_index ? table_index[i] : (int32_t)i) * 256, tid);
  tile_load(tile, raw + i * kRawRecord, 256, tid);
  __syncthreads();
  const OwnerCoords o(tid);
  uint4 wd[8];
#pragma unroll
  for (int st = 0; st < 8; ++st) wd[st] = tile_word(tile, which, o, st);
  const auto reload = [&](int st) { return tile_word(tile, which, o, st); };
  uint8_t* dst = out + i * out_stride;
  encode_cta(wd, sh, tid, k, reload, [&](const EncodePlan& plan, bool& raw_out) -> uint8_t* {
    raw_out = !plan.codes;
    out_len[i] = plan.codes ? kDenseBytes + plan.var_len : kRawRecord;
    return dst;
  });
}

// One record -> token-major rows of `row_bytes` stride starting at `dst`.
__device__ __forceinline__ void decode_to_rows(const uint8_t* rec, int vlen, const HeadTables& tab,
                                               int kv, uint8_t* tile, uint8_t* esc, uint8_t* dst,
                                               int64_t row_bytes, int tid, const PipeConsts& k) {
  const OwnerCoords o(tid);
  auto emit = [&](int st, const uint32_t (&w)[4]) { word_to_tile(tile, kv, o, st, w); };
  if (vlen > kVarCap)
    raw_record_words(rec, tid, emit);
  else
    coded_record_words<true>(rec, vlen, tab, esc, tid, k, [] {}, emit);
  __syncthreads();
  tile_store(tile, dst, row_bytes, tid);
}

constexpr int kDecodeSmem = kTileBytes + kEscBytes;

// ---------------------------------------------------------------------------
// Prefill decompressor (replaces gather_kernel, hbm_kv.cu:452-494): records of
// the listed blocks -> token-major BF16 pages.
//
// Persistent CTAs (two per SM) walk the records r = page * 2 H + rec with a
// stride of the grid.  A producer warp resolves blocks -> rec_addr / rec_len for
// 32 records at a time and streams the coded records through a two-slot ring
// with bulk copies (raw records are read in place after an L2 prefetch), so the
// table look-ups and the record fetch of the next records overlap the decode of
// the current one; eight consumer warps decode a record into the swizzled
// token-major tile and write it out with 16-byte coalesced stores.
// All waits are bounded; a timeout sets bit 0 of g_gather_status.
// ---------------------------------------------------------------------------
constexpr int kGatherSlots = 2;
constexpr int kGatherThreads = kOwners + 32;

__device__ int32_t g_gather_status;

struct GatherSmem {
  __align__(16) uint8_t slots[kGatherSlots][kCodedMax];  // bulk copies need 16-byte alignment
  __align__(16) uint8_t tile[kTileBytes];
  __align__(16) uint8_t esc[kEscBytes];
  __align__(16) HeadTables tabs[kGatherSlots];
  int64_t addr[kGatherSlots];
  int32_t vlen[kGatherSlots];
  __align__(8) uint64_t full[kGatherSlots];
  __align__(8) uint64_t empty[kGatherSlots];
  WaitState wait;
};
static_assert(sizeof(GatherSmem) <= (228 * 1024) / 2 - 1024, "GatherSmem too large for two CTAs per SM");

struct GatherParams {
  const int32_t* blocks;
  const int64_t* rec_addr;
  const int32_t* rec_len;
  const int32_t* plut;
  const uint8_t* slut;
  uint8_t* wk;
  uint8_t* wv;
  int64_t records;  // pages * 2 H
  int H;
  PipeConsts k;
  int32_t* status;        // g_gather_status on this device
  long long wait_limit;   // cycle budget of every bounded wait
  long long skip_record;  // test hook: ordinal of a record the producer leaves out (-1: none)
};

__device__ __forceinline__ void gather_produce(const GatherParams& p, GatherSmem& sm) {
  const int lane = threadIdx.x & 31;
  WaitState* const wait = &sm.wait;
  volatile int* abort = &sm.wait.abort;
  const int per = 2 * p.H;
  uint32_t n = 0;  // records issued so far
  for (int64_t base = blockIdx.x; base < p.records; base += 32LL * gridDim.x) {
    // Lane L resolves the L-th of the next 32 records of this CTA.
    const int64_t r = base + (int64_t)lane * gridDim.x;
    int64_t addr = 0;
    int32_t vlen = 0, rec = 0;
    if (r < p.records) {
      const int64_t page = r / per;
      rec = (int)(r - page * per);
      const int64_t idx = (int64_t)p.blocks[page] * per + rec;
      addr = p.rec_addr[idx];
      vlen = p.rec_len[idx];
    }
    const int64_t left = (p.records - base + gridDim.x - 1) / gridDim.x;
    const int count = (int)(left < 32 ? left : 32);
    for (int j = 0; j < count; ++j) {
      const int64_t a = __shfl_sync(0xffffffffu, addr, j);
      const int32_t v = __shfl_sync(0xffffffffu, vlen, j);
      const int32_t t = __shfl_sync(0xffffffffu, rec, j);
      const uint32_t slot = n % kGatherSlots, use = n / kGatherSlots;
      if (lane == 0) {
        bool ok = true;
        if (use > 0) ok = bounded_wait(&sm.empty[slot], (use - 1) & 1, wait);
        if (ok && (long long)n != p.skip_record) {
          sm.addr[slot] = a;
          sm.vlen[slot] = v;
          sm.tabs[slot] = load_tables(p.plut, p.slut, t);
          if (v > kVarCap || v < kHeaderBytes) {
            prefetch_l2(reinterpret_cast<const void*>(a), kRawRecord);
            mbar_arrive(&sm.full[slot]);
          } else {
            const uint32_t bytes = (uint32_t)(kDenseBytes + (v & ~15));
            mbar_expect_tx(&sm.full[slot], bytes);
            bulk_load(sm.slots[slot], reinterpret_cast<const void*>(a), bytes, &sm.full[slot]);
          }
        }
      }
      ++n;
      __syncwarp();
      if (*abort) return;
    }
  }
}

__device__ __forceinline__ void gather_consume(const GatherParams& p, GatherSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31;
  WaitState* const wait = &sm.wait;
  const int per = 2 * p.H;
  const OwnerCoords o(tid);
  uint32_t n = 0;
  for (int64_t r = blockIdx.x; r < p.records; r += gridDim.x, ++n) {
    const int64_t page = r / per;
    const int rec = (int)(r - page * per);
    const int kv = rec / p.H, head = rec - kv * p.H;
    const uint32_t slot = n % kGatherSlots;
    // A record whose wait ran out is not decoded (its page keeps what the tile
    // held; the status word marks the call invalid).
    const bool landed = bounded_wait(&sm.full[slot], (n / kGatherSlots) & 1, wait);
    const int32_t vlen = sm.vlen[slot];
    auto emit = [&](int st, const uint32_t (&w)[4]) { word_to_tile(sm.tile, kv, o, st, w); };
    auto release = [&] {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.empty[slot]);
    };
    if (!landed) {
    } else if (vlen > kVarCap || vlen < kHeaderBytes) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(sm.addr[slot]);
      release();
      raw_record_words(src, tid, emit);
    } else {
      const HeadTables tab = sm.tabs[slot];
      coded_record_words(sm.slots[slot], vlen, tab, sm.esc, tid, p.k, release, emit);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kOwners) : "memory");  // tile complete
    uint8_t* dst = (kv == 0 ? p.wk : p.wv) + (page * 128 * p.H + head) * 256;
    tile_store(sm.tile, dst, (int64_t)p.H * 256, tid);
    asm volatile("bar.sync 1, %0;" ::"n"(kOwners) : "memory");  // tile and escape scratch free
  }
}

__global__ void __launch_bounds__(kGatherThreads, 2) gather_kernel(GatherParams p) {
  extern __shared__ __align__(16) uint8_t dyn[];
  GatherSmem& sm = *reinterpret_cast<GatherSmem*>(dyn);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGatherSlots; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kOwners / 32);
    }
    sm.wait.abort = 0;
    sm.wait.status = p.status;
    sm.wait.limit = p.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x >= kOwners) {
    gather_produce(p, sm);
  } else {
    gather_consume(p, sm);
  }
  // Nothing may still be writing this CTA's shared memory when it exits (see
  // decode_attn_kernel): after a timeout give copies in flight time to land.
  __syncthreads();
  if (sm.wait.abort && threadIdx.x == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 20000000LL) {
    }
  }
}

// Batch decoder: grid = records.
__global__ void __launch_bounds__(kOwners)
decode_records_kernel(const uint8_t* recs, int64_t rec_stride, const int32_t* rec_len,
                      const int32_t* plut, const uint8_t* slut, const int32_t* table_index,
                      const int32_t* kv, uint8_t* out, PipeConsts k) {
  extern __shared__ __align__(16) uint8_t dyn[];
  const int64_t i = blockIdx.x;
  const HeadTables tab = load_tables(plut, slut, table_index ? table_index[i] : (int32_t)i);
  decode_to_rows(recs + i * rec_stride, rec_len[i], tab, kv[i], dyn, dyn + kTileBytes,
                 out + i * kRawRecord, 256, threadIdx.x, k);
}

}  // namespace
}  // namespace fpb

using namespace fpb;

extern "C" {

const char* fp_last_error(void) { return last_error(); }

const char* fp_version(void) { return "fragpack_b200 0.1.0 (sm_100a)"; }

int fp_hbm_write(const fp_store* store, const void* key, int64_t k_stride0, int64_t k_stride1,
                 const void* value, int64_t v_stride0, int64_t v_stride1,
                 const int64_t* slot_mapping, int64_t num_tokens, int32_t layer, void* stream) {
  if (int rc = check_store(store)) return rc;
  if (num_tokens == 0) return FP_OK;
  FP_REQUIRE(key && value && slot_mapping, "null key / value / slot_mapping");
  FP_REQUIRE(layer >= 0 && layer < store->L, "layer %d out of range", layer);
  FP_REQUIRE((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) % 4 == 0 &&
                 (k_stride0 | k_stride1 | v_stride0 | v_stride1) % 2 == 0,
             "key / value rows must be 4-byte aligned");
  StoreView v{*store};
  // 16-byte row loads need aligned bases and strides; otherwise every token
  // takes the scattered path.
  const int vector_ok =
      (reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) % 16 == 0 &&
      (k_stride0 | k_stride1 | v_stride0 | v_stride1) % 8 == 0;
  const dim3 grid((unsigned)((num_tokens + 15) / 16),
                  (unsigned)((store->H + kWriteHeads - 1) / kWriteHeads));
  write_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      v, static_cast<const uint16_t*>(key), static_cast<const uint16_t*>(value), k_stride0,
      k_stride1, v_stride0, v_stride1, slot_mapping, num_tokens, layer, vector_ok);
  FP_LAUNCH_CHECK("write_kernel");
  return FP_OK;
}

int fp_hbm_encode(const fp_store* store, const uint8_t* rank_of, int32_t layer, uint8_t* arena,
                  int64_t page_bytes, int64_t max_close, void* stream) {
  if (int rc = check_store(store)) return rc;
  if (max_close == 0) return FP_OK;
  FP_REQUIRE(max_close > 0 && max_close <= store->cap, "close list too small");
  FP_REQUIRE(rank_of && arena, "null rank_of / arena");
  FP_REQUIRE(layer >= 0 && layer < store->L, "layer %d out of range", layer);
  FP_REQUIRE(page_bytes % 16 == 0 && page_bytes > 0 && page_bytes < (1LL << 31),
             "bad arena page size %lld", (long long)page_bytes);
  FP_REQUIRE(reinterpret_cast<uintptr_t>(arena) % 16 == 0, "arena must be 16-byte aligned");
  StoreView v{*store};
  encode_kernel<<<dim3((unsigned)max_close, 2 * store->H), kOwners, 0, (cudaStream_t)stream>>>(
      v, layer, arena, page_bytes, rank_of, pipe_consts());
  FP_LAUNCH_CHECK("encode_kernel");
  return FP_OK;
}

int fp_hbm_gather(const int32_t* blocks, int64_t n, const int64_t* rec_addr,
                  const int32_t* rec_len, const int32_t* plut, const uint8_t* slut, void* wk,
                  void* wv, int64_t workspace_bytes, int32_t kv_heads, void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(n > 0 && blocks && rec_addr && rec_len && plut && slut && wk && wv,
             "null gather argument");
  FP_REQUIRE(kv_heads > 0 && 2 * kv_heads <= 65535, "bad kv_heads %d", kv_heads);
  FP_REQUIRE(workspace_bytes >= n * 128 * (int64_t)kv_heads * 256, "workspace too small");
  FP_REQUIRE((reinterpret_cast<uintptr_t>(wk) | reinterpret_cast<uintptr_t>(wv)) % 16 == 0,
             "workspace must be 16-byte aligned");
  static std::atomic<uint64_t> smem_allowed;
  if (int rc = allow_dynamic_smem(gather_kernel, (int)sizeof(GatherSmem), smem_allowed)) return rc;
  GatherParams p;
  p.blocks = blocks;
  p.rec_addr = rec_addr;
  p.rec_len = rec_len;
  p.plut = plut;
  p.slut = slut;
  p.wk = static_cast<uint8_t*>(wk);
  p.wv = static_cast<uint8_t*>(wv);
  p.records = n * 2 * kv_heads;
  p.H = kv_heads;
  p.k = pipe_consts();
  void* status_word = nullptr;
  if (int rc = cuda_status(cudaGetSymbolAddress(&status_word, g_gather_status),
                           "cudaGetSymbolAddress(g_gather_status)"))
    return rc;
  p.status = static_cast<int32_t*>(status_word);
  p.wait_limit = wait_debug().limit;
  p.skip_record = wait_debug().skip_record;
  const int64_t resident = 2LL * device_sms();
  const unsigned grid = (unsigned)(p.records < resident ? p.records : resident);
  gather_kernel<<<grid, kGatherThreads, sizeof(GatherSmem), (cudaStream_t)stream>>>(p);
  FP_LAUNCH_CHECK("gather_kernel");
  return FP_OK;
}

int fp_hbm_gather_status(int32_t* status) {
  FP_REQUIRE(status, "null status");
  if (int rc = cuda_status(cudaMemcpyFromSymbol(status, g_gather_status, sizeof(int32_t)),
                           "cudaMemcpyFromSymbol(g_gather_status)"))
    return rc;
  // Reading clears: the word reports the calls since the previous read.
  const int32_t zero = 0;
  return cuda_status(cudaMemcpyToSymbol(g_gather_status, &zero, sizeof(int32_t)),
                     "cudaMemcpyToSymbol(g_gather_status)");
}

int fp_debug_wait_limit(int64_t cycles, int64_t skip_record) {
  FP_REQUIRE(cycles >= 0, "negative wait limit");
  g_wait_limit.store(cycles > 0 ? cycles : kWaitCycles, std::memory_order_relaxed);
  g_skip_record.store(skip_record, std::memory_order_relaxed);
  return FP_OK;
}

int fp_encode_records(const void* raw, int64_t n, const uint8_t* rank_of,
                      const int32_t* table_index, const int32_t* kv, uint8_t* out,
                      int64_t out_stride, int32_t* out_len, void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(n > 0 && n < (1LL << 31) && raw && rank_of && kv && out && out_len,
             "null encode argument");
  FP_REQUIRE(out_stride >= kRawRecord && out_stride % 16 == 0, "bad out_stride %lld",
             (long long)out_stride);
  FP_REQUIRE((reinterpret_cast<uintptr_t>(raw) | reinterpret_cast<uintptr_t>(out)) % 16 == 0,
             "buffers must be 16-byte aligned");
  constexpr int smem = kTileBytes + (int)sizeof(EncodeShared);
  static std::atomic<uint64_t> smem_allowed;
  if (int rc = allow_dynamic_smem(encode_records_kernel, smem, smem_allowed)) return rc;
  encode_records_kernel<<<(unsigned)n, kOwners, smem, (cudaStream_t)stream>>>(
      static_cast<const uint8_t*>(raw), rank_of, table_index, kv, out, out_stride, out_len,
      pipe_consts());
  FP_LAUNCH_CHECK("encode_records_kernel");
  return FP_OK;
}

int fp_decode_records(const uint8_t* recs, int64_t rec_stride, const int32_t* rec_len, int64_t n,
                      const int32_t* plut, const uint8_t* slut, const int32_t* table_index,
                      const int32_t* kv, void* out, void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(n > 0 && n < (1LL << 31) && recs && rec_len && plut && slut && kv && out,
             "null decode argument");
  FP_REQUIRE(rec_stride % 16 == 0 && rec_stride >= kDenseBytes + kHeaderBytes,
             "bad rec_stride %lld", (long long)rec_stride);
  FP_REQUIRE((reinterpret_cast<uintptr_t>(recs) | reinterpret_cast<uintptr_t>(out)) % 16 == 0,
             "buffers must be 16-byte aligned");
  static std::atomic<uint64_t> smem_allowed;
  if (int rc = allow_dynamic_smem(decode_records_kernel, kDecodeSmem, smem_allowed)) return rc;
  decode_records_kernel<<<(unsigned)n, kOwners, kDecodeSmem, (cudaStream_t)stream>>>(
      recs, rec_stride, rec_len, plut, slut, table_index, kv, static_cast<uint8_t*>(out),
      pipe_consts());
  FP_LAUNCH_CHECK("decode_records_kernel");
  return FP_OK;
}

}  // extern "C"
