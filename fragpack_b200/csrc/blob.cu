// Block blobs: one closed block's records as a self-describing byte string for
// external tiers.  Same bytes as the reference's export / import
// (fragpack/ops/hbm_kv.cu:496-665, format attn_page.py:72-78):
//
//   [0,64)    u32 magic "FPKB", u32 version 1, u32 L, u32 H, i64 bytes, i64 digest
//   [64, ..)  i32 rec_len[L, 2, H]; the head is padded to a 4096 multiple
//   records   in (layer, kv, head) order, each 22528 + rec_len bytes
//
// Both directions run as a layout pass followed by a copy pass:
//  * the layout pass (one CTA per blob) sums the record lengths ONCE with a
//    block-wide scan, writes or validates the head, and leaves every record's
//    offset in the blob in a scratch table; for an import a second small pass
//    (one warp per blob and layer) decides where each record goes - its
//    block's page while it fits, else an overflow slot - and takes the slots;
//  * the copy pass runs one CTA per record, so the copy of one blob is spread
//    over L * 2H CTAs whatever the geometry (any number of KV heads).
#include "fp_api.h"
#include "fp_common.cuh"
#include "fp_store.cuh"

namespace fpb {
namespace {

constexpr uint32_t kMagic = 0x424B5046u;
constexpr uint32_t kVersion = 1;
constexpr int kFixed = 64;
constexpr int64_t kAlign = 4096;
constexpr int kLayoutThreads = 256;
constexpr int kCopyThreads = 256;

__host__ __device__ __forceinline__ int64_t head_bytes(int L, int H) {
  return (kFixed + 8LL * L * H + kAlign - 1) / kAlign * kAlign;
}

__device__ __forceinline__ bool length_ok(int v) {
  return v == kRawVarLen || (v >= kHeaderBytes && v <= kVarCap && (v & 15) == 0);
}

// Exclusive prefix sum of `v` over a CTA of kLayoutThreads threads; `total`
// receives the sum.
__device__ __forceinline__ long long block_exclusive(long long v, long long& total,
                                                     long long* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const long long t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  __syncthreads();  // the previous round's readers are done
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  long long before = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < kLayoutThreads / 32; ++w) {
    if (w < warp) before += warp_sums[w];
    total += warp_sums[w];
  }
  return before + inc - v;
}

// Copies `bytes` (a 16-byte multiple, both ends 16-byte aligned) with the CTA.
__device__ __forceinline__ void copy_record(uint8_t* dst, const uint8_t* src, int bytes) {
  const uint4* from = reinterpret_cast<const uint4*>(src);
  uint4* to = reinterpret_cast<uint4*>(dst);
  const int n = bytes >> 4;
  // Four loads in flight per thread before the first store.
  for (int q = threadIdx.x; q < n; q += 4 * kCopyThreads) {
    uint4 v[4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
      if (q + x * kCopyThreads < n) v[x] = from[q + x * kCopyThreads];
#pragma unroll
    for (int x = 0; x < 4; ++x)
      if (q + x * kCopyThreads < n) to[q + x * kCopyThreads] = v[x];
  }
}

// ---------------------------------------------------------------------------
// Export
// ---------------------------------------------------------------------------
// grid n: blob i's head, its length, and offsets[i, r] of each of its records.
__global__ void __launch_bounds__(kLayoutThreads)
export_layout_kernel(const int32_t* blocks, const int32_t* rec_len, uint8_t* out, int64_t stride,
                     int64_t* lengths, int64_t* offsets, int L, int H, int NB, int64_t digest) {
  __shared__ long long warp_sums[kLayoutThreads / 32];
  const int i = blockIdx.x, tid = threadIdx.x, per = 2 * H, records = L * per;
  const int block = blocks[i];
  uint8_t* blob = out + (int64_t)i * stride;
  int32_t* table = reinterpret_cast<int32_t*>(blob + kFixed);
  long long at = head_bytes(L, H);
  for (int base = 0; base < records; base += kLayoutThreads) {
    const int r = base + tid;
    int len = 0;
    if (r < records) {
      len = rec_len[((int64_t)(r / per) * NB + block) * per + r % per];
      table[r] = len;
    }
    long long tile;
    const long long before = block_exclusive(r < records ? kDenseBytes + len : 0, tile, warp_sums);
    if (r < records) offsets[(int64_t)i * records + r] = at + before;
    at += tile;
  }
  if (tid == 0) {
    uint32_t* h32 = reinterpret_cast<uint32_t*>(blob);
    h32[0] = kMagic;
    h32[1] = kVersion;
    h32[2] = (uint32_t)L;
    h32[3] = (uint32_t)H;
    int64_t* h64 = reinterpret_cast<int64_t*>(blob + 16);
    h64[0] = at;
    h64[1] = digest;
    lengths[i] = (at + kAlign - 1) / kAlign * kAlign;
  }
}

// grid (L * 2H, n): one record each.
__global__ void __launch_bounds__(kCopyThreads)
export_copy_kernel(const int32_t* blocks, const int64_t* rec_addr, const int32_t* rec_len,
                   uint8_t* out, int64_t stride, const int64_t* offsets, int L, int H, int NB) {
  const int r = blockIdx.x, i = blockIdx.y, per = 2 * H;
  const int64_t idx = ((int64_t)(r / per) * NB + blocks[i]) * per + r % per;
  copy_record(out + (int64_t)i * stride + offsets[(int64_t)i * L * per + r],
              reinterpret_cast<const uint8_t*>(rec_addr[idx]), kDenseBytes + rec_len[idx]);
}

// ---------------------------------------------------------------------------
// Import
// ---------------------------------------------------------------------------
// Per blob and record: where the record sits in the source buffer and where it
// goes (0: its layer was not installed).
struct ImportPlan {
  int64_t* from;  // [n, L * 2H] absolute source addresses
  int64_t* to;    // [n, L * 2H] absolute destination addresses
};

// grid n: validates blob i as a whole (so that all of its layers agree) and
// lists its records' source addresses.  A failure sets status[i]; the later
// passes leave such a blob alone.
__global__ void __launch_bounds__(kLayoutThreads)
import_layout_kernel(const uint8_t* src, int64_t src_bytes, const int64_t* offsets,
                     int32_t* status, ImportPlan plan, int L, int H, int64_t digest) {
  __shared__ long long warp_sums[kLayoutThreads / 32];
  const int i = blockIdx.x, tid = threadIdx.x, records = L * 2 * H;
  const int64_t off = offsets[i], head = head_bytes(L, H);
  for (int r = tid; r < records; r += kLayoutThreads) plan.to[(int64_t)i * records + r] = 0;
  if (off < 0 || (off & 15) || off + head > src_bytes) {
    if (tid == 0) atomicOr(&status[i], FP_BLOB_BAD_HEADER);
    return;
  }
  const uint8_t* blob = src + off;
  const uint32_t* h32 = reinterpret_cast<const uint32_t*>(blob);
  const int64_t* h64 = reinterpret_cast<const int64_t*>(blob + 16);
  const int64_t declared = h64[0];
  if (h32[0] != kMagic || h32[1] != kVersion || (int)h32[2] != L || (int)h32[3] != H ||
      h64[1] != digest || declared < head || off + declared > src_bytes) {
    if (tid == 0) atomicOr(&status[i], FP_BLOB_BAD_HEADER);
    return;
  }
  const int32_t* table = reinterpret_cast<const int32_t*>(blob + kFixed);
  long long at = head;
  int bad = 0;
  for (int base = 0; base < records; base += kLayoutThreads) {
    const int r = base + tid;
    int len = 0;
    if (r < records) {
      len = table[r];
      if (!length_ok(len)) {
        bad = 1;
        len = 0;
      }
    }
    long long tile;
    const long long before = block_exclusive(r < records ? kDenseBytes + len : 0, tile, warp_sums);
    if (r < records) plan.from[(int64_t)i * records + r] = reinterpret_cast<int64_t>(blob) + at + before;
    at += tile;
  }
  bad = __syncthreads_or(bad);
  if ((bad || at != declared) && tid == 0) atomicOr(&status[i], FP_BLOB_BAD_LENGTHS);
}

// grid (L, n), one warp: places layer `layer` of blob i.  Coded records go into
// the block's page in record order while they fit; raw records, and coded ones
// that no longer fit, take overflow slots.  If the pool runs out the layer
// takes nothing and keeps its old records (status bit FP_BLOB_NO_OVERFLOW).
__global__ void __launch_bounds__(32)
import_place_kernel(StoreView v, const uint8_t* src, const int64_t* offsets, const int32_t* blocks,
                    int32_t* status, ImportPlan plan, const int64_t* arena_base,
                    const int64_t* arena_stride) {
  const fp_store& s = v.s;
  const int layer = blockIdx.x, i = blockIdx.y, lane = threadIdx.x, per = 2 * s.H;
  if (status[i] & (FP_BLOB_BAD_HEADER | FP_BLOB_BAD_LENGTHS)) return;
  const int block = blocks[i];
  const int32_t* lens =
      reinterpret_cast<const int32_t*>(src + offsets[i] + kFixed) + (int64_t)layer * per;
  const int64_t page = arena_stride[layer];
  const int64_t page_at = arena_base[layer] + (int64_t)block * page;
  int64_t* to = plan.to + ((int64_t)i * s.L + layer) * per;

  // Pass 1: page offsets, tile by tile in record order.  A record that does
  // not fit is set aside and the tile is ranked again without it (at most once
  // per record), so smaller records behind it still get their place.
  int fill = 0;
  for (int base = 0; base < per; base += 32) {
    const int r = base + lane;
    const int len = r < per ? lens[r] : kRawVarLen;
    const int need = kDenseBytes + len;
    bool paged = r < per && len != kRawVarLen;
    int at = 0;
    for (int round = 0; round <= 32; ++round) {
      int inc = paged ? need : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
      }
      at = fill + inc - (paged ? need : 0);
      const uint32_t over = __ballot_sync(0xffffffffu, paged && at + need > page);
      if (over == 0) {
        fill += __shfl_sync(0xffffffffu, inc, 31);
        break;
      }
      if (lane == __ffs(over) - 1) paged = false;
    }
    if (r < per) to[r] = paged ? page_at + at : -1;  // -1: wants an overflow slot
  }
  __syncwarp();
  // Pass 2: overflow slots, each lane for its own records.
  bool short_of_slots = false;
  for (int r = lane; r < per; r += 32) {
    if (to[r] != -1) continue;
    const int slot = v.overflow_take((uint32_t)(block * per + r));
    if (slot < 0) {
      short_of_slots = true;
      to[r] = 0;
    } else {
      to[r] = reinterpret_cast<int64_t>(s.overflow) + (int64_t)slot * kRawRecord;
    }
  }
  if (__any_sync(0xffffffffu, short_of_slots)) {
    for (int r = lane; r < per; r += 32) {
      v.overflow_give_back(to[r]);
      to[r] = 0;
    }
    if (lane == 0) atomicOr(&status[i], FP_BLOB_NO_OVERFLOW);
  } else if (lane == 0) {
    s.fill[(int64_t)layer * s.NB + block] = fill;
  }
}

// grid (L * 2H, n): copies one record to its place and then repoints the
// block's table entry at it; an overflow slot the entry held before is
// returned only now, after the new record is in place.
__global__ void __launch_bounds__(kCopyThreads)
import_copy_kernel(StoreView v, const uint8_t* src, const int64_t* offsets, const int32_t* blocks,
                   ImportPlan plan) {
  const fp_store& s = v.s;
  const int r = blockIdx.x, i = blockIdx.y, per = 2 * s.H;
  const int64_t entry = (int64_t)i * s.L * per + r;
  const int64_t to = plan.to[entry];
  if (to == 0) return;
  const int len = reinterpret_cast<const int32_t*>(src + offsets[i] + kFixed)[r];
  copy_record(reinterpret_cast<uint8_t*>(to), reinterpret_cast<const uint8_t*>(plan.from[entry]),
              kDenseBytes + len);
  __syncthreads();
  if (threadIdx.x == 0) {
    const int64_t idx = ((int64_t)(r / per) * s.NB + blocks[i]) * per + r % per;
    v.overflow_give_back(s.rec_addr[idx]);
    s.rec_addr[idx] = to;
    s.rec_len[idx] = len;
  }
}

}  // namespace
}  // namespace fpb

using namespace fpb;

extern "C" {

int fp_hbm_export(const int32_t* blocks, int64_t n, const int64_t* rec_addr,
                  const int32_t* rec_len, uint8_t* out, int64_t out_bytes, int64_t stride,
                  int64_t* lengths, int64_t* scratch, int32_t L, int32_t H, int32_t NB,
                  int64_t digest, void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(n > 0 && n <= 65535 && blocks && rec_addr && rec_len && out && lengths && scratch,
             "null export argument");
  FP_REQUIRE(L > 0 && H > 0 && NB > 0 && (int64_t)L * 2 * H < (1LL << 31), "bad export geometry");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0,
             "export buffer must be contiguous 16-byte aligned uint8");
  FP_REQUIRE(stride % 16 == 0 && stride >= head_bytes(L, H) + 2LL * L * H * kRawRecord &&
                 out_bytes >= n * stride,
             "export stride or buffer too small");
  cudaStream_t st = (cudaStream_t)stream;
  export_layout_kernel<<<(unsigned)n, kLayoutThreads, 0, st>>>(blocks, rec_len, out, stride,
                                                               lengths, scratch, L, H, NB, digest);
  FP_LAUNCH_CHECK("export_layout_kernel");
  export_copy_kernel<<<dim3((unsigned)(L * 2 * H), (unsigned)n), kCopyThreads, 0, st>>>(
      blocks, rec_addr, rec_len, out, stride, scratch, L, H, NB);
  FP_LAUNCH_CHECK("export_copy_kernel");
  return FP_OK;
}

int fp_hbm_import(const fp_store* store, const uint8_t* src, int64_t src_bytes,
                  const int64_t* offsets, const int32_t* blocks, int64_t n, int32_t* status,
                  int64_t* scratch, const int64_t* arena_base, const int64_t* arena_stride,
                  int64_t digest, void* stream) {
  if (n == 0) return FP_OK;
  if (int rc = check_store(store)) return rc;
  FP_REQUIRE(n > 0 && n <= 65535 && src && offsets && blocks && status && scratch && arena_base &&
                 arena_stride,
             "null import argument");
  FP_REQUIRE(store->L <= 65535, "bad layer count");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0,
             "import buffer must be contiguous 16-byte aligned uint8");
  StoreView v{*store};
  const int64_t records = (int64_t)store->L * 2 * store->H;
  ImportPlan plan{scratch, scratch + n * records};
  cudaStream_t st = (cudaStream_t)stream;
  import_layout_kernel<<<(unsigned)n, kLayoutThreads, 0, st>>>(src, src_bytes, offsets, status, plan,
                                                               store->L, store->H, digest);
  FP_LAUNCH_CHECK("import_layout_kernel");
  import_place_kernel<<<dim3((unsigned)store->L, (unsigned)n), 32, 0, st>>>(
      v, src, offsets, blocks, status, plan, arena_base, arena_stride);
  FP_LAUNCH_CHECK("import_place_kernel");
  import_copy_kernel<<<dim3((unsigned)records, (unsigned)n), kCopyThreads, 0, st>>>(v, src, offsets,
                                                                                    blocks, plan);
  FP_LAUNCH_CHECK("import_copy_kernel");
  return FP_OK;
}

}  // extern "C"
