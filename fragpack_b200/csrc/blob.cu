// Block blobs: one closed block's records as a self-describing byte string for
// external tiers (fragpack/ops/hbm_kv.cu:496-665, format attn_page.py:72-78).
//
//   [0,64)    u32 magic "FPKB", u32 version 1, u32 L, u32 H, i64 bytes, i64 digest
//   [64, ..)  i32 rec_len[L, 2, H]; the head is padded to a 4096 multiple
//   records   in (layer, kv, head) order, each 22528 + rec_len bytes
#include "fp_api.h"
#include "fp_common.cuh"

namespace fpb {
namespace {

constexpr uint32_t kMagic = 0x424B5046u;
constexpr uint32_t kVersion = 1;
constexpr int kFixed = 64;
constexpr int64_t kAlign = 4096;
constexpr int kMaxHeads = 16;
constexpr int kBlobThreads = 256;

__host__ __device__ __forceinline__ int64_t head_bytes(int L, int H) {
  return (kFixed + 8LL * L * H + kAlign - 1) / kAlign * kAlign;
}

__device__ __forceinline__ bool length_ok(int v) {
  return v == kRawVarLen || (v >= kHeaderBytes && v <= kVarCap && (v & 15) == 0);
}

// Block-wide sums of two 64-bit values.
__device__ __forceinline__ void block_sum2(long long& a, long long& b, long long (*red)[2]) {
#pragma unroll
  for (int x = 16; x; x >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, x);
    b += __shfl_xor_sync(0xffffffffu, b, x);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    red[threadIdx.x >> 5][0] = a;
    red[threadIdx.x >> 5][1] = b;
  }
  __syncthreads();
  a = b = 0;
#pragma unroll
  for (int w = 0; w < kBlobThreads / 32; ++w) {
    a += red[w][0];
    b += red[w][1];
  }
}

__device__ __forceinline__ void copy16(uint8_t* dst, const uint8_t* src, int bytes, int tid) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (int q = tid; q < bytes / 16; q += kBlobThreads) d[q] = s[q];
}

// grid (n, L): CTA (i, l) copies layer l's records of blocks[i]; layer 0 also
// writes the head and lengths[i].
__global__ void __launch_bounds__(kBlobThreads)
export_kernel(const int32_t* blocks, const int64_t* rec_addr, const int32_t* rec_len, uint8_t* out,
              int64_t stride, int64_t* lengths, int L, int H, int NB, int64_t digest) {
  __shared__ long long red[kBlobThreads / 32][2];
  const int i = blockIdx.x, layer = blockIdx.y, tid = threadIdx.x, per = 2 * H;
  const int block = blocks[i];
  long long before = 0, total = 0;
  for (int x = tid; x < L * per; x += kBlobThreads) {
    const long long n = kDenseBytes + rec_len[((int64_t)(x / per) * NB + block) * per + x % per];
    total += n;
    if (x / per < layer) before += n;
  }
  block_sum2(before, total, red);
  const int64_t head = head_bytes(L, H);
  uint8_t* blob = out + (int64_t)i * stride;
  if (layer == 0) {
    if (tid == 0) {
      uint32_t* h32 = reinterpret_cast<uint32_t*>(blob);
      h32[0] = kMagic;
      h32[1] = kVersion;
      h32[2] = (uint32_t)L;
      h32[3] = (uint32_t)H;
      int64_t* h64 = reinterpret_cast<int64_t*>(blob + 16);
      h64[0] = head + total;
      h64[1] = digest;
      lengths[i] = (head + total + kAlign - 1) / kAlign * kAlign;
    }
    int32_t* table = reinterpret_cast<int32_t*>(blob + kFixed);
    for (int x = tid; x < L * per; x += kBlobThreads)
      table[x] = rec_len[((int64_t)(x / per) * NB + block) * per + x % per];
  }
  int64_t at = head + before;
  for (int rec = 0; rec < per; ++rec) {
    const int64_t idx = ((int64_t)layer * NB + block) * per + rec;
    const int n = kDenseBytes + rec_len[idx];
    copy16(blob + at, reinterpret_cast<const uint8_t*>(rec_addr[idx]), n, tid);
    at += n;
  }
}

struct ImportView {
  fp_store s;
  __device__ int take(uint32_t hint) const {
    for (int i = 0; i < s.ovf_words; ++i) {
      const int w = (int)((hint + (uint32_t)i) % (uint32_t)s.ovf_words);
      uint32_t seen = *reinterpret_cast<volatile uint32_t*>(&s.ovf_bits[w]);
      while (seen != 0xffffffffu) {
        const uint32_t bit = 1u << (__ffs(~seen) - 1);
        const uint32_t before = atomicOr(&s.ovf_bits[w], bit);
        if (!(before & bit)) return 32 * w + (__ffs(bit) - 1);
        seen = before | bit;
      }
    }
    return -1;
  }
  __device__ void give_back(int64_t addr) const {
    const int64_t base = reinterpret_cast<int64_t>(s.overflow);
    if (addr < base || addr >= base + s.overflow_records * kRawRecord) return;
    const int slot = (int)((addr - base) / kRawRecord);
    atomicAnd(&s.ovf_bits[slot >> 5], ~(1u << (slot & 31)));
  }
};

// grid (n, L): CTA (i, l) validates blob i and installs its layer-l records
// for blocks[i].  Every CTA validates the whole head so that all layers agree;
// a failure sets status[i] and leaves that layer's tables untouched.
__global__ void __launch_bounds__(kBlobThreads)
import_kernel(ImportView v, const uint8_t* src, int64_t src_bytes, const int64_t* offsets,
              const int32_t* blocks, int32_t* status, const int64_t* arena_base,
              const int64_t* arena_stride, int64_t digest) {
  __shared__ long long red[kBlobThreads / 32][2];
  __shared__ int64_t from_at[2 * kMaxHeads], to_at[2 * kMaxHeads];
  __shared__ int failed;
  const fp_store& s = v.s;
  const int i = blockIdx.x, layer = blockIdx.y, tid = threadIdx.x, per = 2 * s.H;
  const int block = blocks[i];
  const int64_t off = offsets[i], head = head_bytes(s.L, s.H);
  if (off < 0 || (off & 15) || off + head > src_bytes) {
    if (tid == 0) atomicOr(&status[i], FP_BLOB_BAD_HEADER);
    return;
  }
  const uint8_t* blob = src + off;
  const uint32_t* h32 = reinterpret_cast<const uint32_t*>(blob);
  const int64_t* h64 = reinterpret_cast<const int64_t*>(blob + 16);
  const int64_t declared = h64[0];
  if (h32[0] != kMagic || h32[1] != kVersion || (int)h32[2] != s.L || (int)h32[3] != s.H ||
      h64[1] != digest || declared < head || off + declared > src_bytes) {
    if (tid == 0) atomicOr(&status[i], FP_BLOB_BAD_HEADER);
    return;
  }
  const int32_t* table = reinterpret_cast<const int32_t*>(blob + kFixed);
  long long before = 0, total = 0;
  int bad = 0;
  for (int x = tid; x < s.L * per; x += kBlobThreads) {
    const int len = table[x];
    const bool ok = length_ok(len);
    bad |= !ok;
    const long long n = kDenseBytes + (ok ? len : 0);
    total += n;
    if (x / per < layer) before += n;
  }
  bad = __syncthreads_or(bad);
  block_sum2(before, total, red);
  if (bad || head + total != declared) {
    if (tid == 0) atomicOr(&status[i], FP_BLOB_BAD_LENGTHS);
    return;
  }
  const int32_t* lens = table + layer * per;
  if (tid == 0) {
    const int64_t page = arena_stride[layer];
    const int64_t page_at = arena_base[layer] + (int64_t)block * page;
    int64_t from = head + before;
    int fill = 0, placed = 0;
    for (; placed < per; ++placed) {
      const int n = kDenseBytes + lens[placed];
      int64_t to;
      if (lens[placed] != kRawVarLen && fill + n <= page) {
        to = page_at + fill;
        fill += n;
      } else {
        const int slot = v.take((uint32_t)(block * per + placed));
        if (slot < 0) break;
        to = reinterpret_cast<int64_t>(s.overflow) + (int64_t)slot * kRawRecord;
      }
      from_at[placed] = from;
      to_at[placed] = to;
      from += n;
    }
    failed = placed < per;
    if (failed) {
      for (int k = 0; k < placed; ++k) v.give_back(to_at[k]);
      atomicOr(&status[i], FP_BLOB_NO_OVERFLOW);
    } else {
      s.fill[(int64_t)layer * s.NB + block] = fill;
    }
  }
  __syncthreads();
  if (failed) return;
  for (int rec = 0; rec < per; ++rec)
    copy16(reinterpret_cast<uint8_t*>(to_at[rec]), blob + from_at[rec], kDenseBytes + lens[rec], tid);
  __syncthreads();
  if (tid < per) {
    // Old overflow records are released only after the new ones are placed.
    const int64_t idx = ((int64_t)layer * s.NB + block) * per + tid;
    v.give_back(s.rec_addr[idx]);
    s.rec_addr[idx] = to_at[tid];
    s.rec_len[idx] = lens[tid];
  }
}

}  // namespace
}  // namespace fpb

using namespace fpb;

extern "C" {

int fp_hbm_export(const int32_t* blocks, int64_t n, const int64_t* rec_addr,
                  const int32_t* rec_len, uint8_t* out, int64_t out_bytes, int64_t stride,
                  int64_t* lengths, int32_t L, int32_t H, int32_t NB, int64_t digest,
                  void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(n > 0 && blocks && rec_addr && rec_len && out && lengths, "null export argument");
  FP_REQUIRE(L > 0 && H > 0 && NB > 0 && L <= 65535, "bad export geometry");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0,
             "export buffer must be contiguous 16-byte aligned uint8");
  FP_REQUIRE(stride % 16 == 0 && stride >= head_bytes(L, H) + 2LL * L * H * kRawRecord &&
                 out_bytes >= n * stride,
             "export stride or buffer too small");
  export_kernel<<<dim3((unsigned)n, L), kBlobThreads, 0, (cudaStream_t)stream>>>(
      blocks, rec_addr, rec_len, out, stride, lengths, L, H, NB, digest);
  FP_LAUNCH_CHECK("export_kernel");
  return FP_OK;
}

int fp_hbm_import(const fp_store* store, const uint8_t* src, int64_t src_bytes,
                  const int64_t* offsets, const int32_t* blocks, int64_t n, int32_t* status,
                  const int64_t* arena_base, const int64_t* arena_stride, int64_t digest,
                  void* stream) {
  if (n == 0) return FP_OK;
  FP_REQUIRE(store && n > 0 && src && offsets && blocks && status && arena_base && arena_stride,
             "null import argument");
  FP_REQUIRE(store->H <= kMaxHeads, "too many KV heads (%d > %d)", store->H, kMaxHeads);
  FP_REQUIRE(store->L > 0 && store->L <= 65535, "bad layer count");
  FP_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0,
             "import buffer must be contiguous 16-byte aligned uint8");
  ImportView v{*store};
  import_kernel<<<dim3((unsigned)n, store->L), kBlobThreads, 0, (cudaStream_t)stream>>>(
      v, src, src_bytes, offsets, blocks, status, arena_base, arena_stride, digest);
  FP_LAUNCH_CHECK("import_kernel");
  return FP_OK;
}

}  // extern "C"
