/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 *
 * CPU restatement (plain C) of the FragPack record codec, used only as the
 * checker in tests, in the smoke check and as the timed CPU baseline of the
 * benchmark.  Nothing under fragpack_b200/ may link, import or call it.
 *
 * Every function cites the reference file:line it restates (paths relative
 * to the reference project root).  The restatement is pinned against the
 * reference implementation by committed golden vectors that were produced by
 * importing the reference codec (tests/golden/make_golden.py).
 *
 * Record geometry (fragpack/compression/attn_page.py:51-71):
 *   128 tokens x 128 dims BF16 = 16384 scalars, 256 virtual threads x 64.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define PAGE_TOKENS 128
#define HEAD_DIM 128
#define RECORD_SCALARS (PAGE_TOKENS * HEAD_DIM)
#define THREADS 256
#define WARPS 8
#define WARP_SCALARS 2048
#define PRIMARY_DIRECT 7
#define TABLE_ENTRIES 22
#define RAW_NIBBLE 15
#define HEADER_BYTES 48
#define LOW_BYTES 16384
#define SYMBOL_BYTES 6144
#define DENSE_BYTES (LOW_BYTES + SYMBOL_BYTES)
#define VAR_CAP 2048
#define RAW_RECORD_BYTES 32768
#define MAX_WARP_RAW 32

/* attn_page.py:83-91  _kernel_order: token-major index of kernel position p. */
static inline int kernel_pos_to_token_major(int kv, int p) {
  const int t = p >> 6, s = p & 63;
  const int w = t >> 5, g = (t >> 2) & 7, c = t & 3;
  const int st = s >> 3, j = (s >> 2) & 1, f = (s >> 1) & 1, e = s & 1;
  const int row = 16 * w + 8 * j + g;
  const int col = 16 * st + 8 * f + 2 * c + e;
  const int tok = kv == 0 ? row : col;
  const int dim = kv == 0 ? col : row;
  return tok * HEAD_DIM + dim;
}

void fpo_kernel_order(int kv, int32_t* out) {
  for (int p = 0; p < RECORD_SCALARS; ++p) out[p] = kernel_pos_to_token_major(kv, p);
}

/* attn_page.py:97-111  calibrate_table: 22 most frequent bytes, ties by value. */
void fpo_calibrate_table(const uint8_t* high, int64_t n, uint8_t* table) {
  int64_t counts[256];
  memset(counts, 0, sizeof counts);
  for (int64_t i = 0; i < n; ++i) counts[high[i]]++;
  uint8_t used[256];
  memset(used, 0, sizeof used);
  for (int k = 0; k < TABLE_ENTRIES; ++k) {
    int best = -1;
    for (int b = 0; b < 256; ++b)
      if (!used[b] && (best < 0 || counts[b] > counts[best])) best = b;
    used[best] = 1;
    table[k] = (uint8_t)best;
  }
}

/* attn_page.py:114-143  primary_lut / secondary_lut. */
void fpo_luts(const uint8_t* table, uint32_t* plut2, uint8_t* slut16) {
  uint8_t p[8];
  memcpy(p, table, PRIMARY_DIRECT);
  p[7] = 0;
  plut2[0] = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
  plut2[1] = (uint32_t)p[4] | ((uint32_t)p[5] << 8) | ((uint32_t)p[6] << 16) | ((uint32_t)p[7] << 24);
  memcpy(slut16, table + PRIMARY_DIRECT, TABLE_ENTRIES - PRIMARY_DIRECT);
  slut16[15] = 0;
}

static inline void put_u32(uint8_t* p, uint32_t v) {
  p[0] = (uint8_t)v;
  p[1] = (uint8_t)(v >> 8);
  p[2] = (uint8_t)(v >> 16);
  p[3] = (uint8_t)(v >> 24);
}
static inline void put_u16(uint8_t* p, uint32_t v) {
  p[0] = (uint8_t)v;
  p[1] = (uint8_t)(v >> 8);
}
static inline uint32_t get_u32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/*
 * attn_page.py:146-209  encode_record (+ _interleave_dense :272-276,
 * _raw_words :279-282).  `raw` is token-major [128,128] BF16 bit patterns.
 * Returns the record length written to `out` (capacity 32768).
 */
int fpo_encode_record(const uint16_t* raw, const uint8_t* table, int kv, uint8_t* out) {
  uint16_t values[RECORD_SCALARS];
  uint8_t rank[RECORD_SCALARS];
  uint8_t rank_of[256];
  memset(rank_of, 255, sizeof rank_of);
  for (int i = 0; i < TABLE_ENTRIES; ++i) rank_of[table[i]] = (uint8_t)i;
  for (int p = 0; p < RECORD_SCALARS; ++p) {
    values[p] = raw[kernel_pos_to_token_major(kv, p)];
    rank[p] = rank_of[values[p] >> 8];
  }
  /* Escape / raw bookkeeping in kernel-scalar order. */
  int n_esc = 0, n_raw = 0;
  int esc_prefix[WARPS], raw_prefix[WARPS], warp_raw[WARPS];
  uint8_t var[VAR_CAP];
  /* Worst-case counts are only reached by records that fall back to raw, so
     nibbles and raw entries are gathered in side arrays first. */
  static _Thread_local uint8_t nibbles[RECORD_SCALARS];
  static _Thread_local uint32_t raw_list[RECORD_SCALARS];
  for (int w = 0; w < WARPS; ++w) {
    esc_prefix[w] = n_esc;
    raw_prefix[w] = n_raw;
    for (int p = w * WARP_SCALARS; p < (w + 1) * WARP_SCALARS; ++p) {
      const int r = rank[p];
      if (r >= PRIMARY_DIRECT) {
        if (r >= TABLE_ENTRIES) {
          nibbles[n_esc] = RAW_NIBBLE;
          raw_list[n_raw++] = (uint32_t)n_esc | ((uint32_t)(values[p] >> 8) << 16);
        } else {
          nibbles[n_esc] = (uint8_t)(r - PRIMARY_DIRECT);
        }
        ++n_esc;
      }
    }
    warp_raw[w] = n_raw - raw_prefix[w];
  }
  const int nibble_bytes = (n_esc + 1) / 2;
  const int raw_offset = (HEADER_BYTES + nibble_bytes + 3) & ~3;
  const int var_len = (raw_offset + 4 * n_raw + 15) & ~15;
  int max_warp_raw = 0;
  for (int w = 0; w < WARPS; ++w)
    if (warp_raw[w] > max_warp_raw) max_warp_raw = warp_raw[w];
  if (var_len > VAR_CAP || max_warp_raw > MAX_WARP_RAW) {
    /* Raw fallback: thread t's 16-byte word st at 16 * (256 st + t). */
    for (int t = 0; t < THREADS; ++t)
      for (int st = 0; st < 8; ++st)
        for (int i = 0; i < 8; ++i)
          put_u16(out + 16 * (256 * st + t) + 2 * i, values[64 * t + 8 * st + i]);
    return RAW_RECORD_BYTES;
  }
  /* Dense low bytes, chunk-major. */
  for (int t = 0; t < THREADS; ++t)
    for (int j = 0; j < 4; ++j)
      for (int i = 0; i < 16; ++i)
        out[16 * (256 * j + t) + i] = (uint8_t)(values[64 * t + 16 * j + i] & 0xFF);
  /* Dense symbols: three u32 per 32-scalar group (attn_page.py:174-181). */
  for (int t = 0; t < THREADS; ++t) {
    uint32_t six[6];
    for (int gi = 0; gi < 2; ++gi) {
      const uint8_t* r = rank + 64 * t + 32 * gi;
      for (int k = 0; k < 3; ++k) {
        uint32_t word = 0;
        for (int j = 0; j < 8; ++j) {
          const uint32_t a = r[8 * k + j] < PRIMARY_DIRECT ? r[8 * k + j] : PRIMARY_DIRECT;
          const uint32_t b = r[24 + j] < PRIMARY_DIRECT ? r[24 + j] : PRIMARY_DIRECT;
          word |= (a & 7u) << (4 * j);
          word |= ((b >> k) & 1u) << (4 * j + 3);
        }
        six[3 * gi + k] = word;
      }
    }
    for (int m = 0; m < 3; ++m) {
      put_u32(out + LOW_BYTES + 8 * (256 * m + t), six[2 * m]);
      put_u32(out + LOW_BYTES + 8 * (256 * m + t) + 4, six[2 * m + 1]);
    }
  }
  /* Variable region (attn_page.py:192-208). */
  memset(var, 0, (size_t)var_len);
  put_u32(var + 0, (uint32_t)n_esc);
  put_u32(var + 4, (uint32_t)n_raw);
  put_u32(var + 8, (uint32_t)raw_offset);
  put_u32(var + 12, 0);
  for (int w = 0; w < WARPS; ++w) {
    put_u16(var + 16 + 2 * w, (uint32_t)esc_prefix[w]);
    put_u16(var + 32 + 2 * w, (uint32_t)raw_prefix[w]);
  }
  for (int i = 0; i < n_esc; ++i)
    var[HEADER_BYTES + (i >> 1)] |= (uint8_t)(nibbles[i] << (4 * (i & 1)));
  for (int i = 0; i < n_raw; ++i) put_u32(var + raw_offset + 4 * i, raw_list[i]);
  memcpy(out + DENSE_BYTES, var, (size_t)var_len);
  return DENSE_BYTES + var_len;
}

/*
 * attn_page.py:212-269  decode_record.  `out` is token-major [128,128].
 * Returns 0, or -1 for a length that no record can have.
 */
int fpo_decode_record(const uint8_t* rec, int len, const uint8_t* table, int kv, uint16_t* out) {
  if (len == RAW_RECORD_BYTES) {
    for (int t = 0; t < THREADS; ++t)
      for (int st = 0; st < 8; ++st)
        for (int i = 0; i < 8; ++i) {
          const uint8_t* p = rec + 16 * (256 * st + t) + 2 * i;
          out[kernel_pos_to_token_major(kv, 64 * t + 8 * st + i)] =
              (uint16_t)(p[0] | (p[1] << 8));
        }
    return 0;
  }
  if (len < DENSE_BYTES + HEADER_BYTES || len > DENSE_BYTES + VAR_CAP) return -1;
  const uint8_t* var = rec + DENSE_BYTES;
  const uint32_t n_esc = get_u32(var), n_raw = get_u32(var + 4), raw_offset = get_u32(var + 8);
  static _Thread_local uint8_t esc_val[RECORD_SCALARS];
  if (n_esc > RECORD_SCALARS || n_raw > n_esc) return -1;
  for (uint32_t i = 0; i < n_esc; ++i) {
    const uint32_t nib = (var[HEADER_BYTES + (i >> 1)] >> (4 * (i & 1))) & 15u;
    esc_val[i] = nib < RAW_NIBBLE ? table[PRIMARY_DIRECT + nib] : 0;
  }
  for (uint32_t i = 0; i < n_raw; ++i) {
    const uint32_t v = get_u32(var + raw_offset + 4 * i);
    esc_val[v & 0xFFFFu] = (uint8_t)(v >> 16);
  }
  uint32_t next_esc = 0;
  for (int t = 0; t < THREADS; ++t) {
    uint32_t six[6];
    for (int m = 0; m < 3; ++m) {
      six[2 * m] = get_u32(rec + LOW_BYTES + 8 * (256 * m + t));
      six[2 * m + 1] = get_u32(rec + LOW_BYTES + 8 * (256 * m + t) + 4);
    }
    for (int gi = 0; gi < 2; ++gi) {
      uint32_t codes[32];
      memset(codes, 0, sizeof codes);
      for (int k = 0; k < 3; ++k)
        for (int j = 0; j < 8; ++j) {
          codes[8 * k + j] = (six[3 * gi + k] >> (4 * j)) & 7u;
          codes[24 + j] |= ((six[3 * gi + k] >> (4 * j + 3)) & 1u) << k;
        }
      for (int s = 0; s < 32; ++s) {
        const int p = 64 * t + 32 * gi + s;
        const int jchunk = (p & 63) >> 4, i = p & 15;
        const uint32_t low = rec[16 * (256 * jchunk + t) + i];
        uint32_t high;
        if (codes[s] < PRIMARY_DIRECT) {
          high = table[codes[s]];
        } else {
          if (next_esc >= n_esc) return -1;
          high = esc_val[next_esc++];
        }
        out[kernel_pos_to_token_major(kv, p)] = (uint16_t)(low | (high << 8));
      }
    }
  }
  return 0;
}

/*
 * Batch forms used by the timed CPU baseline: records are independent, so the
 * loop is spread over the host cores with OpenMP.  `raw` is [n,128,128];
 * `tables` is [n,22] (one per record); `out` has stride 32768 per record.
 */
void fpo_encode_records(int64_t n, const uint16_t* raw, const uint8_t* tables, const int32_t* kv,
                        uint8_t* out, int32_t* lens) {
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t i = 0; i < n; ++i)
    lens[i] = fpo_encode_record(raw + i * RECORD_SCALARS, tables + i * TABLE_ENTRIES, kv[i],
                                out + i * RAW_RECORD_BYTES);
}

int fpo_decode_records(int64_t n, const uint8_t* recs, const int32_t* lens, const uint8_t* tables,
                       const int32_t* kv, uint16_t* out) {
  int bad = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(| : bad)
  for (int64_t i = 0; i < n; ++i)
    bad |= fpo_decode_record(recs + i * RAW_RECORD_BYTES, lens[i], tables + i * TABLE_ENTRIES,
                             kv[i], out + i * RECORD_SCALARS) != 0;
  return bad ? -1 : 0;
}

/*
 * Staging order written by the token writer (fragpack/ops/hbm_kv.cu:223-255):
 * a raw record in kernel order, i.e. _raw_words of the permuted scalars.
 */
void fpo_raw_record(const uint16_t* raw, int kv, uint8_t* out) {
  for (int t = 0; t < THREADS; ++t)
    for (int st = 0; st < 8; ++st)
      for (int i = 0; i < 8; ++i)
        put_u16(out + 16 * (256 * st + t) + 2 * i,
                raw[kernel_pos_to_token_major(kv, 64 * t + 8 * st + i)]);
}

/* Host threads the batch forms use. */
int fpo_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the host threads of the batch forms (a launcher may have pinned the
 * OpenMP default to one); returns what is now in force. */
int fpo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
