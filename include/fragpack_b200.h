/*
 * fragpack_b200 - C ABI of the B200 (sm_100a) FragPack hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, a cudaStream_t), enqueues its kernels on that stream
 * without synchronising, and returns 0 or a negative FP_ERR_* code;
 * fp_last_error() then describes the failure.  Nothing here allocates device
 * memory.  Each function replaces one function of the reference's pybind11
 * module `fragpack_cuda` (fragpack/ops/fragpack_ext.cpp:57-66); the reference
 * file:line of the replaced function is given with each declaration.
 *
 * Layouts (identical to the reference):
 *   record      see fragpack/compression/attn_page.py:1-44
 *   rec_addr    int64 [L, NB, 2, H]  absolute device address of each record
 *   rec_len     int32 [L, NB, 2, H]  record bytes - 22528; 10240 marks a raw record
 *   plut        int32 [.., 2, H, 2]  primary prmt words      (attn_tables.py:96-124)
 *   slut        uint8 [.., 2, H, 16] extended table
 *   rank_of     uint8 [L, 2, H, 256] table rank of a high byte, 255 = absent
 */
#ifndef FRAGPACK_B200_H_
#define FRAGPACK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FP_OK 0
#define FP_ERR_ARGUMENT (-1) /* rejected arguments; nothing was enqueued */
#define FP_ERR_CUDA (-2)     /* a CUDA runtime call or launch failed */

/* Counter slots of fp_store.counters (fragpack/ops/hbm_kv.cu:14-26). */
enum {
  FP_CTR_FREE_TOP = 0,
  FP_CTR_TRANSIENT = 1,
  FP_CTR_CLAIMS = 2,
  FP_CTR_CLOSES = 3,
  FP_CTR_ERR_STAGING = 4,
  FP_CTR_ERR_OVERFLOW = 5,
  FP_CTR_FALLBACKS = 6,
  FP_CTR_ENCODED = 7,
  FP_CTR_SPILLS = 8,
  FP_CTR_HEIRS = 9,
  FP_CTR_DONORS = 10,
  FP_CTR_SEEN_OPEN = 11,  /* blocks seen opening this step (prepare's scan) */
  FP_CTR_SEEN_CLOSE = 12, /* blocks seen closing this step */
  FP_CTR_OVF_FREE = 13,   /* free overflow slots; initialise to overflow_records */
  FP_NUM_COUNTERS = 16
};

/* Import status bits (fragpack/ops/hbm_kv.cu:507). */
enum { FP_BLOB_BAD_HEADER = 1, FP_BLOB_BAD_LENGTHS = 2, FP_BLOB_NO_OVERFLOW = 4 };

/* Bits of the decode status word (see fp_fused_decode). */
enum { FP_DECODE_WAIT_TIMEOUT = 1, FP_DECODE_NOT_PLAIN = 2 };

/* Bit of fp_peers.status. */
enum { FP_PEER_WAIT_TIMEOUT = 1 };

#define FP_MAX_PEERS 8

/*
 * The store state that the reference passes as 13 positional tensors to every
 * hbm_* function (fragpack/ops/hbm_kv.py:287-301, hbm_kv.cu:32-78), plus the
 * two tables this library's prepare uses (slot_owner, seen_list).  The caller
 * allocates everything, zero-filled except: wslot and slot_owner -1,
 * free_stack 0 .. S_p - 1 with counters[FP_CTR_FREE_TOP] = S_p, the bits of
 * ovf_bits past the pool set with counters[FP_CTR_OVF_FREE] = overflow_records,
 * rec_addr pointing at an all-zero raw record with rec_len 10240.
 */
typedef struct fp_store {
  int32_t* counters;    /* [FP_NUM_COUNTERS] */
  int32_t* wslot;       /* [NB] staging slot of an open block, -1 if none */
  int32_t* tags;        /* [4, NB] per-block step stamps */
  int32_t* free_stack;  /* [S_p] */
  uint32_t* ovf_bits;   /* [ovf_words] overflow slots in use (tail bits preset) */
  int32_t* claim_list;  /* [2, cap] claimed blocks, then heirs */
  int32_t* close_list;  /* [2, cap] closing blocks, then the heir of each */
  int64_t* rec_addr;    /* [L, NB, 2, H] */
  int32_t* rec_len;     /* [L, NB, 2, H] */
  uint8_t* staging;     /* [S_p, L, 2, H, 32768] persistent staging */
  uint8_t* scratch;     /* [S_t, 2, H, 32768] one layer of transient staging */
  uint8_t* overflow;    /* [O, 32768] raw records that do not code or fit */
  int32_t* fill;        /* [L, NB] bytes used in each block-layer page */
  int32_t* slot_owner;  /* [S_p + S_t] block that owns each staging slot, -1 if free */
  int32_t* seen_list;   /* [2, cap] blocks seen opening, then closing, this step */
  int64_t overflow_records; /* O */
  int32_t L, H, NB, S_p, S_t, ovf_words, cap;
} fp_store;

/* Message of the calling thread's last failed call ("" if none). */
const char* fp_last_error(void);

/* Library version string. */
const char* fp_version(void);

/*
 * Element counts of the decode workspace for `kv_heads` and `units`
 * (replaces fragpack/ops/fused_attn_decode.py:88-102 workspace_elems):
 * float elements of `opart` and `ml`, int32 elements of `plan`.
 */
int fp_decode_workspace(int32_t kv_heads, int32_t units, int64_t* opart_elems, int64_t* ml_elems,
                        int64_t* plan_elems);

/*
 * Split-KV decode attention for one query token per sequence over compressed
 * KV records.  Replaces fused_decode (fragpack/ops/fused_attn_decode.cu:429-478,
 * bound at fragpack_ext.cpp:60), with the query group handled natively.
 *
 *   q, out       BF16 [B, H * group, 128]; row strides in elements, head stride 128
 *   rec_addr/rec_len  one layer: [NB, 2, H]
 *   plut/slut    one layer: [2, H, 2] / [2, H, 16]
 *   block_table  int32 [B, >= pages]; row stride in elements
 *   seq_lens     int32 [B]; 0 gives a zero output row
 *   opart/ml/plan workspace sized by fp_decode_workspace
 *   group        query heads per KV head: 1, 2, 4 or 8
 *   units        work-unit capacity per KV head, >= B
 *   replan       nonzero: recompute the plan from seq_lens (first layer of a step)
 * `plan` holds 2 + 4 * units + 2 + 260 + 4 * units int32 (fp_decode_workspace
 * gives the count): the reference's plan, a spare word, a status word, the
 * words of the dynamic item schedule and four words per unit of item
 * descriptors.  The int32 at index 2 + 4 * units + 1 is the status word: the
 * kernels OR FP_DECODE_* bits into it when a bounded device-side wait ran out
 * (results are then invalid); the planner clears it.  opart and plan must be
 * 16-byte aligned, ml 8-byte aligned.
 */
int fp_fused_decode(const void* q, int64_t q_stride, const int64_t* rec_addr,
                    const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                    float* opart, int64_t opart_elems, float* ml, int64_t ml_elems, int32_t* plan,
                    int64_t plan_elems, void* out, int64_t out_stride, int32_t batch,
                    int32_t kv_heads, int32_t group, int32_t units, int32_t replan, float scale,
                    int32_t num_sms, void* stream);

/*
 * Comparison arm: the same split-KV decode attention over PLAIN BF16 records
 * (every record raw, 32,768 bytes in fragment order: rec_len > 2048), with no
 * decode step.  It measures what a plain BF16 paged read of the same logical
 * KV costs with the same planner, pipeline, softmax and merge; the reference
 * has no such kernel (its raw records go through decode_attn,
 * fragpack/ops/fused_attn_decode.cu:214-404).  Arguments as fp_fused_decode
 * without the tables.  A coded record met here contributes zeros and sets
 * FP_DECODE_NOT_PLAIN in the status word.
 */
int fp_plain_decode(const void* q, int64_t q_stride, const int64_t* rec_addr,
                    const int32_t* rec_len, const int32_t* block_table, int64_t bt_stride,
                    const int32_t* seq_lens, float* opart, int64_t opart_elems, float* ml,
                    int64_t ml_elems, int32_t* plan, int64_t plan_elems, void* out,
                    int64_t out_stride, int32_t batch, int32_t kv_heads, int32_t group,
                    int32_t units, int32_t replan, float scale, int32_t num_sms, void* stream);

/*
 * Tensor-parallel decode by KV head with the output exchange done by the merge
 * kernel itself: every rank writes its heads of every row straight into every
 * rank's o_proj input buffer through peer pointers (NVLink stores), instead of
 * writing a local tensor that a collective then gathers.  The reference
 * declares this head sharding (fragpack/integrations/vllm/backend.py:223-226)
 * but has no exchange of its own; this replaces the NCCL all-gather a host
 * would otherwise place after fused_decode.
 *
 * One fp_peers per rank.  out[r] / flag[r] are device pointers valid on THIS
 * rank: the rank's own allocation at index `rank`, peer mappings (symmetric
 * memory or IPC; plain peer stores and loads only, no multicast) at the others.
 *   out[r]   rank r's gathered buffer: BF16 [2][B][world * kv_heads * group][128],
 *            two alternating copies so that a rank ahead by one call cannot
 *            overwrite rows a slower rank still reads
 *   flag[r]  rank r's arrival words, int32 [FP_MAX_PEERS]: word s holds the
 *            number of calls rank s has completed
 *   epoch    this rank's call counter, int32 [1], zero before the first call
 *   status   this rank's status word, int32 [1]: FP_PEER_WAIT_TIMEOUT is set
 *            when a peer did not arrive within about two seconds (the rows it
 *            owes are then invalid; the kernel returns, the context stays usable)
 */
typedef struct fp_peers {
  void* out[FP_MAX_PEERS];
  int32_t* flag[FP_MAX_PEERS];
  int32_t* epoch;
  int32_t* status;
  int32_t world, rank;
} fp_peers;

/*
 * fp_fused_decode for one rank of a KV-head-sharded group.  Arguments as
 * fp_fused_decode, except that the output goes to copy `buffer` (0 or 1,
 * alternate it call by call) of every rank's gathered buffer: this rank's
 * kv_heads * group query heads land at heads [rank * kv_heads * group, ...) of
 * each row, row stride `out_stride` elements.  The call then signals its
 * arrival to every rank and enqueues a bounded wait for all ranks' arrivals,
 * so that work enqueued after it on this stream sees the whole gathered copy.
 * Every rank must make the same sequence of calls.
 */
int fp_fused_decode_peers(const void* q, int64_t q_stride, const int64_t* rec_addr,
                          const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                          const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                          float* opart, int64_t opart_elems, float* ml, int64_t ml_elems,
                          int32_t* plan, int64_t plan_elems, const fp_peers* peers,
                          int32_t buffer, int64_t out_stride, int32_t batch, int32_t kv_heads,
                          int32_t group, int32_t units, int32_t replan, float scale,
                          int32_t num_sms, void* stream);

/*
 * fp_fused_decode without a caller-provided workspace, for hosts that cannot
 * call cudaMalloc (or any allocator) on behalf of this library: engines that
 * own all device memory, plugins inside a foreign memory planner, workers whose
 * allocator is frozen while serving.  It has no counterpart in the reference.
 *
 * The opart / ml / plan workspace lives in a fixed array inside the library
 * (about 16.3 MiB, held on every GPU that loads the library until the process
 * exits).  Limits: kv_heads * units <= 4096 and units <= 4096; larger requests
 * are rejected with FP_ERR_ARGUMENT and a message naming the limit.  The call
 * allocates nothing and calls no allocating routine.
 *
 * The first call on a device looks up the array's device address (once per
 * device, with that device current); make that first call before any stream
 * capture begins.  All calls share the one array and it keeps the previous
 * call's contents: a call with replan = 0 reuses the plan of the previous call
 * exactly as fp_fused_decode does with a reused workspace, and calls that can
 * overlap on the GPU (different streams, or different threads) race on it -
 * serialise them.  Arguments are those of fp_fused_decode minus the workspace.
 */
int fp_fused_decode_noalloc(const void* q, int64_t q_stride, const int64_t* rec_addr,
                            const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* seq_lens, void* out, int64_t out_stride, int32_t batch,
                            int32_t kv_heads, int32_t group, int32_t units, int32_t replan,
                            float scale, int32_t num_sms, void* stream);

/*
 * Causal prefill attention directly over compressed records.  Replaces the
 * gather + FlashAttention step of the reference's prefill path
 * (fragpack/integrations/vllm/backend.py:560-575: store.gather, then
 * flash_attn_varlen_func over the BF16 workspace) by one kernel that decodes
 * the records into shared-memory operand tiles and runs both products on the
 * tensor cores (tcgen05); the decompressed KV is never written to HBM.
 *
 *   q, out      BF16 [T, H * group, 128]; row strides in elements (multiples of 8)
 *   rec_addr/rec_len, plut/slut   one layer, as for fp_fused_decode
 *   block_table int32 [R, >= pages]; row stride in elements
 *   q_start     int32 [R + 1]: request r owns query rows q_start[r] .. q_start[r + 1]
 *   ctx_len     int32 [R]: its context length, the new tokens included (they
 *               must already be in the store: fp_hbm_write comes first)
 *   max_query_tokens  the most query rows of any request (sizes the grid)
 *   scale       softmax scale, > 0
 *   status      one int32 of the caller, zeroed once: the kernel ORs
 *               FP_DECODE_WAIT_TIMEOUT into it when a bounded wait ran out
 * Query i of request r sits at position ctx_len[r] - n_r + i and attends the
 * keys up to and including itself.
 */
int fp_prefill_attention(const void* q, int64_t q_stride, const int64_t* rec_addr,
                         const int32_t* rec_len, const int32_t* plut, const uint8_t* slut,
                         const int32_t* block_table, int64_t bt_stride, const int32_t* q_start,
                         const int32_t* ctx_len, void* out, int64_t out_stride, int32_t num_requests,
                         int32_t max_query_tokens, int32_t kv_heads, int32_t group, float scale,
                         int32_t* status, void* stream);

/* hbm_prepare (fragpack/ops/hbm_kv.cu:669-686): start a step. */
int fp_hbm_prepare(const fp_store* store, const int64_t* slot_mapping, int64_t num_tokens,
                   const int32_t* live, int64_t num_live, int32_t step, void* stream);

/*
 * hbm_write (fragpack/ops/hbm_kv.cu:688-705): scatter new K / V tokens
 * BF16 [N, H, 128] (strides in elements, head dim contiguous) into staging.
 */
int fp_hbm_write(const fp_store* store, const void* key, int64_t k_stride0, int64_t k_stride1,
                 const void* value, int64_t v_stride0, int64_t v_stride1,
                 const int64_t* slot_mapping, int64_t num_tokens, int32_t layer, void* stream);

/*
 * hbm_encode (fragpack/ops/hbm_kv.cu:707-723): the block encoder.  Codes this
 * layer's records of every block closed this step into the block's arena page
 * (`arena` + block * `page_bytes`) or raw into the overflow pool.  Output
 * bytes equal attn_page.encode_record (attn_page.py:146-209).
 */
int fp_hbm_encode(const fp_store* store, const uint8_t* rank_of, int32_t layer, uint8_t* arena,
                  int64_t page_bytes, int64_t max_close, void* stream);

/* hbm_commit (fragpack/ops/hbm_kv.cu:725-734): release closed blocks' staging. */
int fp_hbm_commit(const fp_store* store, void* stream);

/*
 * hbm_gather (fragpack/ops/hbm_kv.cu:736-753): the prefill decompressor.
 * Decodes records of `blocks[i]` of one layer into token-major BF16 pages
 * wk / wv [>= n, 128, H, 128].  Its device-side waits are bounded; should one
 * run out, bit 0 of the status word read by fp_hbm_gather_status is set (the
 * workspace contents are then invalid).
 */
int fp_hbm_gather(const int32_t* blocks, int64_t n, const int64_t* rec_addr,
                  const int32_t* rec_len, const int32_t* plut, const uint8_t* slut, void* wk,
                  void* wv, int64_t workspace_bytes, int32_t kv_heads, void* stream);

/* Copies the decompressor's status word to the host (synchronises the device's
 * prior work on the legacy stream) and clears it, so that each read reports the
 * calls since the previous one; zero in normal operation.  No counterpart in
 * the reference. */
int fp_hbm_gather_status(int32_t* status);

/*
 * Test hook, no counterpart in the reference.  Every device-side wait of this
 * library gives up after a cycle budget (about two seconds) and reports through
 * a status word instead of hanging.  This call sets that budget for the
 * launches that follow (`cycles` > 0; 0 restores the default) and names one
 * record per CTA, by its ordinal in the CTA's stream, that the producer warp
 * will leave out (`skip_record` >= 0; -1 none), so that a test can make a wait
 * run out, on purpose and harmlessly, and check the status word.  Process-wide;
 * not for production use.
 */
int fp_debug_wait_limit(int64_t cycles, int64_t skip_record);

/*
 * hbm_export (fragpack/ops/hbm_kv.cu:755-774): closed blocks -> block blobs.
 * Blob i is written at out + i * stride and lengths[i] receives its size (a
 * 4096 multiple).  `scratch` is int64 [n, L * 2 * H] device memory of the
 * caller: the layout pass leaves every record's offset there for the copy pass
 * (one CTA per record).  Any number of KV heads.
 */
int fp_hbm_export(const int32_t* blocks, int64_t n, const int64_t* rec_addr,
                  const int32_t* rec_len, uint8_t* out, int64_t out_bytes, int64_t stride,
                  int64_t* lengths, int64_t* scratch, int32_t L, int32_t H, int32_t NB,
                  int64_t digest, void* stream);

/*
 * hbm_import (fragpack/ops/hbm_kv.cu:776-802): block blobs -> blocks of this
 * store.  status[i] (zeroed by the caller) receives FP_BLOB_* bits; a blob with
 * a bad header or length table is left alone, a layer that finds the overflow
 * pool full keeps its old records.  `scratch` is int64 [2, n, L * 2 * H] device
 * memory of the caller (source and destination address of every record).  A
 * replaced record's overflow slot is returned only after the new record is in
 * place.  Any number of KV heads.
 */
int fp_hbm_import(const fp_store* store, const uint8_t* src, int64_t src_bytes,
                  const int64_t* offsets, const int32_t* blocks, int64_t n, int32_t* status,
                  int64_t* scratch, const int64_t* arena_base, const int64_t* arena_stride,
                  int64_t digest, void* stream);

/*
 * Batch form of attn_page.encode_record (fragpack/compression/attn_page.py:146-209)
 * on the device: record i is token-major uint16 [128,128] at raw + i * 32768,
 * coded with table `rank_of + 256 * table_index[i]` as K (kv[i] = 0) or V (1)
 * into out + i * out_stride (>= 32768, 16-byte multiple); out_len[i] receives
 * the record bytes (32768 for the raw fallback).
 */
int fp_encode_records(const void* raw, int64_t n, const uint8_t* rank_of,
                      const int32_t* table_index, const int32_t* kv, uint8_t* out,
                      int64_t out_stride, int32_t* out_len, void* stream);

/*
 * Batch form of attn_page.decode_record (attn_page.py:212-269): record i at
 * recs + i * rec_stride with rec_len[i] bytes past the dense part (10240 =
 * raw) is decoded to token-major uint16 [128,128] at out + i * 32768.
 */
int fp_decode_records(const uint8_t* recs, int64_t rec_stride, const int32_t* rec_len, int64_t n,
                      const int32_t* plut, const uint8_t* slut, const int32_t* table_index,
                      const int32_t* kv, void* out, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* FRAGPACK_B200_H_ */
