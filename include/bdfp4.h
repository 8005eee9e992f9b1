/*
 * bdfp4 — C ABI of the B200 (sm_100a) NVFP4 KV-cache quantize-on-write and paged
 * FP4 decode-attention kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (passed as void*), launches on that stream, never synchronises, and — unless a
 * comment says otherwise — never allocates. The return value is a status code:
 * 0 on success, a negative BDFP4_E_* value when the host-side argument check
 * refused the call (nothing was launched), or BDFP4_E_CUDA when a CUDA runtime
 * call failed. Device-detected problems (a bounded wait that ran out, a page id
 * outside the cache) are OR-ed into the caller's optional `error_word`.
 *
 * Each declaration cites the interface of OpenBitSys/BitDecoding-FP4 it replaces,
 * as path:line inside that project.
 */
#ifndef BDFP4_H_
#define BDFP4_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BDFP4_PAGE_TOKENS 128 /* tokens per FP4 page (src/nvfp4_decode_kernel/_decode.py:23) */
#define BDFP4_HEAD_DIM 128    /* channels per head (src/nvfp4_decode_kernel/_decode.py:24) */
#define BDFP4_GROUP 16        /* values per E4M3 scale */
#define BDFP4_MAX_SINK 16     /* src/nvfp4_decode_kernel/interface.py:17 */

/* status codes */
#define BDFP4_OK 0
#define BDFP4_E_ARG (-1)      /* a size, pointer or alignment contract is violated */
#define BDFP4_E_UNSUPPORTED (-2) /* a valid request this build has no kernel for */
#define BDFP4_E_CUDA (-3)     /* a CUDA runtime/driver call failed; see bdfp4_last_cuda_error */
#define BDFP4_E_DEVICE (-4)   /* the current device is not sm_100-family */
#define BDFP4_E_TOO_LARGE (-5) /* the request does not fit a fixed-capacity buffer of the library */

/* bits a kernel may OR into *error_word */
#define BDFP4_DEV_WAIT_TIMEOUT 1u /* a bounded mbarrier wait gave up */
#define BDFP4_DEV_BAD_PAGE 2u     /* a page id outside [0, pages) was clamped */

/* NVFP4 scale-candidate sets (src/nvfp4_decode_kernel/scale_mode.py:18-22) */
#define BDFP4_SCALE_AMAX6 0            /* (6) */
#define BDFP4_SCALE_FOUR_SIX 1         /* (6, 4) */
#define BDFP4_SCALE_FOUR_SIX_SIXHALF 2 /* (6, 4, 6.5) */
/* MXFP4 exponent rules: one E8M0 power-of-two scale per 32 values
 * (src/nvfp4_decode_kernel/scale_mode.py:40-49, src/nvfp4_decode_kernel/_block_scale.py:418-546) */
#define BDFP4_SCALE_MXFP4_OCP 3      /* floor(log2(amax)) - 2 */
#define BDFP4_SCALE_MXFP4_ROUND_UP 4 /* the smallest exponent that keeps amax at or below 6 */
#define BDFP4_SCALE_MXFP4_SEARCH 5   /* ocp or ocp + 1, whichever has strictly less squared error */

/* scale format of a cache / of the decode operands */
#define BDFP4_FORMAT_NVFP4 0 /* E4M3 scale per 16 values */
#define BDFP4_FORMAT_MXFP4 1 /* E8M0 scale per 32 values; 128-token pages only */

/* softmax-probability scale rules (src/nvfp4_decode_kernel/p_scale.py:29-40) */
#define BDFP4_P_AMAX6 0              /* amax/6 */
#define BDFP4_P_AMAX2_OR_AMAX6 1     /* amax/2 when amax <= tau else amax/6 */
#define BDFP4_P_AMAX2_OR_AMAX6_C8 2  /* the same on 8*p, LSE corrected by -3 ln 2 (default) */

/* key_shift element types */
#define BDFP4_SHIFT_NONE 0
#define BDFP4_SHIFT_F32 1
#define BDFP4_SHIFT_BF16 2

int bdfp4_version(void);
const char* bdfp4_status_string(int status);
/* Text of the last CUDA error this library saw on the calling thread ("" if none). */
const char* bdfp4_last_cuda_error(void);
/* 0 when the current device can run these kernels (compute capability 10.x), else BDFP4_E_DEVICE.
 * Replaces the device check of src/nvfp4_decode_kernel/_decode.py:730-741. */
int bdfp4_check_device(void);

/*
 * K/V page quantize-on-write plus BF16 tail/sink token writes: one call covers the three
 * roles of the reference's writer launch.
 * Replaces KVCacheWriter.__call__ (src/nvfp4_decode_kernel/quantize_kv_kernel.py:984-1038),
 * its kernel roles _key_page/_value_page/_tail_token (:165-339) and the per-layer "seal"
 * form with a [4, layers] base-address table (:579-583).
 *
 * Page interior layouts (fixed; only the page pitch is free):
 *   K codes  u8 [128 tok][H][64]          byte = channels (2b, 2b+1), even channel in the low nibble
 *   V codes  u8 [H][128 ch][64]           byte = tokens (2b, 2b+1)
 *   scales   u8 [H][2][32][4][4]          byte of (row r, group g, head h) =
 *            h*1024 + (g/4)*512 + (r%32)*16 + (r/32)*4 + g%4; r = token for K, channel for V,
 *            g = channel group for K, token group for V.
 *
 * 64-token pages (page_tokens = 64; the reference has none, src/nvfp4_decode_kernel/_decode.py:23 pins 128).
 * A sequence still moves to FP4 in 128-token steps (seqused_fp4 stays a multiple of 128), each step
 * filling two entries of the row's page table, older 64 tokens first; codes and scale values are
 * those of the 128-token page holding the same tokens, only the byte placement differs. A page's
 * codes are stored per head as the shared-memory image the decode kernel's MMA reads (rows with
 * their 16-byte chunks at the swizzled position), so the kernel fetches them as they lie:
 *   K codes  u8 [H][64 tok][64]           chunk j of token t at position j ^ ((t >> 1) & 3)
 *   V codes  u8 [H][128 ch][32]           byte = tokens (2b, 2b+1); chunk j of channel c at j ^ ((c >> 2) & 1)
 *   K scales u8 [H][2][32][2][4]          byte of (token t, group g, head h) =
 *            h*512 + (g/4)*256 + (t%32)*8 + (t/32)*4 + g%4   (two half atoms; the decode kernel
 *            interleaves the halves of a step's two pages into the 128-row atoms of its MMA)
 *   V scales u8 [H][32][4][4]             byte of (channel c, token group g < 4, head h) =
 *            h*512 + (c%32)*16 + (c/32)*4 + g
 */
typedef struct bdfp4_kv_write_args {
  /* source: [tokens, H, 128] BF16, dense within a token; pitch in elements (multiple of 8) */
  const void* key;   /* NULL: no K role */
  const void* value; /* NULL: no V role */
  int64_t key_token_pitch;
  int64_t value_token_pitch;
  int64_t source_tokens_total; /* tokens in key/value (per-layer writer: all layers, back to back) */
  int32_t heads;               /* KV heads H */
  /* destination regions of ONE layer; ignored when `bases` is given */
  void* key_codes;
  void* key_scales;
  void* value_codes;
  void* value_scales;
  int64_t key_codes_pitch; /* bytes between pages, multiple of 16 */
  int64_t key_scales_pitch;
  int64_t value_codes_pitch;
  int64_t value_scales_pitch;
  /* per-layer form: device int64 [4][layers] addresses (K codes, K scales, V codes, V scales) */
  const int64_t* bases;
  int32_t layers; /* 1 unless `bases` */
  /* work table: item w reads 128 tokens from source_tokens[w], writes page destination_pages[w]
   * (negative: skip). Device int32 [work_items]. */
  const int32_t* source_tokens;
  const int32_t* destination_pages;
  int32_t work_items;
  int32_t key_scale_mode;   /* BDFP4_SCALE_* */
  int32_t value_scale_mode; /* BDFP4_SCALE_* */
  /* K transform: Hadamard rotation and/or subtraction of key_shift[layer][H][128] */
  int32_t rotate_key;
  const void* key_shift;
  int32_t key_shift_type; /* BDFP4_SHIFT_* */
  int32_t layer;          /* selects key_shift / tail layer of a one-layer call */
  /* tail role (NULL tail_key: none): tail buffers BF16 [layers][slots][128+sink_tokens][H][128] */
  void* tail_key;
  void* tail_value;
  int64_t tail_layer_stride; /* elements */
  int64_t tail_slot_stride;  /* elements */
  int32_t sink_tokens;
  const int32_t* query_start_loc; /* [rows+1] */
  const int32_t* seq_lens;        /* [rows] */
  const int32_t* seqused_fp4;     /* [rows] */
  const int32_t* row_to_slot;     /* [rows] */
  int32_t rows;
  int32_t decode_rows;
  int32_t first_row;
  int32_t* error_word; /* optional */
  /* Tokens per cache page: 0 or 128 (the reference's only size), or 64 (see "64-token pages"):
   * a work item then reads 64 tokens. The BF16 tail keeps its 128 rolling rows either way. */
  int32_t page_tokens;
  /* Pages in each destination region. A work item whose destination is at or past it is skipped
   * and BDFP4_DEV_BAD_PAGE is OR-ed into *error_word, so a corrupt work table cannot write outside
   * the cache. 0: unknown, only negative ids are skipped. */
  int32_t pages;
  /* FP32 per-tensor scales, no reference counterpart (the reference's scale is the E4M3 block
   * scale alone, src/nvfp4_decode_kernel/_block_scale.py:272-289): the pages hold x / tensor_scale,
   * i.e. x ~ code * block_scale * tensor_scale, which keeps block scales inside E4M3's range for
   * tensors far from unit magnitude. The division is a multiplication by fl32(1 / tensor_scale)
   * before the block-scale search (K: after the cache-basis transform and its BF16 rounding). The
   * BF16 tail is not scaled. 0 or 1.0: none, and the bytes are those of the reference. The decode
   * call must be given the same values. */
  float key_tensor_scale;
  float value_tensor_scale;
} bdfp4_kv_write_args;

int bdfp4_kv_write(const bdfp4_kv_write_args* args, void* stream);

/*
 * Decode-query quantization (one or two NVFP4 terms, optional Hadamard), the padded BF16
 * copy of the query, and optionally this step's K/V token into the BF16 tail.
 * Replaces quantize_decode_q_to_padded_fp4 (src/nvfp4_decode_kernel/quantize_q_kernel.py:681-1110)
 * and its kernel _quantize_query_kernel (:364-428), including the DecodeTailWrite side
 * (src/nvfp4_decode_kernel/interface.py:45-69).
 *
 * query_codes   u8 [rows][1][Hq][64]
 * query_scales  u8 storage [rows][1][Hq][2][32][4][4]; head h writes row (h % G) of the tile of
 *               KV head h / G, whose 1024 bytes start at (row*Hq + h/G)*1024
 *               (src/nvfp4_decode_kernel/_quantize.py:100-132). Unwritten bytes must already be zero.
 * query_padded  BF16 [rows][128][Hq][128], only [:, 0] written (NULL: skip)
 */
typedef struct bdfp4_quantize_query_args {
  const void* query; /* BF16 [src_rows][Hq][128] */
  int64_t query_row_stride;  /* elements, multiple of 8 */
  int64_t query_head_stride; /* elements, multiple of 8 */
  const int32_t* row_indices; /* optional [rows]: source row of each output row */
  int32_t rows;
  int32_t heads_q;
  int32_t heads_kv;
  int32_t scale_mode; /* BDFP4_SCALE_* */
  int32_t rotate;     /* Hadamard on the query */
  void* query_codes;
  void* query_scales;
  void* query_codes_second; /* NULL: one term */
  void* query_scales_second;
  void* query_padded;
  /* fused tail write (tail_key NULL: none) */
  const void* new_key;   /* BF16 [>=rows][H][128] */
  const void* new_value;
  int64_t new_key_token_pitch;
  int64_t new_value_token_pitch;
  void* tail_key;   /* one layer: BF16 [slots][128+sink_tokens][H][128] */
  void* tail_value;
  int64_t tail_slot_stride; /* elements */
  const int32_t* row_to_slot;
  const int32_t* seq_lens;
  const int32_t* seqused_fp4;
  int32_t rotate_key;
  const float* key_shift; /* FP32 [H][128], already in the rotated basis; NULL: none */
  int32_t sink_tokens;
  /* FP32 per-tensor scale of the query codes (see bdfp4_kv_write_args): the terms hold
   * q / tensor_scale; the padded BF16 copy is not scaled. 0 or 1.0: none. */
  float tensor_scale;
} bdfp4_quantize_query_args;

int bdfp4_quantize_query(const bdfp4_quantize_query_args* args, void* stream);

/*
 * Paged FP4 decode attention, one query token per row.
 * Replaces decode_fp4 / decode_fp4_split (src/nvfp4_decode_kernel/_decode.py:697-1456) and the
 * kernel FP4DecodeKernel (src/nvfp4_decode_kernel/fp4_decode_kernel.py:147-7953) in the one
 * configuration the reference instantiates (head_dim 128, page 128, one query token,
 * transposed scores, BF16 tail and sink from the paged BF16 buffer).
 *
 * Blocks are merged in the reference's order: the BF16 tail, FP4 pages newest to oldest, the
 * BF16 sink. With num_splits > 1 split s owns pages [s*c, min((s+1)*c, n)), c = ceil(n/num_splits),
 * and writes a normalised FP32 partial and a natural-log LSE (-inf when it had nothing);
 * the tail and sink belong to split 0, or to an extra last split when bf16_split != 0
 * (src/nvfp4_decode_kernel/interface.py:24-42). bdfp4_combine then produces the BF16 output.
 */
typedef struct bdfp4_decode_args {
  int32_t rows;
  int32_t heads_q;
  int32_t heads_kv;
  /* query operands as bdfp4_quantize_query wrote them */
  const void* query_codes;
  const void* query_scales;
  const void* query_codes_second; /* NULL: one term */
  const void* query_scales_second;
  const void* query_padded; /* BF16 [rows][128][Hq][128]; required with a tail */
  /* FP4 cache regions */
  const void* key_codes;
  const void* key_scales;
  const void* value_codes;
  const void* value_scales;
  int64_t key_codes_pitch; /* bytes */
  int64_t key_scales_pitch;
  int64_t value_codes_pitch;
  int64_t value_scales_pitch;
  int32_t pages; /* pages in the cache regions */
  const int32_t* page_table; /* int32 [rows][page_table_stride] */
  int64_t page_table_stride;
  int32_t max_pages_per_row;
  const int32_t* seqused_fp4; /* [rows], multiples of 128 */
  /* BF16 tail + sink (tail_key NULL: none): [slots][128 (+16 if seqused_sink)][H][128] */
  const void* tail_key;
  const void* tail_value;
  int64_t tail_slot_stride; /* elements */
  int32_t tail_slots;
  const int32_t* tail_slot_ids;    /* [rows]; negative: no tail for the row */
  const int32_t* seqused_residual; /* [rows] in [0,128] */
  const int32_t* seqused_sink;     /* [rows] in [0,16]; NULL: no sink */
  float softmax_scale;
  int32_t p_scale_mode; /* BDFP4_P_* */
  float p_scale_tau;    /* threshold of the amax2_or_amax6 rules (default 21/1024) */
  /* outputs */
  void* out; /* BF16 [rows][Hq][128] with row stride out_row_stride (elements); used when num_splits == 1.
              * NULL at num_splits == 1: the single part is written as a partial + LSE instead (one KV-axis
              * shard of a longer sequence, to be merged by bdfp4_combine with the other shards' partials) */
  int64_t out_row_stride;
  int32_t num_splits;
  int32_t bf16_split;  /* 1: tail+sink get a split of their own (index num_splits) */
  float* partial_out;  /* FP32 [parts][rows][Hq][128], parts = num_splits + bf16_split */
  float* partial_lse;  /* FP32 [parts][rows][Hq] */
  int32_t* error_word; /* optional */
  /* Split-KV load balance, no reference counterpart: when split 0 also merges the tail and the sink
   * (num_splits > 1, bf16_split == 0) it is charged this many pages for them: with
   * c = ceil((n + cost) / num_splits) split 0 owns pages [0, max(c - cost, 0)) and split s >= 1 the
   * next c pages. 0 keeps the reference's even partition. The merged output is the same up to the
   * rounding of the partials. */
  int32_t bf16_page_cost;
  /* Tokens per cache page: 0 or 128 (the reference's only size), or 64 (see "64-token pages"). */
  int32_t page_tokens;
  /* Fused split merge, no reference counterpart (the reference always launches SplitKCombine,
   * src/nvfp4_decode_kernel/split_k_combine.py:86-133). With num_splits > 1, `out` set and this
   * pointer non-NULL, the part of each (row, KV head) that finishes last merges the partials into
   * `out` itself, with the arithmetic and part order of bdfp4_combine; no merge launch is needed.
   * int32 [rows * heads_kv], zero before the first launch; every launch leaves it zero. Launches
   * that share the array must not overlap on the GPU. */
  int32_t* merge_counters;
  /* Launch order of the rows, no reference counterpart: int32 [rows], a permutation of 0..rows-1
   * (device memory); position i of the launch serves row row_order[i]. A caller with a ragged batch
   * lists the rows longest first: CTAs reach the SMs in launch order, so the longest walks start
   * first and the short ones fill in behind them. NULL: rows in index order. The result does not
   * depend on it. */
  const int32_t* row_order;
  /* BDFP4_FORMAT_*: NVFP4 (0, default) or MXFP4. With MXFP4 the scale regions are E8M0 bytes, one
   * 512-byte atom per (page, head) for K (128 tokens x 4 channel groups of 32) and for V (128
   * channels x 4 token groups of 32), the query scales one atom per (row, KV head), the products
   * are tcgen05.mma kind::mxf4 scale_vec::2X, and the probabilities are quantized per 32 tokens with
   * the one MXFP4 rule (src/nvfp4_decode_kernel/reference.py:331-355); p_scale_mode is ignored.
   * page_tokens must be 128. */
  int32_t scale_format;
  /* FP32 per-tensor scales the cache and the query were written with (0 or 1.0: none): FP4-page
   * scores are multiplied by key_tensor_scale * query_tensor_scale, FP4-page outputs by
   * value_tensor_scale; the BF16 tail and sink are not scaled. */
  float key_tensor_scale;
  float query_tensor_scale;
  float value_tensor_scale;
  /* Parts per row, no reference counterpart: int32 [rows] (device memory), each in 1..num_splits; row r
   * is cut into row_splits[r] parts and the launch's remaining parts of that row find no pages, write
   * an LSE of -inf and leave at once. For ragged batches: the long rows are cut finely enough to
   * bound the launch while the short ones are not cut into set-up. NULL: num_splits parts for every
   * row. Ignored with num_splits == 1 or merge_counters. */
  const int32_t* row_splits;
} bdfp4_decode_args;

int bdfp4_decode(const bdfp4_decode_args* args, void* stream);

/*
 * LSE-weighted merge of FP32 partial outputs into BF16.
 * Replaces combine_split_partials / SplitKCombine (src/nvfp4_decode_kernel/split_k_combine.py:13-136).
 * The same call merges partials gathered from several GPUs.
 * partial_out FP32 [parts][rows][Hq][128], partial_lse FP32 [parts][rows][Hq], out BF16 [rows][Hq][128].
 */
int bdfp4_combine(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                  int32_t heads_q, void* out, int64_t out_row_stride, void* stream);

/*
 * The same merge with explicit distances (in floats) between consecutive parts, for partials that
 * arrive as one gathered record per part, e.g. [O | LSE] blocks received from other GPUs by one
 * all-gather: the KV-axis split of a single long sequence across GPUs. Merge math as above
 * (src/nvfp4_decode_kernel/split_k_combine.py:62-83); the reference has no multi-GPU merge.
 */
/* Merge into another partial instead of the BF16 output: record_out FP32 [rows][Hq][128] normalised,
 * record_lse FP32 [rows][Hq] = the natural-log LSE of all parts together (-inf when none
 * contributed). A rank of a KV-axis shard folds its own split-KV parts with it into the one record
 * it sends to the other ranks. */
int bdfp4_combine_record(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                         int32_t heads_q, float* record_out, float* record_lse, void* stream);
int bdfp4_combine_strided(const float* partial_out, int64_t out_part_stride, const float* partial_lse,
                          int64_t lse_part_stride, int32_t parts, int32_t rows, int32_t heads_q, void* out,
                          int64_t out_row_stride, void* stream);

/*
 * The exchange step of a KV-axis shard as one kernel over peer memory (no counterpart in the
 * reference, which has no multi-GPU path; it replaces bdfp4_combine_record + an all-gather +
 * bdfp4_combine_strided). Every rank owns an exchange region of bdfp4_exchange_bytes(world, rows,
 * heads_q) bytes, allocated with bdfp4_peer_alloc (zeroed; exported as a 64-byte CUDA IPC handle) and
 * mapped by the other ranks with bdfp4_peer_open. One call per rank and step: the kernel folds this
 * rank's `parts` split partials (layout of bdfp4_decode's partial_out / partial_lse) into its [O | LSE]
 * record, stores the record into every rank's region (plain stores to peer addresses), flags it, waits
 * - at most two seconds, then BDFP4_DEV_WAIT_TIMEOUT in `error_word` - for the other ranks' records
 * of the same `step` to arrive in its own region, and merges them in rank order into `out` (BF16
 * [rows][out_row_stride]) with the arithmetic of bdfp4_combine. `step` must change on every call and
 * never be 0; all ranks pass the same value. One process per GPU: the kernels of different ranks wait
 * for each other and must not share a GPU. The peer_* calls allocate, map and synchronise: set-up only.
 */
typedef struct bdfp4_exchange_args {
  const float* partial_out; /* this rank's split partials, [parts][rows][heads_q][128] */
  const float* partial_lse; /* [parts][rows][heads_q], natural log */
  int32_t parts;
  int32_t rows;
  int32_t heads_q;
  int32_t world; /* 1..8 */
  int32_t rank;
  uint32_t step;
  void* regions[8]; /* every rank's exchange region as mapped in this process; regions[rank] is the own one */
  void* out;
  int64_t out_row_stride;
  int32_t* error_word; /* optional */
} bdfp4_exchange_args;

int64_t bdfp4_exchange_bytes(int32_t world, int32_t rows, int32_t heads_q);
int bdfp4_peer_alloc(int64_t bytes, void** local, void* handle /* 64 bytes out */);
int bdfp4_peer_open(const void* handle /* 64 bytes */, void** mapped);
int bdfp4_peer_close(void* mapped);
int bdfp4_peer_free(void* local);
int bdfp4_exchange_merge(const bdfp4_exchange_args* args, void* stream);

/*
 * One step of the device-side slot table that maps the rows of a batch to BF16 tail slots and
 * derives each row's sink / FP4 / rolling-tail lengths and promotion target, with no value read
 * back to the host. Replaces ControlPlane.prepare and its Triton kernel _control_kernel
 * (src/nvfp4_vllm/control.py:140-370, 491-561).
 *
 * A row is keyed on column 0 of its block-table row. Rows i < num_reqs with seq_lens[i] > 0 and a
 * key other than the null block 0 are live; a live row keeps the slot holding its key or takes
 * the least recently seen slot no live row claimed. Outputs are written for indices [0, num_slots):
 * row_to_slot (-1 for a dead row), seqused_sink = min(seq, sink_tokens), seqused_fp4 =
 * ((seq-1)/128)*128, seqused_residual = seq - fp4, promotion_source_tokens = slot*(128+sink_tokens),
 * promotion_pages = the block of page fp4/128 when seq % 128 == 0 else -1; token_to_slot for
 * [0, num_actual_tokens). Violated assumptions are OR-ed into *error_code:
 * 1 continuation prefill, 2 slot lost, 4 stale slot history, 8 no free slot, 16 duplicate key,
 * 32 promotion column past the block table (src/nvfp4_vllm/control.py:107-124).
 */
typedef struct bdfp4_control_args {
  const int32_t* block_table; /* int32 [>=num_reqs][block_table_stride] */
  int64_t block_table_stride;
  int32_t block_table_columns;
  const int32_t* seq_lens;        /* [num_reqs] */
  const int32_t* query_start_loc; /* [num_reqs + 1] */
  int32_t* slot_keys;             /* [num_slots] persistent: block id owning the slot, -1 free */
  int32_t* slot_last_seq;         /* [num_slots] persistent */
  int64_t* slot_last_seen;        /* [num_slots] persistent: step the slot was last owned */
  int64_t* step;                  /* [1] persistent counter */
  int32_t* row_to_slot;           /* [num_slots] */
  int32_t* token_to_slot;         /* [>= num_actual_tokens] */
  int32_t* seqused_sink;          /* [num_slots] */
  int32_t* seqused_fp4;
  int32_t* seqused_residual;
  int32_t* promotion_source_tokens;
  int32_t* promotion_pages;
  int32_t* error_code; /* [1] sticky */
  int32_t num_reqs;    /* <= 256 */
  int32_t num_actual_tokens;
  int32_t num_slots;   /* <= 256 (the reference supports at most 128) */
  int32_t sink_tokens;
} bdfp4_control_args;

int bdfp4_control_step(const bdfp4_control_args* args, void* stream);

/*
 * The quantizer's per-step page work table: slot (row, column) reads tokens
 * query_start_loc[row] + 128*column and writes block_table[row][column] when the row is a fresh
 * prefill (more than one token this step, a slot, column < seqused_fp4/128), else -1.
 * Replaces _work_table_kernel (src/nvfp4_vllm/write.py:28-78).
 */
int bdfp4_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4, const int32_t* row_to_slot,
                     const int32_t* block_table, int64_t block_table_stride, int32_t* source_tokens,
                     int32_t* destination_pages, int32_t num_reqs, int32_t columns_per_row, void* stream);

/*
 * Zero every layer's BF16 tail page (page_elems = (128+sink)*H*128 elements) of the rows that start
 * a request this step (seq_len <= tokens brought), so a recycled slot never shows stale tokens.
 * Replaces _tail_reset_kernel (src/nvfp4_vllm/write.py:81-165). Strides in elements.
 */
int bdfp4_tail_reset(void* tail_key, void* tail_value, int64_t layer_stride, int64_t slot_stride, int32_t layers,
                     int64_t page_elems, const int32_t* query_start_loc, const int32_t* seq_lens,
                     const int32_t* row_to_slot, int32_t num_reqs, void* stream);

/*
 * Split-KV decode for callers that must not allocate device memory. It has no counterpart in the
 * reference, whose split path always takes (or allocates) its partial buffers through torch.
 *
 * Who needs it: a serving engine that has given its whole HBM budget to the KV cache and decodes
 * with its allocator frozen, a plugin entered while the host framework holds its memory pool, or an
 * embedding that has no access to the framework's allocator. For them the FP32 partial outputs and
 * log-sum-exps of the split path live in a fixed array inside this library's device image instead of
 * in caller memory: BDFP4_STATIC_SCRATCH_BYTES on every GPU that loads the library, held until the
 * process exits. The call runs bdfp4_decode with `num_splits` (>= 2) parts into that array and then
 * bdfp4_combine into `out`; `partial_out` / `partial_lse` of `args` are ignored. It calls no
 * cudaMalloc/cudaFree and no allocating library routine.
 *
 * Limit: (num_splits + bf16_split) * rows * heads_q * 129 floats must fit in the array, otherwise
 * BDFP4_E_TOO_LARGE is returned and nothing is launched (8 MiB: e.g. 64 rows x 32 heads x 7 parts).
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call outside any stream capture.
 * The array is shared by every call and keeps the previous call's contents. Nothing in it has to
 * start at zero: each part writes its log-sum-exp on every call (-inf when it had no work) and the
 * merge adds a partial only under a positive weight. Two calls that overlap on the GPU (different
 * streams, or different host threads) race on the array; serialise them on one stream.
 * A fused merge is never used here: `merge_counters` of `args` is ignored. The array's address is
 * remembered per device for the life of the process; after cudaDeviceReset it is stale, so a process
 * that resets a device must not call this entry point on it again.
 */
#define BDFP4_STATIC_SCRATCH_BYTES (8u << 20)
int bdfp4_decode_split_static(const bdfp4_decode_args* args, void* stream);

/*
 * Calibration producers (run once before serving, over one long prefill).
 *
 * bdfp4_key_channel_sums: sums[h][c] += sum over `tokens` of key[t][h][c], in FP64; the mean of
 * the post-RoPE keys is what static key smoothing subtracts. `key` is BF16 [tokens][H][128] with
 * `token_pitch` elements between tokens, `sums` FP64 [H][128] (caller-zeroed at the start of a
 * measurement). Replaces the accumulation of src/nvfp4_vllm/impl.py:209-216.
 *
 * bdfp4_probability_statistics: per-E4M3-code statistics of the FP4 probability operand, from
 * FP32 attention scores [heads][tokens] (row_stride floats between heads) of one query position.
 * Pages are walked newest first as decode does; each 16-token group of the FP4 prefix
 * (fp4_tokens, a multiple of 128; the first sink_tokens positions of page 0 masked) is formed
 * against the running maximum held at its page, multiplied by `multiplier`, and priced under the
 * scale divisors 6, 4, 3, 2 (in that order). Bucketed by the E4M3 code of the group maximum and
 * ADDED to the outputs: group_counts u64 [256], winner_counts u64 [256][4] (lowest error, first
 * wins), error_sums f64 [256][4], oracle_sums f64 [256] (error of the winner).
 * page_max_scratch: FP32 [heads][fp4_tokens/128 + 1]. Replaces online_probability_scale_statistics
 * (src/nvfp4_decode_kernel/reference.py:758-871).
 */
int bdfp4_key_channel_sums(const void* key, int64_t token_pitch, int64_t tokens, int32_t heads, double* sums,
                           void* stream);
int bdfp4_probability_statistics(const float* scores, int64_t row_stride, int32_t heads, int32_t tokens,
                                 int32_t fp4_tokens, float softmax_scale, int32_t sink_tokens, float multiplier,
                                 float* page_max_scratch, uint64_t* group_counts, uint64_t* winner_counts,
                                 double* error_sums, double* oracle_sums, void* stream);

/*
 * MLA latent-cache decode (one compressed KV shared by all query heads). The reference has no
 * code for it (src/nvfp4_vllm/backend.py:102 only forwards `use_mla`; head_dim is pinned to 128
 * at backend.py:112-117), so this layout is this library's own:
 *
 * A token is a 512-channel latent plus a 64-channel BF16 rope key. The latent is cached twice in
 * NVFP4, as four 128-channel pseudo heads of 64-token pages written by bdfp4_kv_write with
 * heads = 4, page_tokens = 64 and the latent given as both `key` and `value`:
 *   key regions   (scales along channels)  feed the score product  q_latent . latent
 *   value regions (scales along tokens)    feed the output product P . latent
 * (a block-scaled MMA needs its scales along the contraction axis, which is the channel axis for
 * the first product and the token axis for the second). Rope keys are cached in BF16 by
 * bdfp4_mla_write_rope, one 8 KB block per page: token t's 128 bytes with 16-byte chunk j stored
 * at position j ^ (t & 7), the shared-memory image the decode kernel's BF16 MMA reads.
 * Bytes per token: 2 x (256 + 32) + 128 = 704.
 *
 * bdfp4_mla_quantize_query: BF16 absorbed query [rows][heads_q][512] (row pitch in elements)
 *   -> codes [rows][heads_q][256] and E4M3 scales [rows][heads_q][32], scale_mode as the K/V modes.
 * bdfp4_mla_decode: out[r][h][:] = softmax_t(scale * (q_latent.latent_t + q_rope.rope_t)) . latent,
 *   BF16 [rows][heads_q][512]; probabilities are quantized per 16 tokens exactly as bdfp4_decode
 *   does (same stale-maximum rule and p_scale_mode). heads_q must be a multiple of 64. The row's
 *   page table lists its 64-token pages oldest first; every listed page must have been written in
 *   full; positions at or past seq_lens[r] are masked. With num_splits > 1 the parts leave FP32
 *   partials [parts][rows][heads_q][512] and natural-log LSEs [parts][rows][heads_q] for
 *   bdfp4_mla_combine.
 */
typedef struct bdfp4_mla_decode_args {
  int32_t rows, heads_q;
  const void* query_codes;  /* u8 [rows][heads_q][256] */
  const void* query_scales; /* u8 [rows][heads_q][32] */
  const void* query_rope;   /* BF16 [rows][heads_q][64] */
  const void* key_codes;    /* the four cache regions of bdfp4_kv_write (heads = 4, page_tokens = 64) */
  const void* key_scales;
  const void* value_codes;
  const void* value_scales;
  int64_t key_codes_pitch, key_scales_pitch, value_codes_pitch, value_scales_pitch; /* bytes per page */
  const void* rope_pages;   /* BF16, 8192 bytes per page at rope_pitch bytes */
  int64_t rope_pitch;
  int32_t pages;
  const int32_t* page_table; /* [rows][page_table_stride] 64-token pages, oldest first; a row's length is
                                cut to the 64 * page_table_stride tokens its entries can cover */
  int64_t page_table_stride;
  const int32_t* seq_lens;   /* [rows] tokens */
  float softmax_scale;
  int32_t p_scale_mode;      /* BDFP4_P_* */
  float p_scale_tau;
  void* out;                 /* BF16 [rows][heads_q][512]; used when num_splits == 1 */
  int32_t num_splits;
  float* partial_out;
  float* partial_lse;
  int32_t* error_word;
} bdfp4_mla_decode_args;

int bdfp4_mla_quantize_query(const void* query, int64_t row_pitch, int32_t rows, int32_t heads_q, int32_t scale_mode,
                             void* codes, void* scales, void* stream);
/* rope: BF16 [tokens][64] with token_pitch elements between tokens; work item i copies tokens
 * source_tokens[i] .. +63 into page destination_pages[i] (negative: skipped). */
int bdfp4_mla_write_rope(const void* rope, int64_t token_pitch, const int32_t* source_tokens,
                         const int32_t* destination_pages, int32_t work_items, void* rope_pages, int64_t rope_pitch,
                         void* stream);
/* One new token per row: row r's token number seq_lens[r] (its length before the call) goes to
 * position seq_lens[r] % 64 of the row's open page in the BF16 staging buffers (latent
 * [rows][64][512], rope [rows][64][64]; a page that starts here has its other positions zeroed), and
 * the work table of the page writers is filled: source_tokens[r] = 64 r (a token index into the
 * staging buffers), destination_pages[r] = page_table[r][seq_lens[r] / 64] (-1 and BDFP4_DEV_BAD_PAGE
 * when that column is past page_table_columns, the row being full, or the entry is not a page of
 * the cache; the token is then staged but written to no page). bdfp4_kv_write and bdfp4_mla_write_rope over that table
 * then re-quantize every row's open page, so the cache always holds all tokens in NVFP4. */
int bdfp4_mla_append(const void* new_latent, const void* new_rope, void* staging_latent, void* staging_rope,
                     const int32_t* seq_lens, const int32_t* page_table, int64_t page_table_stride,
                     int32_t page_table_columns, int32_t rows, int32_t pages, int32_t* source_tokens,
                     int32_t* destination_pages, int32_t* error_word, void* stream);
int bdfp4_mla_decode(const bdfp4_mla_decode_args* args, void* stream);
int bdfp4_mla_combine(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                      int32_t heads_q, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BDFP4_H_ */
