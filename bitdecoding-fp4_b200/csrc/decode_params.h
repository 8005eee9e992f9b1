// Launch parameters of the paged FP4 decode kernel and the entry points of its instantiation
// units. The kernel template lives in decode_kernel.cuh and is instantiated in three translation
// units (NVFP4 with 128-token pages, NVFP4 with 64-token pages, MXFP4) so that they compile side by
// side; decode.cu holds the C ABI and picks one of them.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bdfp4 {

struct DecodeParams {
  int rows, heads_q, heads_kv, ratio;
  const uint8_t* q_codes[2];
  const uint8_t* q_scales[2];
  const __nv_bfloat16* q_padded;
  const uint8_t* k_scales;
  const uint8_t* v_scales;
  int64_t k_scales_pitch, v_scales_pitch;
  const uint8_t* k_codes;  // 64-token pages are fetched with bulk copies, not through the tensor maps
  const uint8_t* v_codes;
  int64_t k_codes_pitch, v_codes_pitch;
  int pages;
  const int32_t* page_table;
  int64_t page_table_stride;
  int max_pages;
  const int32_t* seqused_fp4;
  const __nv_bfloat16* tail_key;
  const __nv_bfloat16* tail_value;
  int64_t tail_slot_stride;
  int tail_slots;
  const int32_t* tail_slot_ids;
  const int32_t* seqused_residual;
  const int32_t* seqused_sink;
  // Softmax scale in log2 units times the score tensor scale (key x query tensor scales): scores are
  // kept in the units the FP4 MMAs deliver, and so are the outputs. The BF16 blocks are converted
  // into those units (scores times bf16_score_scale = 1 / score scale, outputs times
  // bf16_value_scale = 1 / value tensor scale) and the final output is multiplied by out_scale =
  // value tensor scale. All three are exactly 1 without tensor scales.
  float scale_log2;
  float bf16_score_scale, bf16_value_scale, out_scale;
  int p_mode;
  float tau;
  __nv_bfloat16* out;
  int64_t out_row_stride;
  int num_splits, bf16_split, parts, bf16_page_cost;
  float* partial_out;
  float* partial_lse;
  int32_t* error_word;
  // fused merge: the last part of a (row, KV head) tile to finish writes the BF16 output
  int32_t* merge_counters;
  __nv_bfloat16* merged_out;
  const int32_t* row_order;  // launch position -> row (longest rows first), or null
  const int32_t* row_splits;  // parts per row (1..num_splits), or null: num_splits for every row
};

// One launch of decode_kernel<GP, TERMS, STAGES, PT, MX> with GP the smallest of 4, 8, 16 that holds
// `p.ratio` query heads per KV head, TERMS = 2 when `two_terms`, and the ring depth chosen from the
// grid size. Defined in decode_nvfp4_p128.cu, decode_nvfp4_p64.cu and decode_mxfp4.cu.
cudaError_t launch_decode_nvfp4_p128(bool two_terms, const CUtensorMap& k_map, const CUtensorMap& v_map,
                                     const DecodeParams& p, cudaStream_t stream);
cudaError_t launch_decode_nvfp4_p64(bool two_terms, const CUtensorMap& k_map, const CUtensorMap& v_map,
                                    const DecodeParams& p, cudaStream_t stream);
cudaError_t launch_decode_mxfp4(bool two_terms, const CUtensorMap& k_map, const CUtensorMap& v_map,
                                const DecodeParams& p, cudaStream_t stream);

}  // namespace bdfp4
