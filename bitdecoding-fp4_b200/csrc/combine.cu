// LSE-weighted merge of split-KV (or multi-GPU KV-shard) partial outputs into BF16.
// One CTA per (row, query head), one thread per channel; a partial is added only under a
// positive weight so an unwritten slot (its LSE is -inf) can never leak into the output
// (src/nvfp4_decode_kernel/split_k_combine.py:47-83).
#include "common.cuh"
#include "host.h"

namespace bdfp4 {

__global__ void __launch_bounds__(128) combine_kernel(const float* __restrict__ partial_out,
                                                      const float* __restrict__ partial_lse, int parts, int rows,
                                                      int heads_q, __nv_bfloat16* __restrict__ out,
                                                      int64_t out_row_stride, int64_t out_stride,
                                                      int64_t lse_stride) {
  const int head = blockIdx.x;
  const int row = blockIdx.y;
  const int channel = threadIdx.x;
  const float* lse = partial_lse + (int64_t)row * heads_q + head;
  const float* values = partial_out + ((int64_t)row * heads_q + head) * kHeadDim + channel;
  constexpr float kLog2e = 1.4426950408889634f;

  float lse_max = -INFINITY;
  for (int s = 0; s < parts; ++s) lse_max = fmaxf(lse_max, lse[s * lse_stride]);
  if (lse_max == -INFINITY) lse_max = 0.0f;
  float weight_sum = 0.0f;
  for (int s = 0; s < parts; ++s) weight_sum += exp2f(lse[s * lse_stride] * kLog2e - lse_max * kLog2e);
  const float inverse = (weight_sum == 0.0f || weight_sum != weight_sum) ? 0.0f : 1.0f / weight_sum;
  float acc = 0.0f;
  // split order, so a given set of partials always sums to the same bits
  for (int s = 0; s < parts; ++s) {
    const float scale = exp2f(lse[s * lse_stride] * kLog2e - lse_max * kLog2e) * inverse;
    if (scale > 0.0f) acc = acc + scale * values[s * out_stride];
  }
  out[(int64_t)row * out_row_stride + head * kHeadDim + channel] = __float2bfloat16_rn(acc);
}

// The same merge, but into another partial: normalised FP32 output and the natural-log LSE of all
// the parts together, so that a rank can fold its own split-KV parts into the one [O | LSE] record
// it sends to the other ranks.
__global__ void __launch_bounds__(128) combine_record_kernel(const float* __restrict__ partial_out,
                                                             const float* __restrict__ partial_lse, int parts, int rows,
                                                             int heads_q, float* __restrict__ record_out,
                                                             float* __restrict__ record_lse) {
  const int head = blockIdx.x;
  const int row = blockIdx.y;
  const int channel = threadIdx.x;
  const int64_t lse_stride = (int64_t)rows * heads_q;
  const float* lse = partial_lse + (int64_t)row * heads_q + head;
  const float* values = partial_out + ((int64_t)row * heads_q + head) * kHeadDim + channel;
  constexpr float kLog2e = 1.4426950408889634f;
  float lse_max = -INFINITY;
  for (int s = 0; s < parts; ++s) lse_max = fmaxf(lse_max, lse[s * lse_stride]);
  const bool empty = lse_max == -INFINITY;
  if (empty) lse_max = 0.0f;
  float weight_sum = 0.0f;
  for (int s = 0; s < parts; ++s) weight_sum += exp2f(lse[s * lse_stride] * kLog2e - lse_max * kLog2e);
  const float inverse = (weight_sum == 0.0f || weight_sum != weight_sum) ? 0.0f : 1.0f / weight_sum;
  float acc = 0.0f;
  for (int s = 0; s < parts; ++s) {
    const float scale = exp2f(lse[s * lse_stride] * kLog2e - lse_max * kLog2e) * inverse;
    if (scale > 0.0f) acc = acc + scale * values[s * lse_stride * kHeadDim];
  }
  record_out[((int64_t)row * heads_q + head) * kHeadDim + channel] = acc;
  if (channel == 0)
    record_lse[(int64_t)row * heads_q + head] = (empty || inverse == 0.0f) ? -INFINITY : lse_max + logf(weight_sum);
}

}  // namespace bdfp4

extern "C" int bdfp4_combine_record(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                                    int32_t heads_q, float* record_out, float* record_lse, void* stream) {
  if (!partial_out || !partial_lse || !record_out || !record_lse || parts < 1 || rows < 1 || heads_q < 1)
    return BDFP4_E_ARG;
  bdfp4::combine_record_kernel<<<dim3(heads_q, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      partial_out, partial_lse, parts, rows, heads_q, record_out, record_lse);
  return bdfp4::cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_combine_strided(const float* partial_out, int64_t out_part_stride, const float* partial_lse,
                                     int64_t lse_part_stride, int32_t parts, int32_t rows, int32_t heads_q,
                                     void* out, int64_t out_row_stride, void* stream) {
  if (!partial_out || !partial_lse || !out || parts < 1 || rows < 1 || heads_q < 1) return BDFP4_E_ARG;
  if (out_row_stride < (int64_t)heads_q * bdfp4::kHeadDim) return BDFP4_E_ARG;
  if (out_part_stride < (int64_t)rows * heads_q * bdfp4::kHeadDim || lse_part_stride < (int64_t)rows * heads_q)
    return BDFP4_E_ARG;
  bdfp4::combine_kernel<<<dim3(heads_q, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      partial_out, partial_lse, parts, rows, heads_q, static_cast<__nv_bfloat16*>(out), out_row_stride,
      out_part_stride, lse_part_stride);
  return bdfp4::cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_combine(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                             int32_t heads_q, void* out, int64_t out_row_stride, void* stream) {
  return bdfp4_combine_strided(partial_out, (int64_t)rows * heads_q * bdfp4::kHeadDim, partial_lse,
                               (int64_t)rows * heads_q, parts, rows, heads_q, out, out_row_stride, stream);
}
