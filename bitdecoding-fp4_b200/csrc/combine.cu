// LSE-weighted merge of split-KV (or multi-GPU KV-shard) partial outputs into BF16.
// One CTA per (row, query head), one thread per channel; a partial is added only under a
// positive weight so an unwritten slot (its LSE is -inf) can never leak into the output
// (src/nvfp4_decode_kernel/split_k_combine.py:47-83).
#include "common.cuh"
#include "host.h"
#include "merge.cuh"

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
  // Launched with programmatic stream serialization: the CTAs may be resident before the decode
  // launch that writes the partials has finished, so its results are waited for here; the launch
  // behind this one (the next step's query quantizer) may then bring its CTAs up in turn.
  wait_for_prior_kernels();
  dependents_may_launch();

  const float acc = fold_parts(values, out_stride, lse, lse_stride, parts, channel, nullptr);
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
  wait_for_prior_kernels();
  dependents_may_launch();
  float folded_lse;
  const float acc = fold_parts(values, lse_stride * kHeadDim, lse, lse_stride, parts, channel, &folded_lse);
  record_out[((int64_t)row * heads_q + head) * kHeadDim + channel] = acc;
  if (channel == 0) record_lse[(int64_t)row * heads_q + head] = folded_lse;
}

// After a decode launch of this library (which lets its dependents launch early) the merge's CTAs are
// resident by the time the last partial is written; after anything else this is an ordinary launch.
template <typename... Params, typename... Args>
static cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, cudaStream_t stream, Args... args) {
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

}  // namespace bdfp4

extern "C" int bdfp4_combine_record(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                                    int32_t heads_q, float* record_out, float* record_lse, void* stream) {
  if (!partial_out || !partial_lse || !record_out || !record_lse || parts < 1 || rows < 1 || heads_q < 1)
    return BDFP4_E_ARG;
  return bdfp4::cuda_status(bdfp4::launch_overlapped(bdfp4::combine_record_kernel, dim3(heads_q, rows),
                                                     static_cast<cudaStream_t>(stream), partial_out, partial_lse,
                                                     (int)parts, (int)rows, (int)heads_q, record_out, record_lse));
}

extern "C" int bdfp4_combine_strided(const float* partial_out, int64_t out_part_stride, const float* partial_lse,
                                     int64_t lse_part_stride, int32_t parts, int32_t rows, int32_t heads_q,
                                     void* out, int64_t out_row_stride, void* stream) {
  if (!partial_out || !partial_lse || !out || parts < 1 || rows < 1 || heads_q < 1) return BDFP4_E_ARG;
  if (out_row_stride < (int64_t)heads_q * bdfp4::kHeadDim) return BDFP4_E_ARG;
  if (out_part_stride < (int64_t)rows * heads_q * bdfp4::kHeadDim || lse_part_stride < (int64_t)rows * heads_q)
    return BDFP4_E_ARG;
  return bdfp4::cuda_status(bdfp4::launch_overlapped(
      bdfp4::combine_kernel, dim3(heads_q, rows), static_cast<cudaStream_t>(stream), partial_out, partial_lse,
      (int)parts, (int)rows, (int)heads_q, static_cast<__nv_bfloat16*>(out), out_row_stride, out_part_stride,
      lse_part_stride));
}

extern "C" int bdfp4_combine(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                             int32_t heads_q, void* out, int64_t out_row_stride, void* stream) {
  return bdfp4_combine_strided(partial_out, (int64_t)rows * heads_q * bdfp4::kHeadDim, partial_lse,
                               (int64_t)rows * heads_q, parts, rows, heads_q, out, out_row_stride, stream);
}
