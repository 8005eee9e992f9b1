// Calibration producers: the per-channel key sums behind static key smoothing and the
// per-E4M3-code error statistics the probability-scale threshold tau is fitted from.
// Neither is on the serving path; both run once, before serving, over one long prefill.
#include <cmath>

#include "common.cuh"
#include "host.h"

namespace bdfp4 {

// ---- key channel sums --------------------------------------------------------------------------
// sums[h][c] += sum over tokens of key[t][h][c], accumulated in FP64
// (src/nvfp4_vllm/impl.py:209-216 adds `key[:n].double().sum(dim=0)` to the same accumulator).
// One CTA walks a run of tokens for one head; thread c owns channel c, so a token row is one
// coalesced 256-byte read.
__global__ void __launch_bounds__(128) key_sum_kernel(const __nv_bfloat16* __restrict__ key, int64_t token_pitch,
                                                      int64_t tokens, int64_t tokens_per_cta,
                                                      double* __restrict__ sums) {
  const int head = blockIdx.x;
  const int channel = threadIdx.x;
  const int64_t begin = (int64_t)blockIdx.y * tokens_per_cta;
  const int64_t end = min(begin + tokens_per_cta, tokens);
  const __nv_bfloat16* column = key + (int64_t)head * kHeadDim + channel;
  double total = 0.0;
  int64_t t = begin;
  for (; t + 4 <= end; t += 4) {
    const float a = __bfloat162float(column[t * token_pitch]);
    const float b = __bfloat162float(column[(t + 1) * token_pitch]);
    const float c = __bfloat162float(column[(t + 2) * token_pitch]);
    const float d = __bfloat162float(column[(t + 3) * token_pitch]);
    total += ((double)a + (double)b) + ((double)c + (double)d);
  }
  for (; t < end; ++t) total += (double)__bfloat162float(column[t * token_pitch]);
  if (begin < end) atomicAdd(&sums[(int64_t)head * kHeadDim + channel], total);
}

// ---- probability-scale statistics --------------------------------------------------------------
// For every 16-token group of the FP4 pages' softmax probabilities (formed against the running
// maximum the reverse-page online softmax holds when it reaches the page), the squared
// reconstruction error of the FP4 probability operand under each scale divisor 6, 4, 3, 2,
// bucketed by the E4M3 code of the group's maximum
// (src/nvfp4_decode_kernel/reference.py:758-871).

constexpr int kDivisors = 4;

// Pass 1: maxima of the scaled scores of every page (page 0 without its sink positions) and, in
// slot `pages`, of the tokens past the FP4 prefix.
__global__ void __launch_bounds__(128) page_max_kernel(const float* __restrict__ scores, int64_t row_stride, int tokens,
                                                       int fp4_tokens, float softmax_scale, int sink_tokens,
                                                       float* __restrict__ page_max) {
  __shared__ float warp_max[4];
  const int pages = fp4_tokens / kPage;
  const int head = blockIdx.y;
  const int page = blockIdx.x;  // == pages: the tail
  const float* row = scores + (int64_t)head * row_stride;
  float m = -INFINITY;
  if (page < pages) {
    const int token = page * kPage + threadIdx.x;
    if (!(page == 0 && (int)threadIdx.x < sink_tokens)) m = __fmul_rn(row[token], softmax_scale);
  } else {
    for (int token = fp4_tokens + threadIdx.x; token < tokens; token += 128)
      m = fmaxf(m, __fmul_rn(row[token], softmax_scale));
  }
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, step));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0)
    page_max[(int64_t)head * (pages + 1) + page] = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
}

// Pass 2: one CTA per (page, head), one thread per token.
__global__ void __launch_bounds__(128) probability_statistics_kernel(
    const float* __restrict__ scores, int64_t row_stride, int fp4_tokens, float softmax_scale, int sink_tokens,
    float multiplier, const float* __restrict__ page_max, unsigned long long* __restrict__ group_counts,
    unsigned long long* __restrict__ winner_counts, double* __restrict__ error_sums, double* __restrict__ oracle_sums) {
  __shared__ float suffix;
  const int pages = fp4_tokens / kPage;
  const int head = blockIdx.y;
  const int page = blockIdx.x;
  if (threadIdx.x < 32) {
    // maximum over this page, every newer page and the tail: what the walk (newest first) holds here
    const float* maxima = page_max + (int64_t)head * (pages + 1);
    float m = -INFINITY;
    for (int i = page + threadIdx.x; i <= pages; i += 32) m = fmaxf(m, maxima[i]);
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, step));
    if (threadIdx.x == 0) suffix = (m == -INFINITY || m != m || m == INFINITY) ? 0.0f : m;
  }
  __syncthreads();
  const int token = page * kPage + threadIdx.x;
  const bool masked = page == 0 && (int)threadIdx.x < sink_tokens;
  const float scaled = masked ? -INFINITY : __fmul_rn(scores[(int64_t)head * row_stride + token], softmax_scale);
  const float probability = scaled == -INFINITY ? 0.0f : expf(__fsub_rn(scaled, suffix));
  const float value = __fmul_rn(probability, multiplier);
  float maximum = value;
#pragma unroll
  for (int step = 1; step < 16; step <<= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, step));
  const uint32_t code = cvt_e4m3(maximum) & 0xffu;
  const float reciprocals[kDivisors] = {(float)(1.0 / 6.0), (float)(1.0 / 4.0), (float)(1.0 / 3.0), (float)(1.0 / 2.0)};
  float error[kDivisors];
#pragma unroll
  for (int d = 0; d < kDivisors; ++d) {
    const float raw_scale = __fmul_rn(maximum, reciprocals[d]);
    const float stored = e4m3_to_float(cvt_e4m3(fminf(raw_scale, 448.0f)));
    const float quotient = __fdiv_rn(value, fmaxf(raw_scale, 1.0e-30f));
    const float magnitude = e2m1x2_to_float2(cvt_e2m1x2(quotient, 0.0f)).x;
    const float difference = __fsub_rn(__fmul_rn(magnitude, stored), value);
    float e = __fmul_rn(difference, difference);
#pragma unroll
    for (int step = 1; step < 16; step <<= 1) e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, step));
    error[d] = e;
  }
  if ((threadIdx.x & 15) == 0) {
    int winner = 0;
#pragma unroll
    for (int d = 1; d < kDivisors; ++d)
      if (error[d] < error[winner]) winner = d;
    atomicAdd(&group_counts[code], 1ull);
    atomicAdd(&winner_counts[code * kDivisors + winner], 1ull);
#pragma unroll
    for (int d = 0; d < kDivisors; ++d) atomicAdd(&error_sums[code * kDivisors + d], (double)error[d]);
    atomicAdd(&oracle_sums[code], (double)error[winner]);
  }
}

}  // namespace bdfp4

using namespace bdfp4;

extern "C" int bdfp4_key_channel_sums(const void* key, int64_t token_pitch, int64_t tokens, int32_t heads, double* sums,
                                      void* stream_handle) {
  if (!key || !sums || heads < 1 || tokens < 0 || token_pitch < (int64_t)heads * kHeadDim) return BDFP4_E_ARG;
  if (tokens == 0) return BDFP4_OK;
  // about four CTAs per SM, never fewer than 64 tokens per CTA
  int64_t chunks = (4 * 148 + heads - 1) / heads;
  const int64_t most = (tokens + 63) / 64;
  if (chunks > most) chunks = most;
  if (chunks > 65535) chunks = 65535;
  const int64_t tokens_per_cta = (tokens + chunks - 1) / chunks;
  key_sum_kernel<<<dim3(heads, (unsigned)chunks), 128, 0, static_cast<cudaStream_t>(stream_handle)>>>(
      static_cast<const __nv_bfloat16*>(key), token_pitch, tokens, tokens_per_cta, sums);
  return cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_probability_statistics(const float* scores, int64_t row_stride, int32_t heads, int32_t tokens,
                                            int32_t fp4_tokens, float softmax_scale, int32_t sink_tokens,
                                            float multiplier, float* page_max_scratch, uint64_t* group_counts,
                                            uint64_t* winner_counts, double* error_sums, double* oracle_sums,
                                            void* stream_handle) {
  if (!scores || !page_max_scratch || !group_counts || !winner_counts || !error_sums || !oracle_sums)
    return BDFP4_E_ARG;
  if (heads < 1 || heads > 65535 || tokens < 1 || row_stride < tokens) return BDFP4_E_ARG;
  if (fp4_tokens <= 0 || fp4_tokens > tokens || fp4_tokens % kPage) return BDFP4_E_ARG;
  if (sink_tokens < 0 || sink_tokens > kPage) return BDFP4_E_ARG;
  if (!(multiplier > 0.0f) || !(multiplier <= 448.0f) || !(softmax_scale > 0.0f) || !std::isfinite(softmax_scale))
    return BDFP4_E_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const int pages = fp4_tokens / kPage;
  page_max_kernel<<<dim3(pages + 1, heads), 128, 0, stream>>>(scores, row_stride, tokens, fp4_tokens, softmax_scale,
                                                               sink_tokens, page_max_scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_status(e);
  probability_statistics_kernel<<<dim3(pages, heads), 128, 0, stream>>>(
      scores, row_stride, fp4_tokens, softmax_scale, sink_tokens, multiplier, page_max_scratch,
      reinterpret_cast<unsigned long long*>(group_counts), reinterpret_cast<unsigned long long*>(winner_counts),
      error_sums, oracle_sums);
  return cuda_status(cudaGetLastError());
}
