// The LSE-weighted fold of split-KV parts that the merge kernels share: one CTA of 128 threads per
// (row, query head), one thread per channel (src/nvfp4_decode_kernel/split_k_combine.py:47-83).
// A merge runs after the launch it depends on, with nothing else to overlap, so its own load
// latencies are its whole cost: the parts' LSEs come in with ONE parallel load into shared memory
// instead of three dependent passes over global memory, and a channel's partial values are fetched
// eight parts at a time before any of them is used. The arithmetic and its order (part order) are
// unchanged, so a given set of partials always folds to the same bits.
#pragma once

#include "common.cuh"

namespace bdfp4 {

constexpr int kFoldStaged = 256;  // parts whose LSEs fit the staging array; beyond it they are re-read

// Returns the folded, normalised value of this thread's channel; `*lse_out` gets the natural-log LSE of
// all parts together (-inf when none contributed). `values` / `lse` point at this thread's channel /
// this CTA's (row, head) in part 0; consecutive parts are `value_stride` / `lse_stride` floats apart.
// Every thread of the CTA must call it (it holds CTA barriers).
__device__ __forceinline__ float fold_parts(const float* values, int64_t value_stride, const float* lse,
                                            int64_t lse_stride, int parts, int thread, float* lse_out) {
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ float staged[kFoldStaged];
  for (int s = thread; s < min(parts, kFoldStaged); s += 128) staged[s] = __ldcg(lse + s * lse_stride);
  __syncthreads();
  auto lse_of = [&](int s) { return s < kFoldStaged ? staged[s] : __ldcg(lse + s * lse_stride); };
  float lse_max = -INFINITY;
  for (int s = 0; s < parts; ++s) lse_max = fmaxf(lse_max, lse_of(s));
  const bool empty = lse_max == -INFINITY;
  if (empty) lse_max = 0.0f;
  float weight_sum = 0.0f;
  for (int s = 0; s < parts; ++s) weight_sum += exp2f(lse_of(s) * kLog2e - lse_max * kLog2e);
  const float inverse = (weight_sum == 0.0f || weight_sum != weight_sum) ? 0.0f : 1.0f / weight_sum;
  float acc = 0.0f;
  for (int s0 = 0; s0 < parts; s0 += 8) {
    float fetched[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) fetched[u] = s0 + u < parts ? __ldcg(values + (s0 + u) * value_stride) : 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (s0 + u < parts) {
        const float scale = exp2f(lse_of(s0 + u) * kLog2e - lse_max * kLog2e) * inverse;
        if (scale > 0.0f) acc = acc + scale * fetched[u];
      }
    }
  }
  if (lse_out) *lse_out = (empty || inverse == 0.0f) ? -INFINITY : lse_max + logf(weight_sum);
  __syncthreads();  // the staging array may be filled again
  return acc;
}

}  // namespace bdfp4
