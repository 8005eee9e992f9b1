// Paged FP4 decode attention for sm_100a.
//
// One CTA serves one (decode row, KV head[, split]). Per 128-token page it streams
//   K codes 8 KB + K scales 1 KB and V codes 8 KB + V scales 1 KB
// from HBM with TMA into shared-memory rings, and runs two block-scaled tcgen05 MMAs with
// accumulators in tensor memory:
//   S^T[token, q] = K[token, :] . Q[q, :]       A = K page  (128 x 128 E2M1), B = Q tile
//   O^T[chan,  q] = V^T[chan, :] . P[q, :]      A = V page  (128 x 128 E2M1), B = P tile
// Both are M = 128, K = 128 (two K = 64 instructions). Transposed this way a softmax thread
// owns one token (TMEM lane) and the G query heads of the KV head are a handful of columns.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (one thread) and TMEM owner, warps 2-5
// softmax: they read S^T with tcgen05.ld, keep the online-softmax statistics, quantize the
// probabilities to E2M1 + E4M3 scales straight into the shared-memory B operand of the PV MMA,
// and accumulate each page's O^T (read back from TMEM) in registers. The BF16 tail (first) and
// sink (last) blocks are at most 144 tokens and are merged by the same warps with plain FMAs.
//
// Block order, masks, the stale-maximum rule and the probability scale rule follow
// src/nvfp4_decode_kernel/fp4_decode_kernel.py:4830-5055,5352-5854 of OpenBitSys/BitDecoding-FP4.
#pragma once

#include <atomic>
#include <cmath>

#include "common.cuh"
#include "decode_params.h"
#include "host.h"
#include "tcgen05.cuh"

namespace bdfp4 {

constexpr int kStageBytes = 8192 + 1024;  // codes + scales of one K or V page-head
constexpr int kNP = 16;                   // N of the PV MMA (query rows, padded)
constexpr float kRescaleThreshold = 8.0f;  // src/nvfp4_decode_kernel/fp4_decode_kernel.py:93

// TMEM column map (32-bit columns): two S^T stages of 16 columns, the O^T sum (16 columns, 16 spare),
// then the scale-factor blocks, 8 columns (two 4-column atoms) each: Q term 0, Q term 1, K x2, V x2,
// P x2. 128 columns in all, so four CTAs share an SM's 512.
constexpr int kNQ = 16;  // N of the QK MMA (query heads of one KV head, padded)
constexpr int kColS = 0;
constexpr int kColO = 32;
constexpr int kColSFQ = 64;
constexpr int kColSFK = 80;
constexpr int kColSFV = 96;
constexpr int kColSFP = 112;
constexpr int kTmemColumns = 128;


template <int GP, int STAGES>
struct DecodeSmem {
  static constexpr int kStages = STAGES;
  alignas(1024) uint8_t k_stage[kStages][kStageBytes];
  alignas(1024) uint8_t v_stage[kStages][kStageBytes];
  alignas(1024) uint8_t q_tile[2][kNQ * 64];  // one B operand per query term
  alignas(1024) uint8_t p_tile[2][kNP * 64];
  alignas(1024) uint8_t q_sf[2][1024];
  alignas(1024) uint8_t p_sf[2][1024];
  float q_bf16[GP][128];  // BF16 query of the tail/sink blocks, widened
  float p_bf16[GP][128];  // BF16-rounded probabilities of a tail/sink block
  float red[2][4][GP];
  float sum_red[4][GP];
  // the rows' running maxima and the two values derived from them: identical in every softmax
  // thread, so with eight or more rows per thread they live here instead of in registers
  float stat_row_max[GP], stat_threshold[GP], stat_max_scaled[GP];
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t ksf_full[kStages];  // K scale blocks of 64-token pages, which arrive ahead of the codes
  uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], o_full[2];
  int pv_fresh[2];  // per P buffer: 1 when its PV product starts a new sum in tensor memory, 0 when it adds
  int page_ids[2][32];  // physical pages of the producer's current batch of steps
  uint32_t tmem_base;
  int abort_flag;
  int merge_last;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void prefetch_l2(const void* address) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(address));
}

// Named barriers of the softmax threads: one per softmax group (ids 1, 2, ...; 128 threads each).
__device__ __forceinline__ void softmax_barrier(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

template <int THREADS>
__device__ __forceinline__ void all_softmax_barrier() {
  asm volatile("bar.sync 15, %0;" ::"n"(THREADS) : "memory");
}

__device__ __forceinline__ bool softmax_vote_any(bool pred, int id) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, %2, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred), "r"(id)
      : "memory");
  return out != 0;
}

// Physical byte offset of logical byte `offset` in a K-major tile of 64-byte rows under the
// 64-byte swizzle: the 16-byte chunk index is XORed with bits [7,9) of the offset.
__device__ __forceinline__ int swizzle64(int offset) { return offset ^ (((offset >> 7) & 3) << 4); }

// Scale of one group of sixteen probabilities from its maximum
// (src/nvfp4_decode_kernel/_fa4/softmax.py:80-112).
__device__ __forceinline__ float probability_scale(float maximum, int p_mode, float tau) {
  float scale = __fmul_rn(maximum, (float)(1.0 / 6.0));
  if (p_mode != BDFP4_P_AMAX6 && maximum <= tau) scale = __fmul_rn(maximum, 0.5f);
  return scale;
}

// Online-softmax state of one softmax thread: the statistics of the KV head's GP query heads
// (row_max identical in every thread, row_sum a per-thread partial) and the output
// accumulator of the thread's channel.
template <int GP>
struct SoftmaxState {
  float row_max[GP];
  float row_sum[GP];
  float o_acc[GP];
  bool first;
};

// Update the running maxima with a block's maxima; returns the factors the previous
// accumulations must be multiplied by and the maximum the block's probabilities are formed
// against (scaled to log2 units, with the c8 shift folded in).
template <int GP>
__device__ __forceinline__ void update_max(SoftmaxState<GP>& st, const float* block_max, float scale_log2,
                                           float shift, float* acc, float* max_scaled) {
#pragma unroll
  for (int j = 0; j < GP; ++j) {
    float new_max, safe;
    if (st.first) {
      new_max = block_max[j];
      safe = new_max == -INFINITY ? 0.0f : new_max;
      acc[j] = 0.0f;
    } else {
      const float old_max = st.row_max[j];
      new_max = fmaxf(old_max, block_max[j]);
      safe = new_max == -INFINITY ? 0.0f : new_max;
      const float growth = (old_max - safe) * scale_log2;
      if (growth >= -kRescaleThreshold) {
        new_max = old_max;
        safe = old_max;
        acc[j] = 1.0f;
      } else {
        acc[j] = ex2_approx(growth);
      }
    }
    st.row_max[j] = new_max;
    max_scaled[j] = safe * scale_log2 - shift;
  }
}

// A BF16 block (the rolling tail or the sink) merged with plain FMAs by the 128 softmax threads:
// thread `t` scores token `t`, then accumulates channel `t`. `rows0` is the first row of the
// block inside the slot's buffer, positions outside [mask_below, length) are masked.
// A softmax group of 128 threads runs it for its own R of the tile's rows, which start at `row0` of the
// shared per-row arrays; `barrier` is the group's named barrier.
template <int R, typename Smem>
__device__ __forceinline__ void bf16_block(SoftmaxState<R>& st, Smem& sm, const DecodeParams& p, int t, int warp_q,
                                           int lane, const __nv_bfloat16* key_rows, const __nv_bfloat16* value_rows,
                                           int mask_below, int length, float shift, int& red_buf, int row0,
                                           int barrier) {
  const int64_t row_elems = (int64_t)p.heads_kv * kHeadDim;
  float s[R];
  const bool valid = t >= mask_below && t < length;
#pragma unroll
  for (int j = 0; j < R; ++j) s[j] = valid ? 0.0f : -INFINITY;
  if (length <= 16) {
    // A short block (the sink): eight lanes share a token, two 16-byte loads each, so the scores
    // cost one load round trip; they travel to the token's own thread through p_bf16.
    const int token = t >> 3, chunk = t & 7;
    const bool scored = token >= mask_below && token < length;
    float dot[R];
#pragma unroll
    for (int j = 0; j < R; ++j) dot[j] = 0.0f;
    if (scored) {
      const uint4* kpart = reinterpret_cast<const uint4*>(key_rows + (int64_t)token * row_elems + chunk * 16);
      const uint4 raw[2] = {__ldg(kpart), __ldg(kpart + 1)};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const float4 q0 = *reinterpret_cast<const float4*>(&sm.q_bf16[row0 + j][chunk * 16 + c * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&sm.q_bf16[row0 + j][chunk * 16 + c * 8 + 4]);
          float a = dot[j];
          a = fmaf(__uint_as_float(w[0] << 16), q0.x, a);
          a = fmaf(__uint_as_float(w[0] & 0xffff0000u), q0.y, a);
          a = fmaf(__uint_as_float(w[1] << 16), q0.z, a);
          a = fmaf(__uint_as_float(w[1] & 0xffff0000u), q0.w, a);
          a = fmaf(__uint_as_float(w[2] << 16), q1.x, a);
          a = fmaf(__uint_as_float(w[2] & 0xffff0000u), q1.y, a);
          a = fmaf(__uint_as_float(w[3] << 16), q1.z, a);
          a = fmaf(__uint_as_float(w[3] & 0xffff0000u), q1.w, a);
          dot[j] = a;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
      dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], 1);
      dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], 2);
      dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], 4);
      if (chunk == 0) sm.p_bf16[row0 + j][token] = dot[j];
    }
    softmax_barrier(barrier);
    if (valid) {
#pragma unroll
      for (int j = 0; j < R; ++j) s[j] = sm.p_bf16[row0 + j][t];
    }
    softmax_barrier(barrier);  // p_bf16 is written again below
  } else if (valid) {
    const uint4* krow = reinterpret_cast<const uint4*>(key_rows + (int64_t)t * row_elems);
    // Eight 16-byte loads are issued before the first is consumed: the block is latency-bound.
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint4 raw[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) raw[c] = __ldg(krow + half * 8 + c);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
        float k[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          k[2 * i] = __uint_as_float(w[i] << 16);
          k[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const float4 q0 = *reinterpret_cast<const float4*>(&sm.q_bf16[row0 + j][(half * 8 + c) * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&sm.q_bf16[row0 + j][(half * 8 + c) * 8 + 4]);
          float a = s[j];
          a = fmaf(k[0], q0.x, a);
          a = fmaf(k[1], q0.y, a);
          a = fmaf(k[2], q0.z, a);
          a = fmaf(k[3], q0.w, a);
          a = fmaf(k[4], q1.x, a);
          a = fmaf(k[5], q1.y, a);
          a = fmaf(k[6], q1.z, a);
          a = fmaf(k[7], q1.w, a);
          s[j] = a;
        }
      }
    }
  }
  // Scores and outputs of the FP4 pages stay in the units the MMAs deliver them in; with per-tensor
  // scales the BF16 blocks are brought into those units instead (both factors are exactly 1 without).
#pragma unroll
  for (int j = 0; j < R; ++j) s[j] *= p.bf16_score_scale;
  float block_max[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    float m = s[j];
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, step));
    block_max[j] = m;
  }
  if (lane < R) {
    float mine = block_max[0];
#pragma unroll
    for (int j = 1; j < R; ++j) mine = lane == j ? block_max[j] : mine;
    sm.red[red_buf][warp_q][row0 + lane] = mine;
  }
  softmax_barrier(barrier);
#pragma unroll
  for (int j = 0; j < R; ++j)
    block_max[j] = fmaxf(fmaxf(sm.red[red_buf][0][row0 + j], sm.red[red_buf][1][row0 + j]),
                         fmaxf(sm.red[red_buf][2][row0 + j], sm.red[red_buf][3][row0 + j]));
  red_buf ^= 1;
  float acc[R], max_scaled[R];
  update_max<R>(st, block_max, p.scale_log2, shift, acc, max_scaled);
  st.first = false;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const float prob = ex2_approx(s[j] * p.scale_log2 - max_scaled[j]);
    st.row_sum[j] = st.row_sum[j] * acc[j] + prob;
    sm.p_bf16[row0 + j][t] = __bfloat162float(__float2bfloat16_rn(prob));
    st.o_acc[j] *= acc[j];
  }
  softmax_barrier(barrier);
  // PV. The loop is bound by load latency, so each lane keeps sixteen 8-byte loads in flight:
  // a warp owns 32 channels, lane = (token phase lane >> 3, channel quad lane & 7) accumulates
  // tokens phase, phase + 4, ... for its four channels. A masked position carries probability
  // zero and reads row `length - 1`, so the loop has no bounds branch.
  if (length > 0) {
    const int phase = lane >> 3;
    const uint2* vquad = reinterpret_cast<const uint2*>(value_rows + warp_q * 32 + (lane & 7) * 4);
    const int64_t row_quads = row_elems / 4;
    float part[R][4];
#pragma unroll
    for (int j = 0; j < R; ++j) part[j][0] = part[j][1] = part[j][2] = part[j][3] = 0.0f;
#pragma unroll 1
    for (int base = 0; base < length; base += 64) {
      uint2 raw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) raw[i] = __ldg(vquad + (int64_t)min(base + phase + 4 * i, length - 1) * row_quads);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int token = base + phase + 4 * i;
        const float v0 = __uint_as_float(raw[i].x << 16), v1 = __uint_as_float(raw[i].x & 0xffff0000u);
        const float v2 = __uint_as_float(raw[i].y << 16), v3 = __uint_as_float(raw[i].y & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const float pj = sm.p_bf16[row0 + j][token];
          part[j][0] = fmaf(pj, v0, part[j][0]);
          part[j][1] = fmaf(pj, v1, part[j][1]);
          part[j][2] = fmaf(pj, v2, part[j][2]);
          part[j][3] = fmaf(pj, v3, part[j][3]);
        }
      }
    }
    // reduce-scatter over the four token phases (lane bits 3 and 4): bit 3 keeps channel pair
    // 2*bit3, bit 4 keeps channel bit4 of that pair; then lane L fetches channel L of the warp.
    const bool b3 = (lane >> 3) & 1, b4 = (lane >> 4) & 1;
    const int holder = (lane >> 2) + 8 * ((lane >> 1) & 1) + 16 * (lane & 1);
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const float send0 = b3 ? part[j][0] : part[j][2], send1 = b3 ? part[j][1] : part[j][3];
      const float keep0 = b3 ? part[j][2] : part[j][0], keep1 = b3 ? part[j][3] : part[j][1];
      const float pair0 = keep0 + __shfl_xor_sync(0xffffffffu, send0, 8);
      const float pair1 = keep1 + __shfl_xor_sync(0xffffffffu, send1, 8);
      const float one = (b4 ? pair1 : pair0) + __shfl_xor_sync(0xffffffffu, b4 ? pair0 : pair1, 16);
      st.o_acc[j] += __shfl_sync(0xffffffffu, one, holder) * p.bf16_value_scale;
    }
  }
  softmax_barrier(barrier);  // p_bf16 is reused by the next BF16 block
}

// Threads of a CTA: warp 0 copy producer, warp 1 MMA issuer, then SG softmax groups of four warps.
// A softmax thread owns one token of the step and R = GP / SG of the tile's GP query rows: with
// SG = 2 the two groups split the rows between them, so each thread's dependent chain per step is
// that of a tile half as wide. Only SG = 1 is instantiated: for eight query heads per KV head SG = 2
// measured 30 % slower on B200 (a CTA's step got 1.4x faster, but 320 threads per CTA leave room for
// three CTAs per SM at 64 registers or two at 96 instead of four at 80, and the CTAs per SM are what
// hides the step's latency).
__host__ __device__ constexpr int decode_threads(int sg) { return 64 + 128 * sg; }
__host__ __device__ constexpr int decode_min_ctas(int stages, int sg) {
  return sg == 1 ? (stages <= 2 ? 4 : 2) : (stages <= 3 ? 3 : 2);
}

// MXFP4 probability operand: which rows of a chunk take the lower of their two candidate exponents.
// `err[4 * row + k]` are this lane's (token's) terms of the four sums of a row: k = 0 the error under
// the upper exponent, 1 its square, 2 and 3 the same under the lower exponent. The 4 * ROWS values
// cross the warp's 32 lanes in a reduce-scatter butterfly (each step halves the values a lane holds and
// doubles the lanes they are summed over), finished by plain butterfly steps, so that lane L ends up
// with the complete sum of value (L >> SHIFT) & (4 * ROWS - 1); two more exchanges bring mass and squares
// of a candidate together (cost = mass^2 / 32 + squares, one FMA) and then the two candidates. Returns
// the warp's ballot of "the lower exponent costs less"; row `r` of the chunk reads bit
// `mx_verdict_bit<ROWS>(r)`.
template <int ROWS>
struct MxButterfly {
  static_assert(ROWS == 1 || ROWS == 2 || ROWS == 4, "rows per chunk");
  static constexpr int kValues = 4 * ROWS;
  static constexpr int kScatterSteps = ROWS == 1 ? 2 : ROWS == 2 ? 3 : 4;
  static constexpr int kShift = 5 - kScatterSteps;
};

template <int ROWS>
__device__ __forceinline__ constexpr int mx_verdict_bit(int row) {
  return (row * 4) << MxButterfly<ROWS>::kShift;
}

template <int ROWS>
__device__ __forceinline__ uint32_t mx_lower_exponent_wins(float (&err)[4 * ROWS], int lane) {
  using B = MxButterfly<ROWS>;
#pragma unroll
  for (int s = 0; s < B::kScatterSteps; ++s) {
    const int offset = 16 >> s;
    const int held = B::kValues >> (s + 1);
    const bool upper_half = (lane & offset) != 0;
#pragma unroll
    for (int i = 0; i < held; ++i) {
      const float keep = upper_half ? err[i + held] : err[i];
      const float send = upper_half ? err[i] : err[i + held];
      err[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, offset));
    }
  }
  float total = err[0];
#pragma unroll
  for (int offset = 16 >> B::kScatterSteps; offset >= 1; offset >>= 1)
    total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, offset));
  const float partner = __shfl_xor_sync(0xffffffffu, total, 1 << B::kShift);  // mass <-> squares of a candidate
  const bool holds_mass = ((lane >> B::kShift) & 1) == 0;
  const float mass = holds_mass ? total : partner, squares = holds_mass ? partner : total;
  const float cost = __fmaf_rn(mass * 0.03125f, mass, squares);
  const float other = __shfl_xor_sync(0xffffffffu, cost, 2 << B::kShift);     // upper <-> lower candidate
  const bool holds_lower = ((lane >> (B::kShift + 1)) & 1) != 0;
  return __ballot_sync(0xffffffffu, holds_lower ? cost < other : other < cost);
}

template <int GP, int TERMS, int STAGES, int PT, bool MX, int SG>
__global__ void __launch_bounds__(decode_threads(SG), decode_min_ctas(STAGES, SG))
    decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                  const DecodeParams p) {
  using Smem = DecodeSmem<GP, STAGES>;
  constexpr int KS = Smem::kStages;
  constexpr int R = GP / SG;   // query rows per softmax thread
  constexpr int LD = R;        // columns one tcgen05.ld brings (4, 8 or 16)
  constexpr int kThreads = decode_threads(SG);
  constexpr int kSoftmaxThreads = 128 * SG;
  static_assert(GP % SG == 0 && (R == 4 || R == 8 || R == 16), "rows per softmax thread");
  // one PV product covers all GP rows, so whether it starts a new sum is one decision per step:
  // softmax groups deciding separately about their own rows would need a product each
  static_assert(SG == 1, "the tensor-memory O^T sum needs one softmax group");
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which work ---------------------------------------------------------------------------
  // Part-major order: the parts that also merge the BF16 blocks (part 0) are launched first.
  const int tiles = p.rows * p.heads_kv;
  int part = blockIdx.x / tiles;
  if (p.bf16_split) part = (part + p.num_splits) % p.parts;
  const int kv_head = (blockIdx.x % tiles) % p.heads_kv;
  const int launch_row = (blockIdx.x % tiles) / p.heads_kv;
  // CTAs are handed to SMs in launch order; with a ragged batch the caller lists the rows
  // longest first, so that the longest walks start first and the short ones fill the gaps
  const int row = p.row_order ? min(max(p.row_order[launch_row], 0), p.rows - 1) : launch_row;
  const int G = p.ratio;
  // A "page" below is one 128-token step of the walk: one cache page, or with 64-token pages
  // (PT = 64) two consecutive entries of the row's page table.
  constexpr int kEntries = kPage / PT;
  constexpr bool kQkAhead = PT == 128;
  static_assert(!MX || PT == 128, "MXFP4 is built for 128-token pages");
  // scale bytes of one (page, head) of K or V: two 512-byte atoms of E4M3 (16 values per scale), or
  // one atom of E8M0 under MXFP4 (32 values per scale)
  constexpr int kScaleTile = MX ? 512 : 1024;
  const int total_pages = min(p.seqused_fp4[row] / kPage, p.max_pages / kEntries);
  int first_page = 0, last_page = total_pages;
  bool with_bf16 = p.tail_key != nullptr;
  if (p.num_splits > 1) {
    if (part < p.num_splits) {
      // Split 0 also merges the tail and the sink when they have no split of their own; it is
      // then charged `bf16_page_cost` pages for them, so that every split ends at the same time
      // (cost 0 is the even partition of src/nvfp4_decode_kernel/fp4_decode_kernel.py:4686-4746).
      // A row may be cut into fewer parts than the launch has (`row_splits`): its further parts
      // find no pages.
      const int row_parts = p.row_splits ? min(max(p.row_splits[row], 1), p.num_splits) : p.num_splits;
      const int bias = (with_bf16 && !p.bf16_split) ? p.bf16_page_cost : 0;
      const int chunk = (total_pages + bias + row_parts - 1) / row_parts;
      const int first_chunk = max(chunk - bias, 0);
      first_page = part == 0 ? 0 : min(first_chunk + (part - 1) * chunk, total_pages);
      last_page = part < row_parts ? min(first_page + (part == 0 ? first_chunk : chunk), total_pages) : first_page;
      with_bf16 = with_bf16 && !p.bf16_split && part == 0;
    } else {
      first_page = last_page = 0;
    }
  }
  const int num_pages = last_page - first_page;
  if (p.row_splits && p.num_splits > 1 && num_pages == 0 && !with_bf16) {
    // A part with nothing to walk (rows cut into fewer parts than the launch has): it owes the merge
    // an LSE of -inf for each of its heads and nothing else, so it leaves before any set-up. The
    // buffers it writes are free: the launch before this one waited for its own predecessors (among
    // them the previous merge) before it let this launch start.
    if (tid < p.ratio)
      p.partial_lse[((int64_t)part * p.rows + row) * p.heads_q + kv_head * p.ratio + tid] = -INFINITY;
    return;
  }
  int slot = -1, tail_len = 0, sink_len = 0;
  if (p.tail_key) {
    slot = p.tail_slot_ids[row];
    if (slot >= 0 && slot < p.tail_slots) {
      tail_len = min(max(p.seqused_residual[row], 0), kPage);
      if (p.seqused_sink) sink_len = min(max(p.seqused_sink[row], 0), BDFP4_MAX_SINK);
    } else {
      slot = 0;
    }
  }

  // ---- set-up -------------------------------------------------------------------------------
  // The BF16 tail is read with plain loads whose latency is the block's whole cost: start its
  // lines toward L2 now (two 128-byte lines per token for K and for V).
  if (with_bf16) {
    const int64_t row_bytes = (int64_t)p.heads_kv * kHeadDim * 2;
    const int64_t head_offset = ((int64_t)slot * p.tail_slot_stride + kv_head * kHeadDim) * 2;
    for (int i = tid; i < tail_len * 4; i += kThreads) {
      const char* base = reinterpret_cast<const char*>((i & 2) ? p.tail_value : p.tail_key) + head_offset;
      prefetch_l2(base + (int64_t)(i >> 2) * row_bytes + (i & 1) * 128);
    }
  }
  if (tid == 0) {
    for (int s = 0; s < KS; ++s) {
      tc::mbar_init(&sm.k_full[s], 1);
      tc::mbar_init(&sm.k_empty[s], 1);
      tc::mbar_init(&sm.v_full[s], 1);
      tc::mbar_init(&sm.v_empty[s], 1);
      tc::mbar_init(&sm.ksf_full[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(&sm.s_full[s], 1);
      tc::mbar_init(&sm.s_empty[s], kSoftmaxThreads);
      tc::mbar_init(&sm.p_full[s], kSoftmaxThreads);
      tc::mbar_init(&sm.p_empty[s], 1);
      tc::mbar_init(&sm.o_full[s], 1);
    }
    sm.abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tensormap(&k_map);
    tc::prefetch_tensormap(&v_map);
  }
  // zero the Q tiles, P tiles, both scale-atom buffers (contiguous 1 KB blocks) and the BF16 query
  {
    uint4* blocks[4] = {reinterpret_cast<uint4*>(sm.q_tile), reinterpret_cast<uint4*>(sm.p_tile),
                        reinterpret_cast<uint4*>(sm.q_sf), reinterpret_cast<uint4*>(sm.p_sf)};
    for (int i = tid; i < 4 * 128; i += kThreads) blocks[i >> 7][i & 127] = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < GP * 32; i += kThreads) reinterpret_cast<uint4*>(sm.q_bf16)[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  // The first ring stages are requested before the rest of the set-up, which then overlaps the
  // page-table read and the first copies.
  auto request_key = [&](int i, int page, int page_b) {  // one thread
    const int s = i % KS;
    if constexpr (PT == 128) {
      tc::mbar_expect_tx(&sm.k_full[s], 8192 + kScaleTile);
      tc::tma_load_4d(sm.k_stage[s], &k_map, &sm.k_full[s], 0, kv_head, 0, page);
      tc::bulk_load(sm.k_stage[s] + 8192, p.k_scales + (int64_t)page * p.k_scales_pitch + kv_head * kScaleTile,
                    kScaleTile, &sm.k_full[s]);
    } else {
      tc::mbar_expect_tx(&sm.ksf_full[s], 1024);
      tc::mbar_expect_tx(&sm.k_full[s], 8192);
      // tokens 0-63 of the step come from the first entry, 64-127 from the second, each stored as
      // its 4 KB swizzled shared-memory image. The two 512-byte scale blocks land side by side on
      // a barrier of their own: the MMA warp interleaves them into atoms while the codes are
      // still in flight.
      tc::bulk_load(sm.k_stage[s] + 8192, p.k_scales + (int64_t)page * p.k_scales_pitch + kv_head * 512, 512,
                    &sm.ksf_full[s]);
      tc::bulk_load(sm.k_stage[s] + 8192 + 512, p.k_scales + (int64_t)page_b * p.k_scales_pitch + kv_head * 512, 512,
                    &sm.ksf_full[s]);
      tc::bulk_load(sm.k_stage[s], p.k_codes + (int64_t)page * p.k_codes_pitch + kv_head * 4096, 4096, &sm.k_full[s]);
      tc::bulk_load(sm.k_stage[s] + 4096, p.k_codes + (int64_t)page_b * p.k_codes_pitch + kv_head * 4096, 4096,
                    &sm.k_full[s]);
    }
  };
  auto request_value = [&](int i, int page, int page_b) {
    const int s = i % KS;
    tc::mbar_expect_tx(&sm.v_full[s], 8192 + kScaleTile);
    if constexpr (PT == 128) {
      tc::tma_load_3d(sm.v_stage[s], &v_map, &sm.v_full[s], 0, kv_head * kHeadDim, page);
      tc::bulk_load(sm.v_stage[s] + 8192, p.v_scales + (int64_t)page * p.v_scales_pitch + kv_head * kScaleTile,
                    kScaleTile, &sm.v_full[s]);
    } else {
      // one [128 ch][32 B] tile and one scale atom per entry: the two K = 64 steps of the PV MMA
      tc::bulk_load(sm.v_stage[s], p.v_codes + (int64_t)page * p.v_codes_pitch + kv_head * 4096, 4096, &sm.v_full[s]);
      tc::bulk_load(sm.v_stage[s] + 4096, p.v_codes + (int64_t)page_b * p.v_codes_pitch + kv_head * 4096, 4096,
                    &sm.v_full[s]);
      tc::bulk_load(sm.v_stage[s] + 8192, p.v_scales + (int64_t)page * p.v_scales_pitch + kv_head * 512, 512,
                    &sm.v_full[s]);
      tc::bulk_load(sm.v_stage[s] + 8192 + 512, p.v_scales + (int64_t)page_b * p.v_scales_pitch + kv_head * 512, 512,
                    &sm.v_full[s]);
    }
  };
  auto page_of = [&](int i, int entry) {  // physical page of the i-th step this CTA walks (newest first)
    int page = p.page_table[(int64_t)row * p.page_table_stride + (last_page - 1 - i) * kEntries + entry];
    if (page < 0 || page >= p.pages) {
      if (p.error_word) atomicOr(p.error_word, (int)BDFP4_DEV_BAD_PAGE);
      page = min(max(page, 0), p.pages - 1);
    }
    return page;
  };
  const int early = min(KS, num_pages);
  if (warp == 0) {
    const int my_page = lane < early ? page_of(lane, 0) : 0;
    const int my_page_b = (PT == 64 && lane < early) ? page_of(lane, 1) : 0;
    for (int j = 0; j < early; ++j) {
      const int page = __shfl_sync(0xffffffffu, my_page, j);
      const int page_b = __shfl_sync(0xffffffffu, my_page_b, j);
      if (lane == 0) {
        request_key(j, page, page_b);
        request_value(j, page, page_b);
      }
    }
  }
  // Everything up to here reads only the cache and the batch's metadata. The query operands and
  // the BF16 tail come from the launch before this one (the query quantizer): with programmatic
  // dependent launch this kernel may have started while that one was still running, so wait for
  // it here, then let the launch after this one start its own preamble.
  wait_for_prior_kernels();
  dependents_may_launch();
  // Warps 1-5 fetch the query operands: one 16-byte chunk of query codes, one word of query
  // scales and up to two 16-byte chunks of the BF16 query per thread.
  const int qt = tid < 192 ? tid - 32 : -1;  // the 160 threads behind warp 0
  const bool loads_codes = qt >= 0 && qt < TERMS * G * 4;
  // NVFP4: two words per query head and term (one per atom); MXFP4: one (a single atom)
  const bool loads_scales = qt >= 0 && qt < TERMS * G * (MX ? 1 : 2);
  uint4 code_chunk = make_uint4(0, 0, 0, 0);
  uint32_t scale_word = 0;
  uint4 bf16_chunk[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  if (loads_codes) {
    const int g = (qt >> 2) % G, term = (qt >> 2) / G;
    code_chunk = __ldg(reinterpret_cast<const uint4*>(p.q_codes[term] +
                                                      ((int64_t)row * p.heads_q + kv_head * G + g) * 64) + (qt & 3));
  }
  if (loads_scales) {
    if constexpr (MX) {
      const int g = qt % G, term = qt / G;
      scale_word = __ldg(reinterpret_cast<const uint32_t*>(
          p.q_scales[term] + ((int64_t)row * p.heads_q + kv_head) * 512 + g * 16));
    } else {
      const int g = (qt >> 1) % G, term = (qt >> 1) / G;
      scale_word = __ldg(reinterpret_cast<const uint32_t*>(
          p.q_scales[term] + ((int64_t)row * p.heads_q + kv_head) * 1024 + (qt & 1) * 512 + g * 16));
    }
  }
  if (with_bf16 && qt >= 0) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = qt + 160 * k;  // 16-byte chunk: head i / 16, channels 8 * (i % 16) ...
      if (i < G * 16)
        bf16_chunk[k] = __ldg(reinterpret_cast<const uint4*>(
            p.q_padded + (((int64_t)row * kPage) * p.heads_q + kv_head * G + (i >> 4)) * kHeadDim + (i & 15) * 8));
    }
  }
  if (loads_codes) {
    const int g = (qt >> 2) % G, term = (qt >> 2) / G;
    *reinterpret_cast<uint4*>(sm.q_tile[term] + swizzle64(g * 64 + (qt & 3) * 16)) = code_chunk;
  }
  if (loads_scales) {
    if constexpr (MX) {
      *reinterpret_cast<uint32_t*>(sm.q_sf[qt / G] + (qt % G) * 16) = scale_word;
    } else {
      const int g = (qt >> 1) % G, term = (qt >> 1) / G;
      *reinterpret_cast<uint32_t*>(sm.q_sf[term] + (qt & 1) * 512 + g * 16) = scale_word;
    }
  }
  if (with_bf16 && qt >= 0) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = qt + 160 * k;
      if (i < G * 16) {
        const uint32_t w[4] = {bf16_chunk[k].x, bf16_chunk[k].y, bf16_chunk[k].z, bf16_chunk[k].w};
        float* dst = &sm.q_bf16[i >> 4][(i & 15) * 8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          dst[2 * e] = __uint_as_float(w[e] << 16);
          dst[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
      }
    }
  }
  if (warp == 1) {
    tc::tmem_alloc(&sm.tmem_base, kTmemColumns);
    tc::tmem_relinquish();
  }
  tc::fence_proxy_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 0) {
    // ---- copy producer ----------------------------------------------------------------------
    // Lane 0 requests the K stages and lane 1 the V stages, each behind its own ring's empty
    // barriers, so a V stage that is still being read never holds back the next K request. The
    // page ids of up to 32 steps are fetched by the whole warp and parked in shared memory.
    int issued = early;
    bool ok = true;
    for (int base = early; base < num_pages && ok; base += 32) {
      const int count = min(32, num_pages - base);
      if (lane < count) {
        sm.page_ids[0][lane] = page_of(base + lane, 0);
        if constexpr (PT == 64) sm.page_ids[1][lane] = page_of(base + lane, 1);
      }
      __syncwarp();
      if (lane < 2) {
        for (int j = 0; j < count && ok; ++j) {
          const int i = base + j;
          const int s = i % KS;
          const uint32_t parity = ((i / KS) & 1) ^ 1;
          const int page = sm.page_ids[0][j];
          const int page_b = PT == 64 ? sm.page_ids[1][j] : 0;
          if (lane == 0) {
            ok = tc::mbar_wait(&sm.k_empty[s], parity, abort_flag);
            if (ok) request_key(i, page, page_b);
          } else {
            ok = tc::mbar_wait(&sm.v_empty[s], parity, abort_flag);
            if (ok) request_value(i, page, page_b);
          }
          if (ok) issued = i + 1;
        }
      }
      ok = __all_sync(0xffffffffu, ok);  // both lanes are done with this batch's page ids
    }
    // After a give-up, wait (bounded) until every copy already in flight has landed, so that no
    // bulk copy can write into this CTA's shared memory after it exits.
    if (lane < 2 && *abort_flag) {
      const uint64_t start = tc::global_timer_ns();
      for (int i = max(0, issued - KS); i < issued; ++i) {
        const int s = i % KS;
        const uint32_t parity = (i / KS) & 1;
        if (lane == 0) {
          while (!tc::mbar_try_wait(&sm.k_full[s], parity) && tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
          while (PT == 64 && !tc::mbar_try_wait(&sm.ksf_full[s], parity) &&
                 tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
        } else {
          while (!tc::mbar_try_wait(&sm.v_full[s], parity) && tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    // One thread issues every tcgen05 operation. With 64-token pages the whole warp stays in the
    // loop: its 32 lanes interleave the two pages' K scale blocks into MMA atoms.
    const bool issuer = lane == 0;
    if (num_pages > 0 && (issuer || PT == 64)) {
      constexpr uint32_t idesc_qk = MX ? tc::mxf4_idesc(128, kNQ) : tc::nvf4_idesc(128, kNQ);
      constexpr uint32_t idesc_pv = MX ? tc::mxf4_idesc(128, kNP) : tc::nvf4_idesc(128, kNP);
      const uint32_t q_addr = tc::smem_u32(sm.q_tile);
      // One block-scaled MMA over a 64-value slice `k` of the contraction. NVFP4: the slice's four
      // scales per row are the 4-column atom `k` of each operand. MXFP4: both slices' two scales per
      // row share one atom and the instruction picks its byte pair through the scale-factor ids.
      auto block_mma = [&](uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                           int k, bool accumulate) {
        if constexpr (MX)
          tc::mma_mxf4(d, a_desc, b_desc, idesc | tc::mxf4_sf_ids(2 * k, 2 * k), sfa, sfb, accumulate);
        else
          tc::mma_nvf4(d, a_desc, b_desc, idesc, sfa + 4 * k, sfb + 4 * k, accumulate);
      };
      if (issuer) {
#pragma unroll
        for (int term = 0; term < TERMS; ++term) {
          tc::cp_sf_atom(tmem + kColSFQ + 8 * term, tc::sf_atom_desc(tc::smem_u32(sm.q_sf[term])));
          if constexpr (!MX)
            tc::cp_sf_atom(tmem + kColSFQ + 8 * term + 4, tc::sf_atom_desc(tc::smem_u32(sm.q_sf[term]) + 512));
        }
      }
      auto issue_pv = [&](int m) -> bool {  // issuer only
        const int s = m % KS;
        const int b = m & 1;
        const uint32_t ring_parity = (m / KS) & 1;
        const uint32_t pair_parity = (m >> 1) & 1;
        if (!tc::mbar_wait(&sm.v_full[s], ring_parity, abort_flag)) return false;
        if (!tc::mbar_wait(&sm.p_full[b], pair_parity, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t v_addr = tc::smem_u32(sm.v_stage[s]);
        const uint32_t p_addr = tc::smem_u32(sm.p_tile[b]);
        tc::cp_sf_atom(tmem + kColSFV + 8 * b, tc::sf_atom_desc(v_addr + 8192));
        tc::cp_sf_atom(tmem + kColSFP + 8 * b, tc::sf_atom_desc(tc::smem_u32(sm.p_sf[b])));
        if constexpr (!MX) {
          tc::cp_sf_atom(tmem + kColSFV + 8 * b + 4, tc::sf_atom_desc(v_addr + 8192 + 512));
          tc::cp_sf_atom(tmem + kColSFP + 8 * b + 4, tc::sf_atom_desc(tc::smem_u32(sm.p_sf[b]) + 512));
        }
        // O^T keeps adding up in tensor memory over the steps that share their running maxima; the
        // softmax threads say (before they release the P buffer) when a step starts a new sum,
        // having read the old one back first
        const bool fresh = *reinterpret_cast<volatile int*>(&sm.pv_fresh[b]) != 0;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          // 128-token page: one tile of 64-byte rows, K step k at +32 bytes. 64-token pages: one
          // tile of 32-byte rows per page.
          const uint64_t v_desc = PT == 128 ? tc::fp4_tile_desc(v_addr, k) : tc::fp4_half_tile_desc(v_addr + k * 4096);
          block_mma(tmem + kColO, v_desc, tc::fp4_tile_desc(p_addr, k), idesc_pv, tmem + kColSFV + 8 * b,
                    tmem + kColSFP + 8 * b, k, k != 0 || !fresh);
        }
        tc::commit(&sm.o_full[b]);
        tc::commit(&sm.v_empty[s]);
        tc::commit(&sm.p_empty[b]);
        return true;
      };
      bool ok = true;
      for (int i = 0; i < num_pages && ok; ++i) {
        const int s = i % KS;
        const int b = i & 1;
        if constexpr (PT == 64) {
          ok = tc::mbar_wait(&sm.ksf_full[s], (i / KS) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          // K scales arrived as [page][atom][32 rows][8 B]; an atom row is 16 bytes, tokens 0-63
          // (first page) in its low half and 64-127 in its high half. Every lane reads its four
          // 8-byte pieces before any lane writes, so the exchange is done in place.
          uint8_t* sf = sm.k_stage[s] + 8192;
          const uint2 a0 = *reinterpret_cast<const uint2*>(sf + lane * 8);
          const uint2 a1 = *reinterpret_cast<const uint2*>(sf + 256 + lane * 8);
          const uint2 b0 = *reinterpret_cast<const uint2*>(sf + 512 + lane * 8);
          const uint2 b1 = *reinterpret_cast<const uint2*>(sf + 768 + lane * 8);
          __syncwarp();
          *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(a0.x, a0.y, b0.x, b0.y);
          *reinterpret_cast<uint4*>(sf + 512 + lane * 16) = make_uint4(a1.x, a1.y, b1.x, b1.y);
          tc::fence_proxy_async_smem();
          __syncwarp();
        } else {
          ok = tc::mbar_wait(&sm.k_full[s], (i / KS) & 1, abort_flag);
          if (!ok) break;
        }
        if (issuer && PT == 64) ok = tc::mbar_wait(&sm.k_full[s], (i / KS) & 1, abort_flag);
        if (issuer && ok) {
          tc::fence_after_sync();
          const uint32_t k_addr = tc::smem_u32(sm.k_stage[s]);
          tc::cp_sf_atom(tmem + kColSFK + 8 * b, tc::sf_atom_desc(k_addr + 8192));
          if constexpr (!MX) tc::cp_sf_atom(tmem + kColSFK + 8 * b + 4, tc::sf_atom_desc(k_addr + 8192 + 512));
          ok = tc::mbar_wait(&sm.s_empty[b], ((i >> 1) & 1) ^ 1, abort_flag);
          if (ok) {
            tc::fence_after_sync();
            // both query terms accumulate into the same S^T columns: K.Q0 + K.Q1 in FP32
#pragma unroll
            for (int term = 0; term < TERMS; ++term) {
#pragma unroll
              for (int k = 0; k < 2; ++k)
                block_mma(tmem + kColS + kNQ * b, tc::fp4_tile_desc(k_addr, k),
                          tc::fp4_tile_desc(q_addr + term * (kNQ * 64), k), idesc_qk, tmem + kColSFK + 8 * b,
                          tmem + kColSFQ + 8 * term, k, (term | k) != 0);
            }
            tc::commit(&sm.s_full[b]);
            tc::commit(&sm.k_empty[s]);
            // With 128-token pages QK runs two steps ahead of PV (S^T has two buffers): a K stage
            // goes back to its producer lane without waiting for the previous step's
            // probabilities (measured 0.9 % faster; with 64-token pages it measured 1 % slower,
            // so there PV follows one step behind).
            if constexpr (kQkAhead) {
              if (i > 1) ok = issue_pv(i - 2);
            } else {
              if (i > 0) ok = issue_pv(i - 1);
            }
          }
        }
        if constexpr (PT == 64) ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      }
      if (issuer && ok && num_pages > 1 && kQkAhead) ok = issue_pv(num_pages - 2);
      if (issuer && ok) issue_pv(num_pages - 1);
    }
  } else {
    // ---- softmax / accumulate -----------------------------------------------------------------
    const int warp_q = warp & 3;        // TMEM lane quarter this warp may read
    const int t = warp_q * 32 + lane;   // token (S^T lane) and channel (O^T lane) of this thread
    const int sgroup = (warp - 2) >> 2;  // softmax group of this warp
    const int row0 = sgroup * R;         // first of the tile's rows this group owns
    const int barrier = 1 + sgroup;      // the group's named barrier
    const uint32_t lane_base = tmem + ((uint32_t)(warp_q * 32) << 16) + row0;
    const float shift = p.p_mode == BDFP4_P_AMAX2_OR_AMAX6_C8 ? 3.0f : 0.0f;
    SoftmaxState<R> st;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      st.row_max[j] = -INFINITY;
      st.row_sum[j] = 0.0f;
      st.o_acc[j] = 0.0f;
    }
    st.first = true;
    int red_buf = 0;
    const __nv_bfloat16* tail_k = p.tail_key ? p.tail_key + (int64_t)slot * p.tail_slot_stride + kv_head * kHeadDim : nullptr;
    const __nv_bfloat16* tail_v = p.tail_value ? p.tail_value + (int64_t)slot * p.tail_slot_stride + kv_head * kHeadDim : nullptr;
    const int64_t row_elems = (int64_t)p.heads_kv * kHeadDim;

    if (with_bf16) {
      // While page zero has not been sealed the rolling page still holds the sink's tokens.
      const int mask_below = total_pages == 0 ? sink_len : 0;
      bf16_block<R>(st, sm, p, t, warp_q, lane, tail_k, tail_v, mask_below, tail_len, shift, red_buf, row0, barrier);
    }

    // O^T of the FP4 pages adds up in tensor memory, one PV product per step on top of the last. It is
    // read back only when a running maximum moves (rare under the stale-maximum rule): the sum so far
    // then joins `o_acc`, everything is rescaled, and the next product starts a new sum.
    int sum_begin = 0;  // first step of the sum tensor memory currently holds
    // Which row's group maximum this lane ends up holding after the reduce-scatter below: step i
    // hands the upper half of the rows still held to the lanes whose bit i is set.
    constexpr int LOG = R == 4 ? 2 : (R == 8 ? 3 : 4);
    int own_row = 0;
#pragma unroll
    for (int i = 0; i < LOG; ++i) own_row += ((lane >> i) & 1) * (R >> (i + 1));
    const float headroom = kRescaleThreshold / p.scale_log2;  // score growth the stale maximum tolerates
    float threshold[R];   // a score above this forces the running maximum to move
    float max_scaled[R];  // running maximum in log2 units with the c8 shift folded in
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const float safe = st.row_max[j] == -INFINITY ? 0.0f : st.row_max[j];
      max_scaled[j] = safe * p.scale_log2 - shift;
      threshold[j] = 0.0f;
    }
    float own_max_scaled = 0.0f;
    // With eight or more rows per thread the three per-row arrays (24+ registers of values every
    // thread holds identically) are parked in shared memory for the page loop and read back as
    // broadcasts; they change only when a running maximum moves.
    constexpr bool kStatsInSmem = R >= 8 || SG > 1;
    auto refresh_thresholds = [&]() {
      own_max_scaled = max_scaled[0];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        threshold[j] = st.row_max[j] + headroom;
        own_max_scaled = own_row == j ? max_scaled[j] : own_max_scaled;
      }
      if constexpr (kStatsInSmem) {
        // every thread writes the same values; the barrier orders them before the next reads
#pragma unroll
        for (int j = 0; j < R; ++j) {
          sm.stat_row_max[row0 + j] = st.row_max[j];
          sm.stat_threshold[row0 + j] = threshold[j];
          sm.stat_max_scaled[row0 + j] = max_scaled[j];
        }
        softmax_barrier(barrier);
      }
    };
    refresh_thresholds();
    // constant parts of this thread's shared-memory addresses
    const int group = t >> 4;
    const int sf_offset = (group >> 2) * 512 + (row0 + own_row) * 16 + (group & 3);
    const bool stores_sf = (lane & 15) < R;
    // after the nibble transpose a lane of an 8-lane cluster holds one row's codes for 4 (R = 4)
    // or 8 (R = 8) consecutive tokens
    const int pack_row = R == 4 ? (((lane & 1) << 1) | ((lane >> 1) & 1))
                                 : (((lane & 1) << 2) | (lane & 2) | ((lane >> 2) & 1));
    const int pack_offset = R == 4 ? swizzle64((row0 + pack_row) * 64 + (t >> 2) * 2)
                                   : swizzle64((row0 + pack_row) * 64 + (t >> 3) * 4);

    // The sink is read last; its lines are sent toward L2 a few pages before the loop ends.
    auto prefetch_sink = [&]() {
      if (with_bf16 && p.seqused_sink && t < sink_len * 4) {
        const __nv_bfloat16* base = ((t & 2) ? tail_v : tail_k) + (int64_t)(kPage + (t >> 2)) * row_elems;
        prefetch_l2(reinterpret_cast<const char*>(base) + (t & 1) * 128);
      }
    };
    if (num_pages < 3) prefetch_sink();

    bool stop = false;
    for (int i = 0; i < num_pages && !stop; ++i) {
      const int b = i & 1;
      const uint32_t parity = (i >> 1) & 1;
      const int logical_page = last_page - 1 - i;
      if (i == num_pages - 3) prefetch_sink();
      tc::mbar_wait(&sm.s_full[b], parity, abort_flag);
      tc::fence_after_sync();
      float s[R];
      tc::tmem_ld<LD>(lane_base + kColS + kNQ * b, s);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      tc::mbar_arrive(&sm.s_empty[b]);
      if (logical_page == 0 && t < sink_len) {
#pragma unroll
        for (int j = 0; j < R; ++j) s[j] = -INFINITY;
      }
      // does any row's maximum have to move? one predicate per thread, one barrier-wide OR
      bool grows = true;
      if (!st.first) {
        bool own = *abort_flag != 0;
#pragma unroll
        for (int j = 0; j < R; ++j) own = own || s[j] > (kStatsInSmem ? sm.stat_threshold[row0 + j] : threshold[j]);
        grows = softmax_vote_any(own, barrier);
      }
      float acc[R];
      // How a row's scale group is reduced. NVFP4 with up to eight rows: a reduce-scatter leaves each
      // lane with ONE row's 16-token group maximum. NVFP4 with sixteen rows: every lane keeps every
      // row's group maximum. MXFP4: the group is the warp's 32 tokens and is reduced where the
      // probabilities are quantized.
      constexpr bool kScatter = !MX && R <= 8;
      constexpr bool kPerRow = !MX && R > 8;
      float own_group_max;  // maximum of row `own_row` over this lane's 16-token scale group
      if constexpr (kScatter) {
        // reduce-scatter: R - 1 shuffles leave each lane with one row's maximum over R lanes,
        // the remaining butterfly steps finish that row's 16-lane group
        float held[R];
#pragma unroll
        for (int j = 0; j < R; ++j) held[j] = s[j];
#pragma unroll
        for (int step = 0; step < LOG; ++step) {
          const int half = R >> (step + 1);
          const bool upper = (lane >> step) & 1;
#pragma unroll
          for (int k = 0; k < half; ++k) {
            const float send = upper ? held[k] : held[k + half];
            const float keep = upper ? held[k + half] : held[k];
            held[k] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 1 << step));
          }
        }
        own_group_max = held[0];
#pragma unroll
        for (int step = LOG; step < 4; ++step)
          own_group_max = fmaxf(own_group_max, __shfl_xor_sync(0xffffffffu, own_group_max, 1 << step));
      } else {
        own_group_max = 0.0f;  // R = 16 keeps every row's group maximum (below)
      }
      float group_max[R];
      if constexpr (kPerRow) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
          float m = s[j];
#pragma unroll
          for (int step = 1; step < 16; step <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, step));
          group_max[j] = m;
        }
      }
      if (grows) {
        float block_max[R];
        if constexpr (kScatter) {
          const float warp_max = fmaxf(own_group_max, __shfl_xor_sync(0xffffffffu, own_group_max, 16));
          if (lane < R) sm.red[red_buf][warp_q][row0 + own_row] = warp_max;
        } else {
#pragma unroll
          for (int j = 0; j < R; ++j) {
            if constexpr (kPerRow) {
              block_max[j] = fmaxf(group_max[j], __shfl_xor_sync(0xffffffffu, group_max[j], 16));
            } else {
              float m = s[j];
#pragma unroll
              for (int step = 1; step < 32; step <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, step));
              block_max[j] = m;
            }
          }
          if (lane < R) {
            float mine = block_max[0];
#pragma unroll
            for (int j = 1; j < R; ++j) mine = lane == j ? block_max[j] : mine;
            sm.red[red_buf][warp_q][row0 + lane] = mine;
          }
        }
        softmax_barrier(barrier);
#pragma unroll
        for (int j = 0; j < R; ++j)
          block_max[j] = fmaxf(fmaxf(sm.red[red_buf][0][row0 + j], sm.red[red_buf][1][row0 + j]),
                               fmaxf(sm.red[red_buf][2][row0 + j], sm.red[red_buf][3][row0 + j]));
        red_buf ^= 1;
        if constexpr (kStatsInSmem) {
#pragma unroll
          for (int j = 0; j < R; ++j) st.row_max[j] = sm.stat_row_max[row0 + j];
        }
        update_max<R>(st, block_max, p.scale_log2, shift, acc, max_scaled);
        refresh_thresholds();
        stop = *abort_flag != 0;  // uniform: every thread reads it after the same barrier
        if (i > sum_begin) {
          // the products of steps [sum_begin, i) are issued; the last of them reports on o_full
          const int pb = (i - 1) & 1;
          tc::mbar_wait(&sm.o_full[pb], ((i - 1) >> 1) & 1, abort_flag);
          tc::fence_after_sync();
          float o[LD];
          tc::tmem_ld<LD>(lane_base + kColO, o);
          tc::tmem_wait_ld();
          tc::fence_before_sync();
#pragma unroll
          for (int j = 0; j < R; ++j) st.o_acc[j] += o[j];
        }
        sum_begin = i;
#pragma unroll
        for (int j = 0; j < R; ++j) {
          st.o_acc[j] *= acc[j];
          st.row_sum[j] *= acc[j];
        }
      }
      st.first = false;
      float prob[R];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        prob[j] = ex2_approx(fmaf(s[j], p.scale_log2, -(kStatsInSmem ? sm.stat_max_scaled[row0 + j] : max_scaled[j])));
        st.row_sum[j] += prob[j];
      }
      // ---- probabilities -> E2M1 codes on a per-group scale ---------------------------------------
      // First the scaling: prob[j] becomes p / scale of its group, and the group's scale byte is
      // known to the lane that will store it.
      float own_scale = 0.0f;       // kScatter: scale of row `own_row` over this lane's 16-token group
      float group_scale[R];        // kPerRow: every row's group scale
      int mx_exponent[R];          // MX: every row's E8M0 exponent for this warp's 32 tokens
      if constexpr (MX) {
        // The MXFP4 probability operand (src/nvfp4_decode_kernel/reference.py:331-355,
        // fp4_decode_kernel.py:5687-5731): start from the smallest exponent that keeps the group's
        // maximum at or below six; take the exponent below it when that lowers
        // (sum of errors)^2 / 32 + (sum of squared errors), both sums formed by the warp's butterfly
        // and combined by one FMA.
        // Rows are taken four at a time: their 16 error sums (mass and squares under each of the two
        // exponents) cross the warp in ONE reduce-scatter butterfly of 18 shuffles instead of twenty
        // per row.
        constexpr int kChunk = R < 4 ? R : 4;
#pragma unroll
        for (int base = 0; base < R; base += kChunk) {
          float err[4 * kChunk], scaled_upper[kChunk], scaled_lower[kChunk];
          int upper[kChunk];
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const float value = prob[base + j];
            const float maximum = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(value)));
            upper[j] = mx_round_up_exponent(maximum);
            const int lower = max(upper[j] - 1, -127);
            scaled_upper[j] = value * mx_power_of_two(-upper[j]);
            scaled_lower[j] = value * mx_power_of_two(-lower);
            const float read_upper = e2m1x2_to_float2(cvt_e2m1x2(scaled_upper[j], 0.0f)).x * mx_power_of_two(upper[j]);
            const float read_lower = e2m1x2_to_float2(cvt_e2m1x2(scaled_lower[j], 0.0f)).x * mx_power_of_two(lower);
            const float mass_upper = __fsub_rn(read_upper, value), mass_lower = __fsub_rn(read_lower, value);
            err[4 * j + 0] = mass_upper;
            err[4 * j + 1] = __fmul_rn(mass_upper, mass_upper);
            err[4 * j + 2] = mass_lower;
            err[4 * j + 3] = __fmul_rn(mass_lower, mass_lower);
          }
          const uint32_t verdict = mx_lower_exponent_wins<kChunk>(err, lane);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const bool take_lower = (verdict >> mx_verdict_bit<kChunk>(j)) & 1u;
            mx_exponent[base + j] = take_lower ? max(upper[j] - 1, -127) : upper[j];
            prob[base + j] = take_lower ? scaled_lower[j] : scaled_upper[j];
          }
        }
      } else if constexpr (kScatter) {
        // the lane holding a row's group maximum turns it into the group's scale once; the
        // group's lanes fetch the reciprocal from it
        const float maximum = ex2_approx(fmaf(own_group_max, p.scale_log2, -own_max_scaled));
        own_scale = probability_scale(maximum, p.p_mode, p.tau);
        const float own_inverse = rcp_approx(fmaxf(own_scale, 1e-20f));
        const int cluster = lane & ~(R - 1);
#pragma unroll
        for (int j = 0; j < R; ++j) {
          int source = 0;  // the lane pattern whose own_row is j (bit reversal of j)
#pragma unroll
          for (int bit = 0; bit < LOG; ++bit) source |= ((j >> (LOG - 1 - bit)) & 1) << bit;
          prob[j] *= __shfl_sync(0xffffffffu, own_inverse, cluster | source);
        }
      } else {
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const float maximum =
              ex2_approx(fmaf(group_max[j], p.scale_log2, -(kStatsInSmem ? sm.stat_max_scaled[row0 + j] : max_scaled[j])));
          group_scale[j] = probability_scale(maximum, p.p_mode, p.tau);
          prob[j] *= rcp_approx(fmaxf(group_scale[j], 1e-20f));
        }
      }
      // Then the codes into the PV MMA's B operand (rows = query heads, 64 bytes of tokens each).
      if constexpr (R <= 8) {
        // E2M1 codes of this token: one byte per pair of rows, then a nibble transpose across the
        // lanes of an 8-token cluster so that each lane stores one row's run of tokens
        uint32_t codes = 0;
#pragma unroll
        for (int j = 0; j < R; j += 2) codes |= cvt_e2m1x2(prob[j], prob[j + 1]) << (4 * j);
        {
          const uint32_t other = __shfl_xor_sync(0xffffffffu, codes, 1);
          const bool odd = lane & 1;
          const uint32_t even_token = (odd ? other : codes) >> (odd ? 2 * R : 0);  // rows this lane keeps
          const uint32_t odd_token = (odd ? codes : other) >> (odd ? 2 * R : 0);
          if constexpr (R == 4) {
            codes = (even_token & 0xfu) | ((odd_token & 0xfu) << 4) | ((even_token & 0xf0u) << 4) |
                    ((odd_token & 0xf0u) << 8);
          } else {
            codes = (even_token & 0xfu) | ((odd_token & 0xfu) << 4) | ((even_token & 0xf0u) << 4) |
                    ((odd_token & 0xf0u) << 8) | ((even_token & 0xf00u) << 8) | ((odd_token & 0xf00u) << 12) |
                    ((even_token & 0xf000u) << 12) | ((odd_token & 0xf000u) << 16);
          }
        }
        {
          const uint32_t other = __shfl_xor_sync(0xffffffffu, codes, 2);
          const bool upper = lane & 2;
          if constexpr (R == 4) {
            codes = __byte_perm(codes, other, upper ? 0x0015 : 0x0040);
          } else {
            codes = __byte_perm(codes, other, upper ? 0x3726 : 0x5140);
          }
        }
        if constexpr (R == 8) {
          const uint32_t other = __shfl_xor_sync(0xffffffffu, codes, 4);
          codes = __byte_perm(codes, other, (lane & 4) ? 0x3276 : 0x5410);
        }
        // the PV MMA of two pages ago must be done with this P buffer
        tc::mbar_wait(&sm.p_empty[b], parity ^ 1, abort_flag);
        if constexpr (R == 4) {
          *reinterpret_cast<uint16_t*>(sm.p_tile[b] + pack_offset) = (uint16_t)codes;
        } else {
          *reinterpret_cast<uint32_t*>(sm.p_tile[b] + pack_offset) = codes;
        }
      } else {
        uint32_t words[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
          uint32_t word = (cvt_e2m1x2(prob[j], 0.0f) & 0xfu) << (4 * (lane & 7));
          word |= __shfl_xor_sync(0xffffffffu, word, 1);
          word |= __shfl_xor_sync(0xffffffffu, word, 2);
          word |= __shfl_xor_sync(0xffffffffu, word, 4);
          words[j] = word;
        }
        tc::mbar_wait(&sm.p_empty[b], parity ^ 1, abort_flag);
#pragma unroll
        for (int j = 0; j < R; ++j) {
          if ((lane & 7) == (j & 7))
            *reinterpret_cast<uint32_t*>(sm.p_tile[b] + swizzle64((row0 + j) * 64 + (t >> 3) * 4)) = words[j];
        }
      }
      // And the scale bytes into the operand's scale atom: (row r, group g) at r * 16 + g, the
      // second atom of an NVFP4 step 512 bytes on.
      if constexpr (MX) {
        if (lane < R) {
          int mine = mx_exponent[0];
#pragma unroll
          for (int j = 1; j < R; ++j) mine = lane == j ? mx_exponent[j] : mine;
          sm.p_sf[b][(row0 + lane) * 16 + warp_q] = (uint8_t)(mine + 127);
        }
      } else if constexpr (kScatter) {
        if (stores_sf) sm.p_sf[b][sf_offset] = (uint8_t)cvt_e4m3(own_scale);
      } else {
#pragma unroll
        for (int j = 0; j < R; ++j) {
          if ((lane & 15) == j)
            sm.p_sf[b][(group >> 2) * 512 + (row0 + j) * 16 + (group & 3)] = (uint8_t)cvt_e4m3(group_scale[j]);
        }
      }
      if (t == 0) sm.pv_fresh[b] = (grows || i == 0) ? 1 : 0;  // the CTA's first product always starts the sum
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(&sm.p_full[b]);

    }
    if constexpr (kStatsInSmem) {
#pragma unroll
      for (int j = 0; j < R; ++j) st.row_max[j] = sm.stat_row_max[row0 + j];
    }
    if (num_pages > 0) {
      const int pb = (num_pages - 1) & 1;
      tc::mbar_wait(&sm.o_full[pb], ((num_pages - 1) >> 1) & 1, abort_flag);
      tc::fence_after_sync();
      float o[LD];
      tc::tmem_ld<LD>(lane_base + kColO, o);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
#pragma unroll
      for (int j = 0; j < R; ++j) st.o_acc[j] += o[j];  // the sum since the last move of a maximum
    }
    if (with_bf16 && p.seqused_sink) {
      bf16_block<R>(st, sm, p, t, warp_q, lane, tail_k + (int64_t)kPage * row_elems,
                    tail_v + (int64_t)kPage * row_elems, 0, sink_len, shift, red_buf, row0, barrier);
    }

    // ---- normalise and write ------------------------------------------------------------------
    float total[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float v = st.row_sum[j];
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) v += __shfl_xor_sync(0xffffffffu, v, step);
      total[j] = v;
    }
    if (lane < R) {
      float mine = total[0];
#pragma unroll
      for (int j = 1; j < R; ++j) mine = lane == j ? total[j] : mine;
      sm.sum_red[warp_q][row0 + lane] = mine;
    }
    softmax_barrier(barrier);
#pragma unroll
    for (int j = 0; j < R; ++j)
      total[j] = (sm.sum_red[0][row0 + j] + sm.sum_red[1][row0 + j]) + (sm.sum_red[2][row0 + j] + sm.sum_red[3][row0 + j]);
    const bool skip = p.num_splits > 1 && part == p.num_splits && p.tail_key == nullptr;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      if (row0 + j < G) {
        const bool empty = skip || total[j] == 0.0f || total[j] != total[j];
        const float value = empty ? 0.0f : st.o_acc[j] * (1.0f / total[j]) * p.out_scale;
        const int head = kv_head * G + row0 + j;
        if (p.out != nullptr) {
          p.out[(int64_t)row * p.out_row_stride + head * kHeadDim + t] = __float2bfloat16_rn(value);
        } else {
          if (!skip) p.partial_out[(((int64_t)part * p.rows + row) * p.heads_q + head) * kHeadDim + t] = value;
          if (t == j) {
            const float safe = st.row_max[j] == -INFINITY ? 0.0f : st.row_max[j];
            const float lse = empty ? -INFINITY
                                    : (safe * p.scale_log2 + log2f(total[j]) - shift) * 0.6931471805599453f;
            p.partial_lse[((int64_t)part * p.rows + row) * p.heads_q + head] = lse;
          }
        }
      }
    }
    if (p.merge_counters != nullptr) {
      // Fused split merge: every part publishes its partials, then takes a ticket on the tile's
      // counter; the part that draws the last ticket reads all of them back (from L2) and writes
      // the BF16 output exactly as the separate merge kernel would, in part order, and leaves the
      // counter at zero for the next launch (src/nvfp4_decode_kernel/split_k_combine.py:47-83).
      // (every softmax group of the CTA must have published before the ticket is drawn: barrier 15
      // spans all of them)
      __threadfence();
      all_softmax_barrier<kSoftmaxThreads>();
      const int tile = row * p.heads_kv + kv_head;
      if (t == 0 && sgroup == 0) sm.merge_last = atomicAdd(&p.merge_counters[tile], 1) == p.parts - 1;
      all_softmax_barrier<kSoftmaxThreads>();
      if (sm.merge_last) {
        __threadfence();
        if (t == 0 && sgroup == 0) p.merge_counters[tile] = 0;
        constexpr float kLog2e = 1.4426950408889634f;
        const int64_t lse_stride = (int64_t)p.rows * p.heads_q;
        // This CTA sits on the launch's critical path (every tile's last part ends with the kernel),
        // so its reads must not queue behind one another: all the tile's LSEs come in with one
        // parallel load into shared memory (the first K stage, long consumed), and a head's partial
        // values are fetched eight parts at a time before any of them is used. The arithmetic and its
        // order are those of the merge kernel.
        float* staged = reinterpret_cast<float*>(sm.k_stage[0]);  // [part][G]
        const int staged_parts = min(p.parts, (int)(sizeof(sm.k_stage[0]) / sizeof(float)) / G);
        for (int i = t; i < staged_parts * R; i += 128) {
          const int s = i / R, j = row0 + i % R;
          if (j < G) staged[s * G + j] = __ldcg(p.partial_lse + s * lse_stride + (int64_t)row * p.heads_q + kv_head * G + j);
        }
        softmax_barrier(barrier);
        for (int j = row0; j < min(row0 + R, G); ++j) {  // each group merges the heads it owns
          const int head = kv_head * G + j;
          const float* lse = p.partial_lse + (int64_t)row * p.heads_q + head;
          const float* values = p.partial_out + ((int64_t)row * p.heads_q + head) * kHeadDim + t;
          auto lse_of = [&](int s) { return s < staged_parts ? staged[s * G + j] : __ldcg(lse + s * lse_stride); };
          float lse_max = -INFINITY;
          for (int s = 0; s < p.parts; ++s) lse_max = fmaxf(lse_max, lse_of(s));
          if (lse_max == -INFINITY) lse_max = 0.0f;
          float weight_sum = 0.0f;
          for (int s = 0; s < p.parts; ++s) weight_sum += exp2f(lse_of(s) * kLog2e - lse_max * kLog2e);
          const float inverse = (weight_sum == 0.0f || weight_sum != weight_sum) ? 0.0f : 1.0f / weight_sum;
          float acc = 0.0f;
          for (int s0 = 0; s0 < p.parts; s0 += 8) {
            float fetched[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              fetched[u] = s0 + u < p.parts ? __ldcg(values + (s0 + u) * lse_stride * kHeadDim) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              if (s0 + u < p.parts) {
                const float scale = exp2f(lse_of(s0 + u) * kLog2e - lse_max * kLog2e) * inverse;
                if (scale > 0.0f) acc = acc + scale * fetched[u];
              }
            }
          }
          p.merged_out[(int64_t)row * p.out_row_stride + head * kHeadDim + t] = __float2bfloat16_rn(acc);
        }
      }
    }
  }

  // ---- teardown -------------------------------------------------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0 && sm.abort_flag && p.error_word) atomicOr(p.error_word, (int)BDFP4_DEV_WAIT_TIMEOUT);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemColumns);
  }
}

// ---- launch ----------------------------------------------------------------------------------

template <int GP, int TERMS, int STAGES, int PT, bool MX, int SG = 1>
static cudaError_t launch_decode_staged(const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeParams& p,
                                        cudaStream_t stream) {
  const int smem = (int)sizeof(DecodeSmem<GP, STAGES>) + 1024;
  static PerDeviceOnce configured;
  const int slot = current_device_slot();
  if (slot < 0 || !configured.done[slot]) {
    cudaError_t e = cudaFuncSetAttribute(decode_kernel<GP, TERMS, STAGES, PT, MX, SG>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (slot >= 0) configured.done[slot] = true;
  }
  const int grid = p.rows * p.heads_kv * p.parts;
  // Programmatic stream serialization: after the query quantizer (which signals early) the CTAs
  // come up, set up and request their first cache pages while it still runs; after any other kernel
  // the launch starts when that kernel has finished, as an ordinary launch would.
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(decode_threads(SG));
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, decode_kernel<GP, TERMS, STAGES, PT, MX, SG>, k_map, v_map, p);
}

// Ring depth follows the grid: a launch with more than two CTAs per SM is given two K and two V
// stages per CTA so that four CTAs (and their four independent softmax chains) share an SM and
// the whole grid is resident at once; a smaller launch gets deeper rings instead.
template <int GP, int TERMS, int PT, bool MX>
static cudaError_t launch_decode(const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeParams& p,
                                 cudaStream_t stream) {
  static std::atomic<int> sm_counts[kDeviceSlots] = {};
  const int slot = current_device_slot();
  int sms = slot >= 0 ? sm_counts[slot].load() : 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (slot >= 0) sm_counts[slot] = sms;
  }
  const int grid = p.rows * p.heads_kv * p.parts;
  if constexpr (GP <= 8) {
    if (grid > 2 * sms) return launch_decode_staged<GP, TERMS, 2, PT, MX>(k_map, v_map, p, stream);
    return launch_decode_staged<GP, TERMS, 5, PT, MX>(k_map, v_map, p, stream);
  } else {
    return launch_decode_staged<GP, TERMS, 4, PT, MX>(k_map, v_map, p, stream);
  }
}

}  // namespace bdfp4
