// Shared device helpers: NVFP4 conversions and the block-scale search.
//
// The arithmetic follows the quantizer of OpenBitSys/BitDecoding-FP4
// (src/nvfp4_decode_kernel/_block_scale.py:218-327) operation for operation, because
// its results feed an argmin whose candidates are often one float apart:
//   scale   = E4M3_rn_satfinite(amax * fl32(1/divisor))        (a multiply, not a divide)
//   inverse = 1.0f / (scale + 1e-30f)                           (IEEE division)
//   codes   = cvt.rn.satfinite.e2m1x2.f32(x * inverse)
//   error   = sum_i fma(d_i, d_i, error), d_i = fma(mag_i, scale, -x_i), in element order,
//             with mag_i read back from the stored nibble
//   a later candidate wins only on a strictly smaller error.
// Every step is spelled with a rounding-explicit intrinsic so nvcc can neither contract
// nor reassociate it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bdfp4 {

constexpr int kPage = 128;
constexpr int kHeadDim = 128;
constexpr int kGroup = 16;
constexpr int kGroupsPerVec = kHeadDim / kGroup;  // 8
constexpr int kMaxCandidates = 3;

// MXFP4 exponent rules (src/nvfp4_decode_kernel/scale_mode.py:40-49); 0 = an NVFP4 mode
constexpr int kMxNone = 0, kMxOcp = 1, kMxRoundUp = 2, kMxSearch = 3;

struct ScaleCandidates {
  int count;
  float reciprocal[kMaxCandidates];  // fl32(1/divisor), tie-break order
  int mx_rule;                       // kMx*: E8M0 scale per 32 values instead of the candidates above
};

// `mode` is a BDFP4_SCALE_* id: 0-2 NVFP4 candidate sets, 3-5 the MXFP4 rules.
__host__ __device__ inline ScaleCandidates scale_candidates(int mode) {
  ScaleCandidates c;
  c.count = 1;
  c.reciprocal[0] = (float)(1.0 / 6.0);
  c.reciprocal[1] = (float)(1.0 / 4.0);
  c.reciprocal[2] = (float)(1.0 / 6.5);
  c.mx_rule = kMxNone;
  if (mode == 1) c.count = 2;
  if (mode == 2) c.count = 3;
  if (mode >= 3) c.mx_rule = mode - 2;
  return c;
}

// Two floats -> one byte of two E2M1 codes; `lo` lands in the low nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t out;
  asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tcvt.u16.u8 %0, b;\n\t}"
      : "=h"(out)
      : "f"(hi), "f"(lo));
  return (uint32_t)out;
}

__device__ __forceinline__ uint32_t pack_e2m1x8(const float* v) {
  return cvt_e2m1x2(v[0], v[1]) | (cvt_e2m1x2(v[2], v[3]) << 8) | (cvt_e2m1x2(v[4], v[5]) << 16) |
         (cvt_e2m1x2(v[6], v[7]) << 24);
}

// One byte of two E2M1 codes -> their two values (low nibble first).
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
  uint32_t pair;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(pair) : "r"(byte & 0xffu));
  __half2 h = *reinterpret_cast<__half2*>(&pair);
  return __half22float2(h);
}

// float -> E4M3 byte, round-to-nearest-even, saturating at 448.
__device__ __forceinline__ uint32_t cvt_e4m3(float x) {
  uint16_t out;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(0.0f), "f"(x));
  return (uint32_t)(out & 0xffu);
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  uint32_t pair;
  uint16_t in = (uint16_t)(byte & 0xffu);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(in));
  __half2 h = *reinterpret_cast<__half2*>(&pair);
  return __low2float(h);
}

struct GroupCodes {
  float scale;    // the E4M3 value the group stores, as a float
  uint32_t lo;    // elements 0..7, element 0 in the lowest nibble
  uint32_t hi;    // elements 8..15
};

// One candidate over one group of sixteen values: the codes it would store.
__device__ __forceinline__ void encode16(const float* x, float scale, uint32_t& lo, uint32_t& hi) {
  const float inverse = __fdiv_rn(1.0f, __fadd_rn(scale, 1.0e-30f));
  float scaled[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) scaled[i] = __fmul_rn(x[i], inverse);
  lo = pack_e2m1x8(scaled);
  hi = pack_e2m1x8(scaled + 8);
}

// Squared reconstruction error of stored codes, accumulated by FMA in element order.
__device__ __forceinline__ float reconstruction_error16(const float* x, float scale, uint32_t lo, uint32_t hi) {
  float error = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t word = (i < 4) ? lo : hi;
    const float2 m0 = e2m1x2_to_float2(word >> (8 * (i & 3)));
    const int e = 2 * i;
    float d = __fmaf_rn(m0.x, scale, -x[e]);
    error = __fmaf_rn(d, d, error);
    d = __fmaf_rn(m0.y, scale, -x[e + 1]);
    error = __fmaf_rn(d, d, error);
  }
  return error;
}

__device__ __forceinline__ float candidate_scale(float amax, float reciprocal) {
  return e4m3_to_float(cvt_e4m3(__fmul_rn(amax, reciprocal)));
}

// Two candidates priced together: every multiply and FMA runs as one packed FP32x2 instruction
// with candidate A in the low lane and B in the high lane. Each lane rounds on its own, so the
// errors are bit for bit those of two scalar evaluations.
__device__ __forceinline__ void price_two16(const float* x, float scale_a, float scale_b, uint32_t& lo_a,
                                            uint32_t& hi_a, uint32_t& lo_b, uint32_t& hi_b, float& error_a,
                                            float& error_b) {
  const float2 scale = make_float2(scale_a, scale_b);
  const float2 inverse = make_float2(__fdiv_rn(1.0f, __fadd_rn(scale_a, 1.0e-30f)),
                                     __fdiv_rn(1.0f, __fadd_rn(scale_b, 1.0e-30f)));
  float2 error = make_float2(0.0f, 0.0f);
  uint32_t words_a[2] = {0, 0}, words_b[2] = {0, 0};
#pragma unroll
  for (int pair = 0; pair < 8; ++pair) {
    const float x0 = x[2 * pair], x1 = x[2 * pair + 1];
    const float2 s0 = __fmul2_rn(make_float2(x0, x0), inverse);
    const float2 s1 = __fmul2_rn(make_float2(x1, x1), inverse);
    const uint32_t byte_a = cvt_e2m1x2(s0.x, s1.x);
    const uint32_t byte_b = cvt_e2m1x2(s0.y, s1.y);
    words_a[pair >> 2] |= byte_a << (8 * (pair & 3));
    words_b[pair >> 2] |= byte_b << (8 * (pair & 3));
    const float2 mag_a = e2m1x2_to_float2(byte_a);
    const float2 mag_b = e2m1x2_to_float2(byte_b);
    float2 d = __ffma2_rn(make_float2(mag_a.x, mag_b.x), scale, make_float2(-x0, -x0));
    error = __ffma2_rn(d, d, error);
    d = __ffma2_rn(make_float2(mag_a.y, mag_b.y), scale, make_float2(-x1, -x1));
    error = __ffma2_rn(d, d, error);
  }
  lo_a = words_a[0];
  hi_a = words_a[1];
  lo_b = words_b[0];
  hi_b = words_b[1];
  error_a = error.x;
  error_b = error.y;
}

// The group's winning scale and codes under `cand` (first candidate wins ties). With a single
// candidate there is nothing to compare, so no error is computed.
__device__ __forceinline__ GroupCodes quantize_group16(const float* x, const ScaleCandidates& cand) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  GroupCodes best;
  best.scale = candidate_scale(amax, cand.reciprocal[0]);
  if (cand.count == 1) {
    encode16(x, best.scale, best.lo, best.hi);
    return best;
  }
  const float scale_b = candidate_scale(amax, cand.reciprocal[1]);
  uint32_t lo_b, hi_b;
  float best_error, error_b;
  price_two16(x, best.scale, scale_b, best.lo, best.hi, lo_b, hi_b, best_error, error_b);
  if (error_b < best_error) {
    best.scale = scale_b;
    best.lo = lo_b;
    best.hi = hi_b;
    best_error = error_b;
  }
  for (int c = 2; c < cand.count; ++c) {
    const float scale = candidate_scale(amax, cand.reciprocal[c]);
    uint32_t lo, hi;
    encode16(x, scale, lo, hi);
    const float error = reconstruction_error16(x, scale, lo, hi);
    if (error < best_error) {
      best.scale = scale;
      best.lo = lo;
      best.hi = hi;
      best_error = error;
    }
  }
  return best;
}

// ---- MXFP4: E2M1 codes on a power-of-two scale shared by 32 values ---------------------------
// (src/nvfp4_decode_kernel/_block_scale.py:384-546, CPU model src/nvfp4_decode_kernel/reference.py:262-328)

// 2^e for an E8M0 exponent in [-127, 127]; 2^-127 is the one subnormal.
__device__ __forceinline__ float mx_power_of_two(int e) {
  return __uint_as_float(e < -126 ? (1u << 22) : ((uint32_t)(e + 127) << 23));
}

// floor(log2(amax)) - 2 clamped below at -127, read off the exponent field: a zero or subnormal
// maximum lands on the clamp (_block_scale.py:418-427).
__device__ __forceinline__ int mx_ocp_exponent(float amax) {
  return max((int)((__float_as_uint(amax) >> 23) & 0xffu) - 129, -127);
}

// The smallest exponent whose scale keeps amax at or below six: one more than the OCP exponent
// exactly when the mantissa is above 1.5, which is when adding 0x3FFFFF carries into the exponent
// field (_block_scale.py:430-440).
__device__ __forceinline__ int mx_round_up_exponent(float amax) {
  return max((int)((__float_as_uint(amax) + 0x3FFFFFu) >> 23) - 129, -127);
}

// The stored byte of a power-of-two scale: its exponent field (0 for 2^-127).
__device__ __forceinline__ uint32_t e8m0_byte(float scale) { return (__float_as_uint(scale) >> 23) & 0xffu; }

// Sixteen values on the scale 2^e: their codes and the squared error of this half of the group.
__device__ __forceinline__ void mx_encode16(const float* x, int e, uint32_t& lo, uint32_t& hi, float& error) {
  const float scale = mx_power_of_two(e), inverse = mx_power_of_two(-e);
  float scaled[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) scaled[i] = __fmul_rn(x[i], inverse);
  lo = pack_e2m1x8(scaled);
  hi = pack_e2m1x8(scaled + 8);
  error = reconstruction_error16(x, scale, lo, hi);
}

// One lane's half of a 32-value group that it shares with the adjacent lane (lane ^ 1): the
// maximum and, under the search rule, the two halves' errors are exchanged by shuffle; a half's
// error is accumulated by FMA in element order and the group's is the one FP32 sum of the halves
// (reference.py:113-118). Every lane of the warp must call it.
__device__ __forceinline__ GroupCodes mx_quantize_pair16(const float* x, int rule) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  int e = rule == kMxRoundUp ? mx_round_up_exponent(amax) : mx_ocp_exponent(amax);
  GroupCodes best;
  float error;
  mx_encode16(x, e, best.lo, best.hi, error);
  if (rule == kMxSearch) {
    const int above = min(e + 1, 127);
    uint32_t lo, hi;
    float error_above;
    mx_encode16(x, above, lo, hi, error_above);
    const float total = __fadd_rn(error, __shfl_xor_sync(0xffffffffu, error, 1));
    const float total_above = __fadd_rn(error_above, __shfl_xor_sync(0xffffffffu, error_above, 1));
    if (total_above < total) {
      e = above;
      best.lo = lo;
      best.hi = hi;
    }
  }
  best.scale = mx_power_of_two(e);
  return best;
}

// A whole 32-value group held by one thread: `words` receives its 16 bytes of codes.
__device__ __forceinline__ float mx_quantize32(const float* x, int rule, uint32_t* words) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
  int e = rule == kMxRoundUp ? mx_round_up_exponent(amax) : mx_ocp_exponent(amax);
  float error0, error1;
  mx_encode16(x, e, words[0], words[1], error0);
  mx_encode16(x + 16, e, words[2], words[3], error1);
  if (rule == kMxSearch) {
    const int above = min(e + 1, 127);
    uint32_t other[4];
    float above0, above1;
    mx_encode16(x, above, other[0], other[1], above0);
    mx_encode16(x + 16, above, other[2], other[3], above1);
    if (__fadd_rn(above0, above1) < __fadd_rn(error0, error1)) {
      e = above;
#pragma unroll
      for (int i = 0; i < 4; ++i) words[i] = other[i];
    }
  }
  return mx_power_of_two(e);
}

// x - decode(codes) * scale for one group, one rounding per element
// (src/nvfp4_decode_kernel/_block_scale.py:602-623).
__device__ __forceinline__ void group_residual16(const float* x, const GroupCodes& q, float* residual) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t word = (i < 4) ? q.lo : q.hi;
    const float2 m = e2m1x2_to_float2(word >> (8 * (i & 3)));
    residual[2 * i] = __fmaf_rn(-m.x, q.scale, x[2 * i]);
    residual[2 * i + 1] = __fmaf_rn(-m.y, q.scale, x[2 * i + 1]);
  }
}

// Sixteen BF16 values (32 bytes, 16-byte aligned) -> FP32.
__device__ __forceinline__ void load_bf16x16(const __nv_bfloat16* p, float* out) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void store_bf16x16(__nv_bfloat16* p, const float* v) {
  uint4 a, b;
  a.x = pack_bf16x2(v[0], v[1]);
  a.y = pack_bf16x2(v[2], v[3]);
  a.z = pack_bf16x2(v[4], v[5]);
  a.w = pack_bf16x2(v[6], v[7]);
  b.x = pack_bf16x2(v[8], v[9]);
  b.y = pack_bf16x2(v[10], v[11]);
  b.z = pack_bf16x2(v[12], v[13]);
  b.w = pack_bf16x2(v[14], v[15]);
  reinterpret_cast<uint4*>(p)[0] = a;
  reinterpret_cast<uint4*>(p)[1] = b;
}

// Round sixteen FP32 values to BF16 and back, in place.
__device__ __forceinline__ void round_to_bf16(float* v) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
}

// Unnormalised Sylvester-Hadamard butterflies over one 128-channel head held by 8 adjacent
// lanes, sixteen channels each (lane `group` owns channels 16*group..16*group+15). Index bits
// are taken lowest first and each stage maps (a, c) -> (a + c, a - c) in FP32, which is the
// order of src/nvfp4_decode_kernel/quantize_q_kernel.py:105-135 and of
// src/nvfp4_decode_kernel/quantize_kv_kernel.py:123-162.
__device__ __forceinline__ void hadamard_butterflies(float* v, int group) {
  // stride 1 inside each adjacent pair; the wider strides and the cross-lane stages work on
  // adjacent pairs with packed FP32x2 instructions (each lane rounds like the scalar add or
  // subtract: a - c == fma(c, -1, a) exactly)
  float2 p[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float lo = v[2 * k], hi = v[2 * k + 1];
    p[k] = make_float2(__fadd_rn(lo, hi), __fsub_rn(lo, hi));
  }
  const float2 minus = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int stride = 1; stride < 8; stride <<= 1) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if ((k & stride) == 0) {
        const float2 lo = p[k], hi = p[k + stride];
        p[k] = __fadd2_rn(lo, hi);
        p[k + stride] = __ffma2_rn(hi, minus, lo);
      }
    }
  }
#pragma unroll
  for (int bit = 0; bit < 3; ++bit) {
    const int mask = 1 << bit;
    // partner - own on the upper lane, own + partner on the lower
    const float sign = (group & mask) != 0 ? -1.0f : 1.0f;
    const float2 sign2 = make_float2(sign, sign);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 own = p[k];
      const float2 partner = make_float2(__shfl_xor_sync(0xffffffffu, own.x, mask),
                                         __shfl_xor_sync(0xffffffffu, own.y, mask));
      p[k] = __ffma2_rn(own, sign2, partner);
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    v[2 * k] = p[k].x;
    v[2 * k + 1] = p[k].y;
  }
}

constexpr float kInvSqrt128 = 0.08838834764831845f;  // fl32(1/sqrt(128))

// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute
// may start while the kernel before it in the stream is still running, once that kernel has called
// dependents_may_launch() in every CTA (or finished); what it reads or writes of that kernel's
// data must come after wait_for_prior_kernels(), which returns when the earlier kernels have
// completed and their writes are visible. Both are no-ops in an ordinary launch.
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_prior_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Byte offset of (row, group) inside one head's 1024-byte scale tile.
__host__ __device__ __forceinline__ int scale_tile_offset(int row, int group) {
  return (group >> 2) * 512 + (row & 31) * 16 + (row >> 5) * 4 + (group & 3);
}

}  // namespace bdfp4
