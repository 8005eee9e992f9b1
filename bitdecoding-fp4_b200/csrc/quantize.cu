// NVFP4 quantize-on-write kernels: K pages, V pages, BF16 tail/sink tokens and the decode
// query. One thread owns one 16-value scale group; a head vector is eight adjacent lanes, so
// global loads are 256-byte coalesced runs and the Hadamard's upper three index bits are
// warp shuffles. Scale bytes are staged in shared memory and leave as whole 1024-byte tiles.
#include <cmath>

#include "common.cuh"
#include "host.h"

namespace bdfp4 {

struct KvWriteParams {
  const __nv_bfloat16* key;
  const __nv_bfloat16* value;
  int64_t key_pitch, value_pitch;  // elements per token
  int64_t source_layer_stride;     // tokens
  int heads;
  uint8_t* region[4];  // K codes, K scales, V codes, V scales (one-layer form)
  int64_t pitch[4];    // bytes per page
  const int64_t* bases;  // [4][layers] or null
  int layers;
  const int32_t* source_tokens;
  const int32_t* destination_pages;
  int work_items;
  ScaleCandidates key_cand, value_cand;
  const void* key_shift;  // [layers][H][128]
  int layer;
  // tail role
  __nv_bfloat16* tail_key;
  __nv_bfloat16* tail_value;
  int64_t tail_layer_stride, tail_slot_stride;
  int sink_tokens;
  const int32_t* query_start_loc;
  const int32_t* seq_lens;
  const int32_t* seqused_fp4;
  const int32_t* row_to_slot;
  int rows, decode_rows, first_row;
  int pages;              // pages in each destination region (0: unknown)
  int32_t* error_word;
  float key_inverse_scale, value_inverse_scale;  // fl32(1 / tensor scale); 1 when there is none
};

// A work item's destination page, or -1 when the item is to be skipped: a negative id by
// convention, an id past the cache because a corrupt work table must not write outside it
// (that one is reported).
__device__ __forceinline__ int destination_page(const KvWriteParams& p, int work) {
  const int page = p.destination_pages[work];
  if (page >= 0 && p.pages > 0 && page >= p.pages) {
    if (threadIdx.x == 0 && p.error_word) atomicOr(p.error_word, (int)BDFP4_DEV_BAD_PAGE);
    return -1;
  }
  return page;
}

// The pages hold x / tensor_scale: a multiplication by the reciprocal, rounded once.
__device__ __forceinline__ void apply_inverse_scale(float* v, float inverse, int n = 16) {
  if (inverse != 1.0f) {
#pragma unroll
    for (int j = 0; j < n; ++j) v[j] = __fmul_rn(v[j], inverse);
  }
}

template <int SHIFT_TYPE>
__device__ __forceinline__ void load_shift16(const void* shift, int64_t offset, float* out) {
  if (SHIFT_TYPE == BDFP4_SHIFT_F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(shift) + offset);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(p + i);
      out[4 * i] = v.x;
      out[4 * i + 1] = v.y;
      out[4 * i + 2] = v.z;
      out[4 * i + 3] = v.w;
    }
  } else if (SHIFT_TYPE == BDFP4_SHIFT_BF16) {
    load_bf16x16(static_cast<const __nv_bfloat16*>(shift) + offset, out);
  }
}

// Raw K -> the basis the cache stores: rotate, scale by 1/sqrt(128), subtract the shift, round
// to BF16 once. The multiply and the subtract round separately
// (src/nvfp4_decode_kernel/quantize_kv_kernel.py:123-162).
template <int SHIFT_TYPE, bool ROTATE>
__device__ __forceinline__ void cache_basis16(float* v, int group, const void* shift, int64_t shift_offset) {
  if (ROTATE) {
    hadamard_butterflies(v, group);
    const float inverse = (float)0.08838834764831845;
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], inverse);
  }
  if (SHIFT_TYPE != BDFP4_SHIFT_NONE) {
    float centre[16];
    load_shift16<SHIFT_TYPE>(shift, shift_offset, centre);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fsub_rn(v[j], centre[j]);
  }
  if (ROTATE || SHIFT_TYPE != BDFP4_SHIFT_NONE) round_to_bf16(v);
}

// 64-token pages are stored as the decode kernel's shared-memory images, one contiguous block per
// (page, head), so that the kernel fetches them with plain bulk copies:
//   K codes [H][64 tok][64 B]   16-byte chunk j of token t at position j ^ ((t >> 1) & 3)
//   V codes [H][128 ch][32 B]   16-byte chunk j of channel c at position j ^ ((c >> 2) & 1)
// Byte of (token, channel group) inside a 64-token page's 512-byte K scale block: two half
// atoms [group / 4][token % 32][token / 32][group % 4]. The decode kernel interleaves the halves
// of two such pages into the 128-row atoms its MMA reads.
__host__ __device__ __forceinline__ int key_scale_offset64(int token, int group) {
  return (group >> 2) * 256 + (token & 31) * 8 + (token >> 5) * 4 + (group & 3);
}

// One CTA = one head of one K page of PT tokens: 8 * PT scale groups, PT / 32 per thread.
template <int SHIFT_TYPE, bool ROTATE, int PT, bool MX>
__device__ __forceinline__ void key_page_body(const KvWriteParams& p, int item, int grid_layer, uint8_t* scale_tile) {
  // MXFP4 (128-token pages only) stores one E8M0 byte per 32 channels: half the scale bytes
  constexpr bool mx = MX;
  constexpr int scale_bytes = mx ? PT * 4 : PT * 8;
  const int layer = p.bases ? grid_layer : p.layer;
  const int head = item % p.heads;
  const int work = item / p.heads;
  const int page = destination_page(p, work);
  if (page < 0) return;
  const int64_t source_token = (int64_t)p.source_tokens[work] + (int64_t)grid_layer * p.source_layer_stride;
  uint8_t* codes = p.bases ? reinterpret_cast<uint8_t*>(p.bases[0 * p.layers + layer]) : p.region[0];
  uint8_t* scales = p.bases ? reinterpret_cast<uint8_t*>(p.bases[1 * p.layers + layer]) : p.region[1];
  codes += (int64_t)page * p.pitch[0];
  scales += (int64_t)page * p.pitch[1] + head * scale_bytes;

#pragma unroll 1
  for (int it = 0; it < PT / 32; ++it) {
    const int index = it * 256 + threadIdx.x;
    const int token = index >> 3;
    const int group = index & 7;
    float v[16];
    load_bf16x16(p.key + (source_token + token) * p.key_pitch + head * kHeadDim + group * kGroup, v);
    cache_basis16<SHIFT_TYPE, ROTATE>(v, group, p.key_shift,
                                      ((int64_t)layer * p.heads + head) * kHeadDim + group * kGroup);
    apply_inverse_scale(v, p.key_inverse_scale);
    // an MXFP4 group of 32 channels is shared by the lanes holding channel groups 2k and 2k + 1
    GroupCodes q;
    if constexpr (mx) q = mx_quantize_pair16(v, p.key_cand.mx_rule);
    else q = quantize_group16(v, p.key_cand);
    if constexpr (PT == 128) {
      *reinterpret_cast<uint2*>(codes + ((int64_t)token * p.heads + head) * 64 + group * 8) = make_uint2(q.lo, q.hi);
    } else {
      // head-major rows whose 16-byte chunks sit where the 64-byte shared-memory swizzle wants them
      const int chunk = (group >> 1) ^ ((token >> 1) & 3);
      *reinterpret_cast<uint2*>(codes + (int64_t)head * (PT * 64) + token * 64 + chunk * 16 + (group & 1) * 8) =
          make_uint2(q.lo, q.hi);
    }
    if constexpr (mx) {
      // one atom per head: (token, 32-channel group g) at (token % 32) * 16 + (token / 32) * 4 + g
      if ((group & 1) == 0) scale_tile[scale_tile_offset(token, group >> 1)] = (uint8_t)e8m0_byte(q.scale);
    } else {
      scale_tile[PT == 128 ? scale_tile_offset(token, group) : key_scale_offset64(token, group)] =
          (uint8_t)cvt_e4m3(q.scale);
    }
  }
  __syncthreads();
  if (threadIdx.x < scale_bytes / 4)
    reinterpret_cast<uint32_t*>(scales)[threadIdx.x] = reinterpret_cast<const uint32_t*>(scale_tile)[threadIdx.x];
}

template <int SHIFT_TYPE, bool ROTATE, int PT, bool MX>
__global__ void __launch_bounds__(256) key_page_kernel(const KvWriteParams p) {
  __shared__ __align__(16) uint8_t scale_tile[PT * 8];
  key_page_body<SHIFT_TYPE, ROTATE, PT, MX>(p, blockIdx.x, blockIdx.z, scale_tile);
}

// One CTA = one head of one V page of PT tokens. Scale groups run along the page's tokens, so the
// [token][channel] tile is staged in shared memory and read back by columns. A channel's codes
// are PT / 2 bytes; its PT / 16 scales sit at the 128-token layout's offsets (one atom per 64 tokens).
template <int PT>
struct ValueTile {
  static constexpr int kCodeBytes = PT / 2;         // per channel
  static constexpr int kCodePitch = kCodeBytes + 8;  // staging pitch (bank spread)
  static constexpr int kScaleBytes = PT * 8;
  static constexpr int kSmem = PT * kHeadDim * 2 + kHeadDim * kCodePitch + kScaleBytes;
};

template <int PT, bool MX>
__device__ __forceinline__ void value_page_body(const KvWriteParams& p, int item, int grid_layer, uint8_t* smem) {
  using T = ValueTile<PT>;
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem);  // [PT][128]
  uint8_t* code_tile = smem + PT * kHeadDim * 2;                 // [128][kCodePitch]
  uint8_t* scale_tile = code_tile + kHeadDim * T::kCodePitch;    // [kScaleBytes]
  constexpr bool mx = MX;
  constexpr int scale_bytes = mx ? T::kScaleBytes / 2 : T::kScaleBytes;
  const int layer = p.bases ? grid_layer : p.layer;
  const int head = item % p.heads;
  const int work = item / p.heads;
  const int page = destination_page(p, work);
  if (page < 0) return;
  const int64_t source_token = (int64_t)p.source_tokens[work] + (int64_t)grid_layer * p.source_layer_stride;
  uint8_t* codes = p.bases ? reinterpret_cast<uint8_t*>(p.bases[2 * p.layers + layer]) : p.region[2];
  uint8_t* scales = p.bases ? reinterpret_cast<uint8_t*>(p.bases[3 * p.layers + layer]) : p.region[3];
  codes += (int64_t)page * p.pitch[2] + (int64_t)head * (kHeadDim * T::kCodeBytes);
  scales += (int64_t)page * p.pitch[3] + head * scale_bytes;

#pragma unroll
  for (int it = 0; it < PT / 16; ++it) {
    const int index = it * 256 + threadIdx.x;  // 16-byte chunk of the tile
    const int token = index >> 4;
    const int chunk = index & 15;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.value + (source_token + token) * p.value_pitch +
                                                         head * kHeadDim + chunk * 8));
    reinterpret_cast<uint4*>(tile)[index] = v;
  }
  __syncthreads();
  if constexpr (mx) {
    // MXFP4: a thread owns a whole group of 32 tokens of one channel; one atom of E8M0 bytes per head
#pragma unroll 1
    for (int it = 0; it < PT / 64; ++it) {
      const int index = it * 256 + threadIdx.x;
      const int channel = index & 127;
      const int group = index >> 7;  // 32-token group
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[(group * 32 + i) * kHeadDim + channel]);
      apply_inverse_scale(v, p.value_inverse_scale, 32);
      uint32_t words[4];
      const float scale = mx_quantize32(v, p.value_cand.mx_rule, words);
      uint2* dst = reinterpret_cast<uint2*>(code_tile + channel * T::kCodePitch + group * 16);
      dst[0] = make_uint2(words[0], words[1]);
      dst[1] = make_uint2(words[2], words[3]);
      scale_tile[scale_tile_offset(channel, group)] = (uint8_t)e8m0_byte(scale);
    }
  } else {
#pragma unroll 1
    for (int it = 0; it < PT / 32; ++it) {
      const int index = it * 256 + threadIdx.x;
      const int channel = index & 127;
      const int group = index >> 7;  // token group
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(tile[(group * 16 + i) * kHeadDim + channel]);
      apply_inverse_scale(v, p.value_inverse_scale);
      const GroupCodes q = quantize_group16(v, p.value_cand);
      *reinterpret_cast<uint2*>(code_tile + channel * T::kCodePitch + group * 8) = make_uint2(q.lo, q.hi);
      scale_tile[scale_tile_offset(channel, group)] = (uint8_t)cvt_e4m3(q.scale);
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < PT / 32; ++it) {
    const int index = it * 256 + threadIdx.x;  // 8-byte chunk of the code tile
    const int channel = index / (T::kCodeBytes / 8);
    const int chunk = index % (T::kCodeBytes / 8);
    // a 64-token page stores each 32-byte row with its 16-byte halves placed as the 32-byte
    // shared-memory swizzle wants them
    const int dst = PT == 128 ? index : channel * 4 + ((((chunk >> 1) ^ ((channel >> 2) & 1)) << 1) | (chunk & 1));
    reinterpret_cast<uint2*>(codes)[dst] =
        *reinterpret_cast<const uint2*>(code_tile + channel * T::kCodePitch + chunk * 8);
  }
  if (threadIdx.x < scale_bytes / 4)
    reinterpret_cast<uint32_t*>(scales)[threadIdx.x] = reinterpret_cast<const uint32_t*>(scale_tile)[threadIdx.x];
}

template <int PT, bool MX>
__global__ void __launch_bounds__(256) value_page_kernel(const KvWriteParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  value_page_body<PT, MX>(p, blockIdx.x, blockIdx.z, smem);
}

// K and V pages in one launch: even CTAs quantize a K page head, odd CTAs the V page head of the
// same work item. The K role is bound by arithmetic and the V role by its loads and the staging
// tile, so CTAs of both kinds resident on one SM overlap instead of running back to back.
// (Five CTAs per SM measured faster for 64-token pages, four for 128-token pages.)
template <int SHIFT_TYPE, bool ROTATE, int PT, bool MX>
__global__ void __launch_bounds__(256, MX ? 2 : (PT == 64 ? 5 : 4)) kv_page_kernel(const KvWriteParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int item = blockIdx.x >> 1;
  if (blockIdx.x & 1)
    value_page_body<PT, MX>(p, item, blockIdx.z, smem);
  else
    key_page_body<SHIFT_TYPE, ROTATE, PT, MX>(p, item, blockIdx.z, smem);
}

// One 16-element group of one token's new K or V into the BF16 tail: at `offset` of the rolling
// page when that is not negative, and at 128 + position of the sink below `sink_tokens`.
// `item` runs over the token's K groups padded to whole warps, then its V groups
// (src/nvfp4_decode_kernel/quantize_q_kernel.py:138-258).
template <int SHIFT_TYPE, bool ROTATE>
__device__ __forceinline__ void write_tail_token(const __nv_bfloat16* key, const __nv_bfloat16* value,
                                                 int64_t key_pitch, int64_t value_pitch, const void* key_shift,
                                                 int64_t shift_layer_offset, __nv_bfloat16* tail_key,
                                                 __nv_bfloat16* tail_value, int64_t slot_stride, int64_t token,
                                                 int slot, int position, int offset, int item, int heads,
                                                 int sink_tokens) {
  const int items = heads * kGroupsPerVec;
  const int key_span = (items + 31) / 32 * 32;
  const int64_t row_elems = (int64_t)heads * kHeadDim;
  if (item < key_span) {
    const bool active = item < items;
    const int head = active ? item / kGroupsPerVec : heads - 1;
    const int group = item % kGroupsPerVec;
    float v[16];
    const __nv_bfloat16* src = key + token * key_pitch + head * kHeadDim + group * kGroup;
    const uint4 raw0 = __ldg(reinterpret_cast<const uint4*>(src));
    const uint4 raw1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    uint4 out0 = raw0, out1 = raw1;
    if (ROTATE || SHIFT_TYPE != BDFP4_SHIFT_NONE) {
      load_bf16x16(src, v);
      cache_basis16<SHIFT_TYPE, ROTATE>(v, group, key_shift,
                                        shift_layer_offset + (int64_t)head * kHeadDim + group * kGroup);
      out0 = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                        pack_bf16x2(v[6], v[7]));
      out1 = make_uint4(pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]),
                        pack_bf16x2(v[14], v[15]));
    }
    if (active && slot >= 0) {
      __nv_bfloat16* base = tail_key + (int64_t)slot * slot_stride + head * kHeadDim + group * kGroup;
      if (offset >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)offset * row_elems);
        dst[0] = out0;
        dst[1] = out1;
      }
      if (position < sink_tokens) {
        uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)(kPage + position) * row_elems);
        dst[0] = out0;
        dst[1] = out1;
      }
    }
  } else {
    const int v_index = item - key_span;
    if (v_index < items && slot >= 0) {
      const int head = v_index / kGroupsPerVec;
      const int group = v_index % kGroupsPerVec;
      const __nv_bfloat16* src = value + token * value_pitch + head * kHeadDim + group * kGroup;
      const uint4 raw0 = __ldg(reinterpret_cast<const uint4*>(src));
      const uint4 raw1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
      __nv_bfloat16* base = tail_value + (int64_t)slot * slot_stride + head * kHeadDim + group * kGroup;
      if (offset >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)offset * row_elems);
        dst[0] = raw0;
        dst[1] = raw1;
      }
      if (position < sink_tokens) {
        uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)(kPage + position) * row_elems);
        dst[0] = raw0;
        dst[1] = raw1;
      }
    }
  }
}

__host__ __device__ inline int tail_chunks_for(int heads) {
  const int groups = heads * kGroupsPerVec;
  return ((groups + 31) / 32 * 32 + groups + 127) / 128;
}

// The writer's tail role: rows [first_row, decode_rows) get one candidate (their newest token);
// every later row gets 128 + sink_tokens candidates, one per rolling position past its FP4
// prefix and one per sink position (src/nvfp4_decode_kernel/quantize_kv_kernel.py:258-339).
template <int SHIFT_TYPE, bool ROTATE>
__global__ void __launch_bounds__(128) tail_token_kernel(const KvWriteParams p) {
  const int tail_chunks = tail_chunks_for(p.heads);
  const int item = blockIdx.x;
  const int candidates = kPage + p.sink_tokens;
  const int candidate = item / tail_chunks;
  const int decode_count = p.decode_rows - p.first_row;
  const bool is_decode = candidate < decode_count;
  const int later = candidate - decode_count;
  const int row = is_decode ? p.first_row + candidate : p.decode_rows + later / candidates;
  const int within = later % candidates;
  const int start = p.query_start_loc[row];
  const int seq_len = p.seq_lens[row];
  const int quantized = p.seqused_fp4[row];
  const int slot = p.row_to_slot[row];
  const int computed = seq_len - (p.query_start_loc[row + 1] - start);
  const bool rolling = within < kPage;
  const int position = is_decode ? seq_len - 1 : (rolling ? quantized + within : within - kPage);
  if (slot >= 0 && position < seq_len && position >= computed && (is_decode || rolling || position < quantized)) {
    write_tail_token<SHIFT_TYPE, ROTATE>(
        p.key, p.value, p.key_pitch, p.value_pitch, p.key_shift, (int64_t)p.layer * p.heads * kHeadDim,
        p.tail_key + (int64_t)p.layer * p.tail_layer_stride, p.tail_value + (int64_t)p.layer * p.tail_layer_stride,
        p.tail_slot_stride, (int64_t)start + position - computed, slot, position, position - quantized,
        (item % tail_chunks) * 128 + threadIdx.x, p.heads, p.sink_tokens);
  }
}

template <int PT, bool MX>
static cudaError_t launch_value_pages(const KvWriteParams& p, int page_items, cudaStream_t stream) {
  const int smem = ValueTile<PT>::kSmem;
  static PerDeviceOnce configured;
  const int slot = current_device_slot();
  if (slot < 0 || !configured.done[slot]) {
    cudaError_t e = cudaFuncSetAttribute(value_page_kernel<PT, MX>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (slot >= 0) configured.done[slot] = true;
  }
  value_page_kernel<PT, MX><<<dim3(page_items, 1, p.layers), 256, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int SHIFT_TYPE, bool ROTATE, int PT, bool MX>
static cudaError_t launch_kv_pages(const KvWriteParams& p, int page_items, cudaStream_t stream) {
  const int smem = ValueTile<PT>::kSmem;
  static PerDeviceOnce configured;
  const int slot = current_device_slot();
  if (slot < 0 || !configured.done[slot]) {
    cudaError_t e = cudaFuncSetAttribute(kv_page_kernel<SHIFT_TYPE, ROTATE, PT, MX>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (slot >= 0) configured.done[slot] = true;
  }
  kv_page_kernel<SHIFT_TYPE, ROTATE, PT, MX><<<dim3(2 * page_items, 1, p.layers), 256, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int SHIFT_TYPE, bool ROTATE>
static cudaError_t launch_kv_write(const KvWriteParams& p, int page_tokens, cudaStream_t stream) {
  const int page_items = p.heads * p.work_items;
  const bool key_pages = p.key && (p.region[0] || p.bases) && page_items > 0;
  const bool value_pages = p.value && (p.region[2] || p.bases) && page_items > 0;
  const bool mx_key = p.key_cand.mx_rule != kMxNone, mx_value = p.value_cand.mx_rule != kMxNone;
  const dim3 grid(page_items, 1, p.layers);
  // K and V pages of one scale format go in one launch; MXFP4 exists for 128-token pages only
  const bool fused = key_pages && value_pages && mx_key == mx_value;
  if (fused) {
    cudaError_t e = mx_key             ? launch_kv_pages<SHIFT_TYPE, ROTATE, 128, true>(p, page_items, stream)
                    : page_tokens == 64 ? launch_kv_pages<SHIFT_TYPE, ROTATE, 64, false>(p, page_items, stream)
                                        : launch_kv_pages<SHIFT_TYPE, ROTATE, 128, false>(p, page_items, stream);
    if (e != cudaSuccess) return e;
  }
  if (key_pages && !fused) {
    if (mx_key)
      key_page_kernel<SHIFT_TYPE, ROTATE, 128, true><<<grid, 256, 0, stream>>>(p);
    else if (page_tokens == 64)
      key_page_kernel<SHIFT_TYPE, ROTATE, 64, false><<<grid, 256, 0, stream>>>(p);
    else
      key_page_kernel<SHIFT_TYPE, ROTATE, 128, false><<<grid, 256, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  if (value_pages && !fused) {
    cudaError_t e = mx_value           ? launch_value_pages<128, true>(p, page_items, stream)
                    : page_tokens == 64 ? launch_value_pages<64, false>(p, page_items, stream)
                                        : launch_value_pages<128, false>(p, page_items, stream);
    if (e != cudaSuccess) return e;
  }
  if (p.tail_key) {
    const int tail_items = ((p.decode_rows - p.first_row) + (p.rows - p.decode_rows) * (kPage + p.sink_tokens)) *
                           tail_chunks_for(p.heads);
    if (tail_items > 0) {
      tail_token_kernel<SHIFT_TYPE, ROTATE><<<tail_items, 128, 0, stream>>>(p);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
  }
  return cudaSuccess;
}

// ---------------------------------------------------------------------------------------------
// Decode query
// ---------------------------------------------------------------------------------------------

struct QueryParams {
  const __nv_bfloat16* query;
  int64_t row_stride, head_stride;
  const int32_t* row_indices;
  int rows, heads_q, heads_kv;
  ScaleCandidates cand;
  uint8_t* codes[2];
  uint8_t* scales[2];
  __nv_bfloat16* padded;
  int query_chunks;
  // tail
  const __nv_bfloat16* new_key;
  const __nv_bfloat16* new_value;
  int64_t new_key_pitch, new_value_pitch;
  __nv_bfloat16* tail_key;
  __nv_bfloat16* tail_value;
  int64_t tail_slot_stride;
  const int32_t* row_to_slot;
  const int32_t* seq_lens;
  const int32_t* seqused_fp4;
  const float* key_shift;
  int sink_tokens;
  float inverse_scale;  // fl32(1 / tensor scale); 1 when there is none
};

// The atom's four E4M3 scale bytes as one word, gathered from its four adjacent lanes.
__device__ __forceinline__ uint32_t gather_scale_word(float scale, int slot) {
  uint32_t word = cvt_e4m3(scale) << (slot * 8);
  word |= __shfl_xor_sync(0xffffffffu, word, 1);
  word |= __shfl_xor_sync(0xffffffffu, word, 2);
  return word;
}

__device__ __forceinline__ void store_query_term(const QueryParams& p, int term, const GroupCodes& q, int row,
                                                 int head, int group, bool active) {
  const bool mx = p.cand.mx_rule != kMxNone;
  uint32_t word;
  if (mx) {
    // the head's four E8M0 bytes sit in its even lanes (one per 32-channel group): gather them
    word = (group & 1) ? 0u : e8m0_byte(q.scale) << ((group >> 1) * 8);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    word |= __shfl_xor_sync(0xffffffffu, word, 4);
  } else {
    word = gather_scale_word(q.scale, group & 3);
  }
  if (!active) return;
  *reinterpret_cast<uint2*>(p.codes[term] + ((int64_t)row * p.heads_q + head) * 64 + group * 8) =
      make_uint2(q.lo, q.hi);
  const int ratio = p.heads_q / p.heads_kv;
  const int packed_row = head % ratio;
  const int kv_head = head / ratio;
  if (mx) {
    // one 512-byte atom per (row, KV head) tile: the storage is [rows][1][Hq][1][32][4][4]
    if (group == 0) {
      uint8_t* tile = p.scales[term] + ((int64_t)row * p.heads_q + kv_head) * 512;
      *reinterpret_cast<uint32_t*>(tile + (packed_row & 31) * 16 + (packed_row >> 5) * 4) = word;
    }
  } else if ((group & 3) == 0) {
    uint8_t* tile = p.scales[term] + ((int64_t)row * p.heads_q + kv_head) * 1024;
    *reinterpret_cast<uint32_t*>(tile + (group >> 2) * 512 + (packed_row & 31) * 16 + (packed_row >> 5) * 4) = word;
  }
}

template <bool ROTATE, bool SECOND, bool TAIL, bool ROTATE_KEY, bool SHIFT_KEY>
__global__ void __launch_bounds__(128) quantize_query_kernel(const QueryParams p) {
  const int row = blockIdx.x;
  const int chunk = blockIdx.y;
  // First the kernels before this one must be over (their results visible): the buffers written
  // here may still be read by the previous decode launch, and whatever starts early behind this
  // kernel reads the cache those kernels may have written. Then the decode launch that follows may
  // bring its CTAs up and request its first cache pages while this kernel runs; it waits for this
  // kernel's end before it reads the query or the tail.
  wait_for_prior_kernels();
  dependents_may_launch();
  if (TAIL && chunk >= p.query_chunks) {
    const int position = p.seq_lens[row] - 1;
    write_tail_token<SHIFT_KEY ? BDFP4_SHIFT_F32 : BDFP4_SHIFT_NONE, ROTATE_KEY>(
        p.new_key, p.new_value, p.new_key_pitch, p.new_value_pitch, p.key_shift, 0, p.tail_key, p.tail_value,
        p.tail_slot_stride, row, p.row_to_slot[row], position, position - p.seqused_fp4[row],
        (chunk - p.query_chunks) * 128 + threadIdx.x, p.heads_kv, p.sink_tokens);
    return;
  }
  const int item = chunk * 128 + threadIdx.x;
  const bool active = item < p.heads_q * kGroupsPerVec;
  const int head = active ? item / kGroupsPerVec : p.heads_q - 1;
  const int group = item % kGroupsPerVec;
  const int source_row = p.row_indices ? p.row_indices[row] : row;
  const __nv_bfloat16* src = p.query + (int64_t)source_row * p.row_stride + (int64_t)head * p.head_stride + group * kGroup;
  float v[16];
  load_bf16x16(src, v);
  if (ROTATE) {
    hadamard_butterflies(v, group);
    const float inverse = (float)0.08838834764831845;
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], inverse);
  }
  if (p.padded && active) {
    store_bf16x16(p.padded + (((int64_t)row * kPage) * p.heads_q + head) * kHeadDim + group * kGroup, v);
  }
  apply_inverse_scale(v, p.inverse_scale);
  const bool mx = p.cand.mx_rule != kMxNone;
  const GroupCodes first = mx ? mx_quantize_pair16(v, p.cand.mx_rule) : quantize_group16(v, p.cand);
  store_query_term(p, 0, first, row, head, group, active);
  if (SECOND) {
    float residual[16];
    group_residual16(v, first, residual);
    const GroupCodes second = mx ? mx_quantize_pair16(residual, p.cand.mx_rule) : quantize_group16(residual, p.cand);
    store_query_term(p, 1, second, row, head, group, active);
  }
}

// Launched with programmatic stream serialization: after a decode launch of this library (which
// signals early) its CTAs are resident by the time that kernel ends; after anything else it starts
// when that kernel has finished, as an ordinary launch would.
template <typename Kernel>
static cudaError_t launch_overlapped(Kernel kernel, dim3 grid, const QueryParams& p, cudaStream_t stream) {
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
  return cudaLaunchKernelEx(&config, kernel, p);
}

template <bool ROTATE, bool SECOND>
static cudaError_t launch_query(const QueryParams& p, dim3 grid, bool tail, bool rotate_key, bool shift_key,
                                cudaStream_t stream) {
  if (!tail) return launch_overlapped(quantize_query_kernel<ROTATE, SECOND, false, false, false>, grid, p, stream);
  if (rotate_key && shift_key)
    return launch_overlapped(quantize_query_kernel<ROTATE, SECOND, true, true, true>, grid, p, stream);
  if (rotate_key) return launch_overlapped(quantize_query_kernel<ROTATE, SECOND, true, true, false>, grid, p, stream);
  if (shift_key) return launch_overlapped(quantize_query_kernel<ROTATE, SECOND, true, false, true>, grid, p, stream);
  return launch_overlapped(quantize_query_kernel<ROTATE, SECOND, true, false, false>, grid, p, stream);
}

}  // namespace bdfp4

using namespace bdfp4;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int bdfp4_kv_write(const bdfp4_kv_write_args* a, void* stream_handle) {
  if (!a) return BDFP4_E_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (a->heads < 1 || a->work_items < 0) return BDFP4_E_ARG;
  const int page_tokens = a->page_tokens == 0 ? kPage : a->page_tokens;
  if (page_tokens != 128 && page_tokens != 64) return BDFP4_E_UNSUPPORTED;
  if (a->key_scale_mode < 0 || a->key_scale_mode > BDFP4_SCALE_MXFP4_SEARCH || a->value_scale_mode < 0 ||
      a->value_scale_mode > BDFP4_SCALE_MXFP4_SEARCH)
    return BDFP4_E_ARG;
  const bool mx_key = a->key_scale_mode >= BDFP4_SCALE_MXFP4_OCP, mx_value = a->value_scale_mode >= BDFP4_SCALE_MXFP4_OCP;
  if ((mx_key || mx_value) && page_tokens != 128) return BDFP4_E_UNSUPPORTED;
  if (a->pages < 0) return BDFP4_E_ARG;
  auto bad_scale = [](float s) { return s != 0.0f && !(s > 0.0f && isfinite(s)); };
  if (bad_scale(a->key_tensor_scale) || bad_scale(a->value_tensor_scale)) return BDFP4_E_ARG;
  const bool per_layer = a->bases != nullptr;
  const bool write_key = a->key && (per_layer || a->key_codes);
  const bool write_value = a->value && (per_layer || a->value_codes);
  const bool write_tail = a->tail_key != nullptr;
  if (!write_key && !write_value && !write_tail) return BDFP4_E_ARG;
  if (per_layer && write_tail) return BDFP4_E_ARG;  // a per-layer writer writes no tail
  if ((a->tail_key == nullptr) != (a->tail_value == nullptr)) return BDFP4_E_ARG;
  if (per_layer && a->layers < 1) return BDFP4_E_ARG;
  if (a->key && (!aligned16(a->key) || a->key_token_pitch % 8)) return BDFP4_E_ARG;
  if (a->value && (!aligned16(a->value) || a->value_token_pitch % 8)) return BDFP4_E_ARG;
  if (write_tail && (!a->key || !a->value)) return BDFP4_E_ARG;
  if (!per_layer) {
    if (write_key && (!a->key_scales || !aligned16(a->key_codes) || !aligned16(a->key_scales) ||
                      a->key_codes_pitch % 16 || a->key_scales_pitch % 16))
      return BDFP4_E_ARG;
    if (write_value && (!a->value_scales || !aligned16(a->value_codes) || !aligned16(a->value_scales) ||
                        a->value_codes_pitch % 16 || a->value_scales_pitch % 16))
      return BDFP4_E_ARG;
  } else {
    if (a->key_codes_pitch % 16 || a->key_scales_pitch % 16 || a->value_codes_pitch % 16 ||
        a->value_scales_pitch % 16)
      return BDFP4_E_ARG;
  }
  if ((write_key || write_value) && a->work_items > 0 && (!a->source_tokens || !a->destination_pages))
    return BDFP4_E_ARG;
  if (a->key_shift_type < 0 || a->key_shift_type > 2) return BDFP4_E_ARG;
  if ((a->key_shift != nullptr) != (a->key_shift_type != BDFP4_SHIFT_NONE)) return BDFP4_E_ARG;
  if ((a->key_shift || a->rotate_key) && !a->key) return BDFP4_E_ARG;
  const int layers = per_layer ? a->layers : 1;
  if (per_layer && a->source_tokens_total % layers) return BDFP4_E_ARG;
  if (write_tail) {
    if (a->sink_tokens < 0 || a->sink_tokens > BDFP4_MAX_SINK) return BDFP4_E_ARG;
    if (a->rows > 0 && (!a->query_start_loc || !a->seq_lens || !a->seqused_fp4 || !a->row_to_slot))
      return BDFP4_E_ARG;
    if (a->rows < 0 || a->decode_rows < 0 || a->decode_rows > a->rows || a->first_row < 0 ||
        a->first_row > a->decode_rows)
      return BDFP4_E_ARG;
  }

  KvWriteParams p{};
  p.key = static_cast<const __nv_bfloat16*>(a->key);
  p.value = static_cast<const __nv_bfloat16*>(a->value);
  p.key_pitch = a->key_token_pitch;
  p.value_pitch = a->value_token_pitch;
  p.source_layer_stride = per_layer ? a->source_tokens_total / layers : 0;
  p.heads = a->heads;
  p.region[0] = write_key ? static_cast<uint8_t*>(a->key_codes) : nullptr;
  p.region[1] = static_cast<uint8_t*>(a->key_scales);
  p.region[2] = write_value ? static_cast<uint8_t*>(a->value_codes) : nullptr;
  p.region[3] = static_cast<uint8_t*>(a->value_scales);
  p.pitch[0] = a->key_codes_pitch;
  p.pitch[1] = a->key_scales_pitch;
  p.pitch[2] = a->value_codes_pitch;
  p.pitch[3] = a->value_scales_pitch;
  p.bases = a->bases;
  p.layers = layers;
  p.source_tokens = a->source_tokens;
  p.destination_pages = a->destination_pages;
  p.work_items = a->work_items;
  p.key_cand = scale_candidates(a->key_scale_mode);
  p.value_cand = scale_candidates(a->value_scale_mode);
  p.key_shift = a->key_shift;
  p.layer = a->layer;
  p.tail_key = static_cast<__nv_bfloat16*>(a->tail_key);
  p.tail_value = static_cast<__nv_bfloat16*>(a->tail_value);
  p.tail_layer_stride = a->tail_layer_stride;
  p.tail_slot_stride = a->tail_slot_stride;
  p.sink_tokens = a->sink_tokens;
  p.query_start_loc = a->query_start_loc;
  p.seq_lens = a->seq_lens;
  p.seqused_fp4 = a->seqused_fp4;
  p.row_to_slot = a->row_to_slot;
  p.rows = a->rows;
  p.decode_rows = a->decode_rows;
  p.first_row = a->first_row;
  p.pages = a->pages;
  p.error_word = a->error_word;
  p.key_inverse_scale = a->key_tensor_scale == 0.0f ? 1.0f : 1.0f / a->key_tensor_scale;
  p.value_inverse_scale = a->value_tensor_scale == 0.0f ? 1.0f : 1.0f / a->value_tensor_scale;
  if (!write_key) p.key = write_tail ? p.key : nullptr;
  if (!write_value) p.value = write_tail ? p.value : nullptr;

  cudaError_t e;
  const bool rot = a->rotate_key != 0;
  switch (a->key_shift_type) {
    case BDFP4_SHIFT_F32:
      e = rot ? launch_kv_write<BDFP4_SHIFT_F32, true>(p, page_tokens, stream)
              : launch_kv_write<BDFP4_SHIFT_F32, false>(p, page_tokens, stream);
      break;
    case BDFP4_SHIFT_BF16:
      e = rot ? launch_kv_write<BDFP4_SHIFT_BF16, true>(p, page_tokens, stream)
              : launch_kv_write<BDFP4_SHIFT_BF16, false>(p, page_tokens, stream);
      break;
    default:
      e = rot ? launch_kv_write<BDFP4_SHIFT_NONE, true>(p, page_tokens, stream)
              : launch_kv_write<BDFP4_SHIFT_NONE, false>(p, page_tokens, stream);
  }
  return bdfp4::cuda_status(e);
}

extern "C" int bdfp4_quantize_query(const bdfp4_quantize_query_args* a, void* stream_handle) {
  if (!a) return BDFP4_E_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (a->rows < 1 || a->heads_q < 1 || a->heads_kv < 1 || a->heads_q % a->heads_kv) return BDFP4_E_ARG;
  if (a->scale_mode < 0 || a->scale_mode > BDFP4_SCALE_MXFP4_SEARCH) return BDFP4_E_ARG;
  if (a->tensor_scale != 0.0f && !(a->tensor_scale > 0.0f && isfinite(a->tensor_scale))) return BDFP4_E_ARG;
  if (!a->query || !aligned16(a->query) || a->query_row_stride % 8 || a->query_head_stride % 8) return BDFP4_E_ARG;
  if (!a->query_codes || !a->query_scales || !aligned16(a->query_codes) || !aligned16(a->query_scales))
    return BDFP4_E_ARG;
  if ((a->query_codes_second == nullptr) != (a->query_scales_second == nullptr)) return BDFP4_E_ARG;
  if (a->query_padded && !aligned16(a->query_padded)) return BDFP4_E_ARG;
  const bool tail = a->tail_key != nullptr;
  if (tail) {
    if (!a->tail_value || !a->new_key || !a->new_value || !a->row_to_slot || !a->seq_lens || !a->seqused_fp4)
      return BDFP4_E_ARG;
    if (!aligned16(a->new_key) || !aligned16(a->new_value) || a->new_key_token_pitch % 8 ||
        a->new_value_token_pitch % 8)
      return BDFP4_E_ARG;
    if (a->sink_tokens < 0 || a->sink_tokens > BDFP4_MAX_SINK) return BDFP4_E_ARG;
  }
  QueryParams p{};
  p.query = static_cast<const __nv_bfloat16*>(a->query);
  p.row_stride = a->query_row_stride;
  p.head_stride = a->query_head_stride;
  p.row_indices = a->row_indices;
  p.rows = a->rows;
  p.heads_q = a->heads_q;
  p.heads_kv = a->heads_kv;
  p.cand = scale_candidates(a->scale_mode);
  p.codes[0] = static_cast<uint8_t*>(a->query_codes);
  p.scales[0] = static_cast<uint8_t*>(a->query_scales);
  p.codes[1] = static_cast<uint8_t*>(a->query_codes_second);
  p.scales[1] = static_cast<uint8_t*>(a->query_scales_second);
  p.padded = static_cast<__nv_bfloat16*>(a->query_padded);
  p.query_chunks = (a->heads_q * kGroupsPerVec + 127) / 128;
  p.new_key = static_cast<const __nv_bfloat16*>(a->new_key);
  p.new_value = static_cast<const __nv_bfloat16*>(a->new_value);
  p.new_key_pitch = a->new_key_token_pitch;
  p.new_value_pitch = a->new_value_token_pitch;
  p.tail_key = static_cast<__nv_bfloat16*>(a->tail_key);
  p.tail_value = static_cast<__nv_bfloat16*>(a->tail_value);
  p.tail_slot_stride = a->tail_slot_stride;
  p.row_to_slot = a->row_to_slot;
  p.seq_lens = a->seq_lens;
  p.seqused_fp4 = a->seqused_fp4;
  p.key_shift = a->key_shift;
  p.sink_tokens = a->sink_tokens;
  p.inverse_scale = a->tensor_scale == 0.0f ? 1.0f : 1.0f / a->tensor_scale;
  const int tail_chunks = tail ? tail_chunks_for(a->heads_kv) : 0;
  const dim3 grid(a->rows, p.query_chunks + tail_chunks, 1);
  const bool second = a->query_codes_second != nullptr;
  const bool rotate = a->rotate != 0;
  cudaError_t e;
  if (rotate && second)
    e = launch_query<true, true>(p, grid, tail, a->rotate_key != 0, a->key_shift != nullptr, stream);
  else if (rotate)
    e = launch_query<true, false>(p, grid, tail, a->rotate_key != 0, a->key_shift != nullptr, stream);
  else if (second)
    e = launch_query<false, true>(p, grid, tail, a->rotate_key != 0, a->key_shift != nullptr, stream);
  else
    e = launch_query<false, false>(p, grid, tail, a->rotate_key != 0, a->key_shift != nullptr, stream);
  return bdfp4::cuda_status(e);
}
