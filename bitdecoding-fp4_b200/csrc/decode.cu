// C ABI of the paged FP4 decode: argument checks, tensor maps, and the choice among the kernel's
// instantiation units (decode_nvfp4_p128.cu, decode_nvfp4_p64.cu, decode_mxfp4.cu). The kernel
// itself is decode_kernel.cuh.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "decode_params.h"
#include "host.h"

namespace bdfp4 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(entry);
  });
  return fn;
}


// ---- tensor maps of a cache, remembered per host thread --------------------------------------------
struct CacheMapKey {
  const void* key_codes;
  const void* value_codes;
  int heads_kv, page_tokens, pages;
  int64_t key_pitch, value_pitch;
  bool operator==(const CacheMapKey& o) const {
    return key_codes == o.key_codes && value_codes == o.value_codes && heads_kv == o.heads_kv &&
           page_tokens == o.page_tokens && pages == o.pages && key_pitch == o.key_pitch && value_pitch == o.value_pitch;
  }
};
struct CacheMapEntry {
  CacheMapKey key;
  CUtensorMap k_map, v_map;
  uint64_t last_use;
};
constexpr int kCacheMapEntries = 8;  // one per layer group of a caller is plenty; least recently used goes

static bool encode_cache_maps(EncodeTiledFn encode, const CacheMapKey& c, CUtensorMap* k_map, CUtensorMap* v_map) {
  {
    // K codes of 128-token pages: [pages][128 tok][H][64 B]; one box = one head of one page, rows of
    // 64 bytes. (64-token pages are fetched with bulk copies; their maps are encoded but unused.)
    const cuuint64_t dims[4] = {64, (cuuint64_t)c.heads_kv, (cuuint64_t)c.page_tokens, (cuuint64_t)c.pages};
    const cuuint64_t strides[3] = {64, (cuuint64_t)c.heads_kv * 64, (cuuint64_t)c.key_pitch};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)c.page_tokens, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    if (encode(k_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(c.key_codes), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  {
    // V codes: [pages][H * 128 ch][page_tokens / 2 B]; the row is the swizzle span
    const cuuint64_t row_bytes = (cuuint64_t)c.page_tokens / 2;
    const cuuint64_t dims[3] = {row_bytes, (cuuint64_t)c.heads_kv * kHeadDim, (cuuint64_t)c.pages};
    const cuuint64_t strides[2] = {row_bytes, (cuuint64_t)c.value_pitch};
    const cuuint32_t box[3] = {(cuuint32_t)row_bytes, kHeadDim, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (encode(v_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(c.value_codes), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               c.page_tokens == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

static bool cached_cache_maps(EncodeTiledFn encode, const void* key_codes, const void* value_codes, int heads_kv,
                              int page_tokens, int pages, int64_t key_pitch, int64_t value_pitch, CUtensorMap* k_map,
                              CUtensorMap* v_map) {
  // A tensor map holds a device address, which means the same thing in every context of the
  // process's unified address space, so the device is not part of the key.
  static thread_local CacheMapEntry entries[kCacheMapEntries];
  static thread_local int used = 0;
  static thread_local uint64_t clock = 0;
  const CacheMapKey key{key_codes, value_codes, heads_kv, page_tokens, pages, key_pitch, value_pitch};
  ++clock;
  int victim = 0;
  for (int i = 0; i < used; ++i) {
    if (entries[i].key == key) {
      entries[i].last_use = clock;
      *k_map = entries[i].k_map;
      *v_map = entries[i].v_map;
      return true;
    }
    if (entries[i].last_use < entries[victim].last_use) victim = i;
  }
  if (!encode_cache_maps(encode, key, k_map, v_map)) return false;
  if (used < kCacheMapEntries) victim = used++;
  entries[victim] = CacheMapEntry{key, *k_map, *v_map, clock};
  return true;
}

}  // namespace bdfp4

using namespace bdfp4;

extern "C" int bdfp4_decode(const bdfp4_decode_args* a, void* stream_handle) {
  if (!a) return BDFP4_E_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (a->rows < 1 || a->heads_q < 1 || a->heads_kv < 1 || a->heads_q % a->heads_kv) return BDFP4_E_ARG;
  const int ratio = a->heads_q / a->heads_kv;
  if (ratio > 16) return BDFP4_E_UNSUPPORTED;
  if (!a->query_codes || !a->query_scales) return BDFP4_E_ARG;
  if ((a->query_codes_second == nullptr) != (a->query_scales_second == nullptr)) return BDFP4_E_ARG;
  if (!a->key_codes || !a->key_scales || !a->value_codes || !a->value_scales) return BDFP4_E_ARG;
  if (a->pages < 1 || !a->page_table || !a->seqused_fp4 || a->max_pages_per_row < 0) return BDFP4_E_ARG;
  if (a->page_table_stride < a->max_pages_per_row) return BDFP4_E_ARG;
  auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (misaligned(a->query_codes) || misaligned(a->query_scales) || misaligned(a->key_codes) ||
      misaligned(a->key_scales) || misaligned(a->value_codes) || misaligned(a->value_scales))
    return BDFP4_E_ARG;
  if (a->key_codes_pitch % 16 || a->key_scales_pitch % 16 || a->value_codes_pitch % 16 ||
      a->value_scales_pitch % 16)
    return BDFP4_E_ARG;
  const int page_tokens = a->page_tokens == 0 ? kPage : a->page_tokens;
  if (page_tokens != 128 && page_tokens != 64) return BDFP4_E_UNSUPPORTED;
  if (a->scale_format != BDFP4_FORMAT_NVFP4 && a->scale_format != BDFP4_FORMAT_MXFP4) return BDFP4_E_ARG;
  const bool mx = a->scale_format == BDFP4_FORMAT_MXFP4;
  if (mx && page_tokens != 128) return BDFP4_E_UNSUPPORTED;
  // bytes per (page, head): codes 64 per token (K) or page_tokens / 2 per channel (V); scales 8 per
  // token (NVFP4: one E4M3 byte per 16 values) or 4 (MXFP4: one E8M0 byte per 32)
  const int64_t head_codes = (int64_t)page_tokens * 64, head_scales = (int64_t)page_tokens * (mx ? 4 : 8);
  if (a->key_codes_pitch < a->heads_kv * head_codes || a->value_codes_pitch < a->heads_kv * head_codes ||
      a->key_scales_pitch < a->heads_kv * head_scales || a->value_scales_pitch < a->heads_kv * head_scales)
    return BDFP4_E_ARG;
  const bool tail = a->tail_key != nullptr;
  if (tail) {
    if (!a->tail_value || !a->tail_slot_ids || !a->seqused_residual || !a->query_padded || a->tail_slots < 1)
      return BDFP4_E_ARG;
    if (misaligned(a->tail_key) || misaligned(a->tail_value) || misaligned(a->query_padded)) return BDFP4_E_ARG;
  }
  if (!(a->softmax_scale > 0.0f) || !isfinite(a->softmax_scale)) return BDFP4_E_ARG;
  if (a->p_scale_mode < 0 || a->p_scale_mode > 2) return BDFP4_E_ARG;
  if (a->num_splits < 1 || a->bf16_page_cost < 0) return BDFP4_E_ARG;
  auto bad_scale = [](float s) { return s != 0.0f && !(s > 0.0f && isfinite(s)); };
  if (bad_scale(a->key_tensor_scale) || bad_scale(a->query_tensor_scale) || bad_scale(a->value_tensor_scale))
    return BDFP4_E_ARG;
  const bool own_bf16 = a->num_splits > 1 && a->bf16_split != 0;
  // One part may leave either as BF16 `out` or, when `out` is null, as an FP32 partial with its
  // LSE (a KV-axis shard of a longer sequence whose partials are merged elsewhere).
  const bool writes_out = a->num_splits == 1 && a->out != nullptr;
  if (writes_out) {
    if (a->out_row_stride < (int64_t)a->heads_q * kHeadDim) return BDFP4_E_ARG;
  } else if (!a->partial_out || !a->partial_lse) {
    return BDFP4_E_ARG;
  }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return BDFP4_E_CUDA;

  // The two tensor maps depend only on the cache regions and their geometry, which a serving layer
  // keeps for its whole life: they are encoded once per distinct cache and looked up afterwards.
  CUtensorMap k_map, v_map;
  if (!cached_cache_maps(encode, a->key_codes, a->value_codes, a->heads_kv, page_tokens, a->pages,
                         a->key_codes_pitch, a->value_codes_pitch, &k_map, &v_map))
    return BDFP4_E_ARG;

  DecodeParams p{};
  p.rows = a->rows;
  p.heads_q = a->heads_q;
  p.heads_kv = a->heads_kv;
  p.ratio = ratio;
  p.q_codes[0] = static_cast<const uint8_t*>(a->query_codes);
  p.q_scales[0] = static_cast<const uint8_t*>(a->query_scales);
  p.q_codes[1] = static_cast<const uint8_t*>(a->query_codes_second);
  p.q_scales[1] = static_cast<const uint8_t*>(a->query_scales_second);
  p.q_padded = static_cast<const __nv_bfloat16*>(a->query_padded);
  p.k_scales = static_cast<const uint8_t*>(a->key_scales);
  p.v_scales = static_cast<const uint8_t*>(a->value_scales);
  p.k_scales_pitch = a->key_scales_pitch;
  p.v_scales_pitch = a->value_scales_pitch;
  p.k_codes = static_cast<const uint8_t*>(a->key_codes);
  p.v_codes = static_cast<const uint8_t*>(a->value_codes);
  p.k_codes_pitch = a->key_codes_pitch;
  p.v_codes_pitch = a->value_codes_pitch;
  p.pages = a->pages;
  p.page_table = a->page_table;
  p.page_table_stride = a->page_table_stride;
  p.max_pages = a->max_pages_per_row;
  p.seqused_fp4 = a->seqused_fp4;
  p.tail_key = static_cast<const __nv_bfloat16*>(a->tail_key);
  p.tail_value = static_cast<const __nv_bfloat16*>(a->tail_value);
  p.tail_slot_stride = a->tail_slot_stride;
  p.tail_slots = a->tail_slots;
  p.tail_slot_ids = a->tail_slot_ids;
  p.seqused_residual = a->seqused_residual;
  p.seqused_sink = tail ? a->seqused_sink : nullptr;
  const float score_scale = (a->key_tensor_scale == 0.0f ? 1.0f : a->key_tensor_scale) *
                            (a->query_tensor_scale == 0.0f ? 1.0f : a->query_tensor_scale);
  const float value_scale = a->value_tensor_scale == 0.0f ? 1.0f : a->value_tensor_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f * score_scale;
  p.bf16_score_scale = 1.0f / score_scale;
  p.bf16_value_scale = 1.0f / value_scale;
  p.out_scale = value_scale;
  p.p_mode = mx ? (int)BDFP4_P_AMAX6 : a->p_scale_mode;  // MXFP4 has one probability rule and no c8 shift
  p.tau = a->p_scale_tau;
  p.out = writes_out ? static_cast<__nv_bfloat16*>(a->out) : nullptr;
  p.out_row_stride = a->out_row_stride;
  p.num_splits = a->num_splits;
  p.bf16_split = own_bf16 ? 1 : 0;
  p.bf16_page_cost = a->bf16_page_cost;
  p.parts = a->num_splits + (own_bf16 ? 1 : 0);
  p.partial_out = a->partial_out;
  p.partial_lse = a->partial_lse;
  p.error_word = a->error_word;
  // With a counter array and an output, a split launch merges its own partials.
  const bool merges = !writes_out && a->merge_counters != nullptr && a->out != nullptr;
  if (merges && a->out_row_stride < (int64_t)a->heads_q * kHeadDim) return BDFP4_E_ARG;
  p.merge_counters = merges ? a->merge_counters : nullptr;
  p.merged_out = merges ? static_cast<__nv_bfloat16*>(a->out) : nullptr;
  p.row_order = a->row_order;
  p.row_splits = (a->num_splits > 1 && a->merge_counters == nullptr) ? a->row_splits : nullptr;

  const bool two = a->query_codes_second != nullptr;
  cudaError_t e;
  if (mx)
    e = launch_decode_mxfp4(two, k_map, v_map, p, stream);
  else if (page_tokens == 128)
    e = launch_decode_nvfp4_p128(two, k_map, v_map, p, stream);
  else
    e = launch_decode_nvfp4_p64(two, k_map, v_map, p, stream);
  return bdfp4::cuda_status(e);
}

// ---- split decode without caller-provided scratch ----------------------------------------------
//
// Some callers of this library are not allowed to allocate device memory at the point where they
// decode: an engine that has handed all of its HBM budget to the KV cache and runs with allocation
// disabled, a plugin that is entered from inside a host framework's memory-pool critical section,
// or an embedding without access to the framework's allocator at all. The split path of
// bdfp4_decode needs a place for its FP32 partial outputs and log-sum-exps; here that place is a
// fixed array inside the library's own device image, so the call allocates nothing.
namespace bdfp4 {

constexpr size_t kStaticScratchFloats = BDFP4_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_split_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_split_scratch_address[kMaxDevices] = {};
static std::mutex g_split_scratch_mutex;

// The device address of g_split_scratch on the current device. In host code the array's name is
// only a handle for the runtime, never an address a kernel may be given, so the address is looked
// up once per device (with that device current) and remembered.
static cudaError_t split_scratch_address(float** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_split_scratch_mutex);
  if (!g_split_scratch_address[device]) {
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_split_scratch);
    if (e != cudaSuccess) return e;
    g_split_scratch_address[device] = address;
  }
  *out = g_split_scratch_address[device];
  return cudaSuccess;
}

}  // namespace bdfp4

extern "C" int bdfp4_decode_split_static(const bdfp4_decode_args* a, void* stream) {
  if (!a) return BDFP4_E_ARG;
  if (a->num_splits < 2 || a->rows < 1 || a->heads_q < 1 || !a->out) return BDFP4_E_ARG;
  if (a->out_row_stride < (int64_t)a->heads_q * kHeadDim) return BDFP4_E_ARG;
  bdfp4_decode_args local = *a;
  local.merge_counters = nullptr;  // the merge below is the only one: no fused merge on top of it
  // An extra part for the BF16 blocks exists only when there are BF16 blocks: a part that nothing
  // writes would leave the previous call's log-sum-exp in the shared array.
  local.bf16_split = (a->bf16_split != 0 && a->tail_key != nullptr) ? 1 : 0;
  const int64_t parts = (int64_t)a->num_splits + local.bf16_split;
  const int64_t lse_floats = parts * a->rows * a->heads_q;
  const int64_t out_floats = lse_floats * kHeadDim;
  if (out_floats + lse_floats > (int64_t)kStaticScratchFloats) return BDFP4_E_TOO_LARGE;
  float* scratch = nullptr;
  cudaError_t e = split_scratch_address(&scratch);
  if (e != cudaSuccess) return bdfp4::cuda_status(e);
  local.partial_out = scratch;
  local.partial_lse = scratch + out_floats;
  const int status = bdfp4_decode(&local, stream);
  if (status != BDFP4_OK) return status;
  return bdfp4_combine(local.partial_out, local.partial_lse, (int32_t)parts, a->rows, a->heads_q, a->out,
                       a->out_row_stride, stream);
}
