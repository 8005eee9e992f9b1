// Device-side serving metadata: the slot table that maps decode rows to BF16 tail slots, the
// per-step page work table of the quantizer, and the clearing of a new request's tail pages.
// Nothing here reads a length back to the host; every launch shape comes from host integers.
//
// These are CUDA restatements of the reference's Triton kernels
// (src/nvfp4_vllm/control.py:140-370, src/nvfp4_vllm/write.py:28-128 of OpenBitSys/BitDecoding-FP4).
#include "common.cuh"
#include "host.h"

namespace bdfp4 {

constexpr int kFreeKey = -1;
constexpr int kNullBlock = 0;
constexpr int kInactive = -1;
constexpr int kMaxControl = 256;  // rows and slots one CTA can match (the reference supports 128)

struct ControlParams {
  const int32_t* block_table;
  int64_t block_table_stride;
  int block_table_columns;
  const int32_t* seq_lens;
  const int32_t* query_start_loc;
  int32_t* slot_keys;
  int32_t* slot_last_seq;
  int64_t* slot_last_seen;
  int64_t* step;
  int32_t* row_to_slot;
  int32_t* token_to_slot;
  int32_t* seqused_sink;
  int32_t* seqused_fp4;
  int32_t* seqused_residual;
  int32_t* promotion_source_tokens;
  int32_t* promotion_pages;
  int32_t* error_code;
  int num_reqs, num_actual_tokens, num_slots, sink, tail_tokens;
};

// One CTA; thread i owns batch row i and slot i. A row keys on column 0 of its block-table row
// (the physical block holding its first page), which stays fixed for the life of a request. Rows
// that match a slot keep it; the others take the unclaimed slots, least recently seen first.
__global__ void control_kernel(const ControlParams p) {
  __shared__ int s_key[kMaxControl], s_slot_key[kMaxControl], s_slot_seq[kMaxControl];
  __shared__ long long s_slot_seen[kMaxControl];
  __shared__ int s_matched[kMaxControl], s_needs[kMaxControl], s_free[kMaxControl];
  __shared__ int s_free_rank[kMaxControl], s_slot[kMaxControl], s_seq[kMaxControl], s_live[kMaxControl];
  __shared__ int s_q_begin[kMaxControl], s_q_end[kMaxControl];
  __shared__ int s_errors;
  __shared__ long long s_step;
  const int i = threadIdx.x;
  const int n = blockDim.x;
  if (i == 0) {
    s_step = *p.step + 1;
    *p.step = s_step;
    s_errors = 0;
  }
  const bool in_batch = i < p.num_reqs;
  const bool is_slot = i < p.num_slots;
  const int key = in_batch ? p.block_table[(int64_t)i * p.block_table_stride] : kFreeKey;
  const int seq = in_batch ? p.seq_lens[i] : 0;
  const int q_begin = in_batch ? p.query_start_loc[i] : 0;
  const int q_end = in_batch ? p.query_start_loc[i + 1] : 0;
  const int query_len = q_end - q_begin;
  const bool live = in_batch && seq > 0 && key != kNullBlock;
  const int computed = seq - query_len;
  const int slot_key = is_slot ? p.slot_keys[i] : kFreeKey;
  const int slot_last_seq = is_slot ? p.slot_last_seq[i] : -1;
  const long long slot_last_seen = is_slot ? p.slot_last_seen[i] : -1;
  s_key[i] = key;
  s_seq[i] = seq;
  s_live[i] = live;
  s_q_begin[i] = q_begin;
  s_q_end[i] = q_end;
  s_slot_key[i] = slot_key;
  s_slot_seq[i] = slot_last_seq;
  s_slot_seen[i] = slot_last_seen;
  __syncthreads();

  // the lowest slot whose key this live row carries
  int matched = p.num_slots;
  if (live) {
    for (int j = 0; j < p.num_slots; ++j) {
      if (s_slot_key[j] == key) {
        matched = j;
        break;
      }
    }
  }
  const bool has_match = matched < p.num_slots;
  const int matched_last_seq = has_match ? s_slot_seq[matched] : 0;
  s_matched[i] = matched;
  const bool needs_slot = live && !has_match;
  s_needs[i] = needs_slot;
  __syncthreads();

  bool claimed = false;
  int need_rank = -1;
  for (int r = 0; r < n; ++r) {
    if (is_slot && s_matched[r] == i) claimed = true;
    if (r <= i && s_needs[r]) ++need_rank;
  }
  const bool free_slot = is_slot && !claimed;
  s_free[i] = free_slot;
  __syncthreads();
  int free_rank = 0;
  for (int j = 0; j < n; ++j) {
    if (s_free[j] && (s_slot_seen[j] < slot_last_seen || (s_slot_seen[j] == slot_last_seen && j < i))) ++free_rank;
  }
  s_free_rank[i] = free_rank;
  __syncthreads();
  int allocated = 0;
  bool got_slot = false;
  if (needs_slot) {
    for (int j = 0; j < n; ++j) {
      if (s_free[j] && s_free_rank[j] == need_rank) {
        allocated += j;
        got_slot = true;
      }
    }
  }
  int slot = has_match ? matched : allocated;
  if (!live) slot = kInactive;
  s_slot[i] = slot;

  int errors = 0;
  if (live && query_len > 1 && computed > 0) errors |= 1;                       // a prompt split across steps
  if (needs_slot && computed > 0) errors |= 2;                                   // a row with history matched no slot
  if (has_match && matched_last_seq != computed && computed > 0) errors |= 4;    // stale slot history
  if (needs_slot && !got_slot) errors |= 8;                                      // no free slot
  if (live) {
    int same = 0;
    for (int r = 0; r < n; ++r) same += (s_live[r] && s_key[r] == key) ? 1 : 0;
    if (same > 1) errors |= 16;                                                  // two live rows share a block
  }
  __syncthreads();

  // slot state follows its owner (the lowest row that landed on it); unclaimed slots keep theirs
  if (is_slot) {
    int owner = n;
    for (int r = 0; r < n; ++r) {
      if (s_live[r] && s_slot[r] == i) {
        owner = r;
        break;
      }
    }
    if (owner < n) {
      p.slot_keys[i] = s_key[owner];
      p.slot_last_seq[i] = s_seq[owner];
      p.slot_last_seen[i] = s_step;
    }
    p.row_to_slot[i] = slot;
    const int sink = live ? min(seq, p.sink) : 0;
    const int live_seq = live ? seq : 0;
    const int fp4 = live_seq > 0 ? ((live_seq - 1) / kPage) * kPage : 0;
    p.seqused_sink[i] = sink;
    p.seqused_fp4[i] = fp4;
    p.seqused_residual[i] = live_seq - fp4;
    // where promotion would read and write if this step filled the tail
    const int column = fp4 / kPage;
    const bool crossing = live && seq > 0 && seq % kPage == 0;
    const bool in_bounds = column < p.block_table_columns;
    if (crossing && !in_bounds) errors |= 32;
    p.promotion_source_tokens[i] = live ? slot * p.tail_tokens : 0;
    p.promotion_pages[i] =
        (crossing && in_bounds) ? p.block_table[(int64_t)i * p.block_table_stride + column] : kInactive;
  }
  if (errors) atomicOr(&s_errors, errors);
  __syncthreads();
  if (i == 0 && s_errors) atomicOr(p.error_code, s_errors);

  for (int token = i; token < p.num_actual_tokens; token += n) {
    int owner_slot = 0;
    for (int r = 0; r < p.num_reqs; ++r) {
      if (s_live[r] && token >= s_q_begin[r] && token < s_q_end[r]) owner_slot += s_slot[r];
    }
    p.token_to_slot[token] = owner_slot;
  }
}

// For each (row, page column) slot of the quantizer's grid: which tokens to read, which page to
// write. Only a fresh prefill row (more than one token this step, and a slot) contributes pages.
__global__ void work_table_kernel(const int32_t* query_start_loc, const int32_t* seqused_fp4,
                                  const int32_t* row_to_slot, const int32_t* block_table,
                                  int64_t block_table_stride, int32_t* source_tokens, int32_t* destination_pages,
                                  int columns_per_row) {
  const int row = blockIdx.x;
  const int start = query_start_loc[row];
  const int end = query_start_loc[row + 1];
  const int slot = row_to_slot[row];
  const int full_pages = seqused_fp4[row] / kPage;
  const bool row_writes = (end - start > 1) && slot >= 0;
  for (int column = threadIdx.x; column < columns_per_row; column += blockDim.x) {
    const bool active = row_writes && column < full_pages;
    const int out = row * columns_per_row + column;
    source_tokens[out] = start + column * kPage;
    destination_pages[out] = active ? block_table[(int64_t)row * block_table_stride + column] : -1;
  }
}

// Zero every layer's tail page of the rows that start a request this step (sequence no longer than
// what the step brought), so a recycled slot never shows its previous tenant's tokens.
__global__ void tail_reset_kernel(__nv_bfloat16* tail_key, __nv_bfloat16* tail_value, int64_t layer_stride,
                                  int64_t slot_stride, const int32_t* query_start_loc, const int32_t* seq_lens,
                                  const int32_t* row_to_slot, int num_reqs, int64_t page_elems) {
  const int layer = blockIdx.x;
  const int row = blockIdx.y;
  if (row >= num_reqs) return;
  const int slot = row_to_slot[row];
  const int start = query_start_loc[row];
  const int end = query_start_loc[row + 1];
  const int seq_len = seq_lens[row];
  if (slot < 0 || seq_len > end - start) return;
  uint4* k = reinterpret_cast<uint4*>(tail_key + layer * layer_stride + slot * slot_stride);
  uint4* v = reinterpret_cast<uint4*>(tail_value + layer * layer_stride + slot * slot_stride);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int64_t idx = threadIdx.x; idx < page_elems / 8; idx += blockDim.x) {
    k[idx] = zero;
    v[idx] = zero;
  }
}

}  // namespace bdfp4

using namespace bdfp4;

extern "C" int bdfp4_control_step(const bdfp4_control_args* a, void* stream) {
  if (!a) return BDFP4_E_ARG;
  if (a->num_reqs < 0 || a->num_slots < 1 || a->num_slots > kMaxControl || a->num_reqs > kMaxControl)
    return BDFP4_E_ARG;
  if (a->num_actual_tokens < 0 || a->sink_tokens < 0 || a->sink_tokens > BDFP4_MAX_SINK) return BDFP4_E_ARG;
  if (!a->block_table || !a->seq_lens || !a->query_start_loc || !a->slot_keys || !a->slot_last_seq ||
      !a->slot_last_seen || !a->step || !a->row_to_slot || !a->seqused_sink || !a->seqused_fp4 ||
      !a->seqused_residual || !a->promotion_source_tokens || !a->promotion_pages || !a->error_code)
    return BDFP4_E_ARG;
  if (a->num_actual_tokens > 0 && !a->token_to_slot) return BDFP4_E_ARG;
  ControlParams p{};
  p.block_table = a->block_table;
  p.block_table_stride = a->block_table_stride;
  p.block_table_columns = a->block_table_columns;
  p.seq_lens = a->seq_lens;
  p.query_start_loc = a->query_start_loc;
  p.slot_keys = a->slot_keys;
  p.slot_last_seq = a->slot_last_seq;
  p.slot_last_seen = a->slot_last_seen;
  p.step = a->step;
  p.row_to_slot = a->row_to_slot;
  p.token_to_slot = a->token_to_slot;
  p.seqused_sink = a->seqused_sink;
  p.seqused_fp4 = a->seqused_fp4;
  p.seqused_residual = a->seqused_residual;
  p.promotion_source_tokens = a->promotion_source_tokens;
  p.promotion_pages = a->promotion_pages;
  p.error_code = a->error_code;
  p.num_reqs = a->num_reqs;
  p.num_actual_tokens = a->num_actual_tokens;
  p.num_slots = a->num_slots;
  p.sink = a->sink_tokens;
  p.tail_tokens = kPage + a->sink_tokens;
  int threads = 32;
  while (threads < a->num_reqs || threads < a->num_slots) threads *= 2;
  control_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return bdfp4::cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4,
                                const int32_t* row_to_slot, const int32_t* block_table,
                                int64_t block_table_stride, int32_t* source_tokens, int32_t* destination_pages,
                                int32_t num_reqs, int32_t columns_per_row, void* stream) {
  if (num_reqs < 0 || columns_per_row < 0) return BDFP4_E_ARG;
  if (num_reqs == 0 || columns_per_row == 0) return BDFP4_OK;
  if (!query_start_loc || !seqused_fp4 || !row_to_slot || !block_table || !source_tokens || !destination_pages)
    return BDFP4_E_ARG;
  work_table_kernel<<<num_reqs, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      query_start_loc, seqused_fp4, row_to_slot, block_table, block_table_stride, source_tokens, destination_pages,
      columns_per_row);
  return bdfp4::cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_tail_reset(void* tail_key, void* tail_value, int64_t layer_stride, int64_t slot_stride,
                                int32_t layers, int64_t page_elems, const int32_t* query_start_loc,
                                const int32_t* seq_lens, const int32_t* row_to_slot, int32_t num_reqs,
                                void* stream) {
  if (layers < 1 || num_reqs < 0 || page_elems < 8 || page_elems % 8) return BDFP4_E_ARG;
  if (num_reqs == 0) return BDFP4_OK;
  if (!tail_key || !tail_value || !query_start_loc || !seq_lens || !row_to_slot) return BDFP4_E_ARG;
  if ((reinterpret_cast<uintptr_t>(tail_key) | reinterpret_cast<uintptr_t>(tail_value)) & 15) return BDFP4_E_ARG;
  if (layer_stride % 8 || slot_stride % 8) return BDFP4_E_ARG;
  tail_reset_kernel<<<dim3(layers, num_reqs), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(tail_key), static_cast<__nv_bfloat16*>(tail_value), layer_stride, slot_stride,
      query_start_loc, seq_lens, row_to_slot, num_reqs, page_elems);
  return bdfp4::cuda_status(cudaGetLastError());
}
