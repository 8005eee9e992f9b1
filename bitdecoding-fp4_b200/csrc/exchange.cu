// The exchange step of a KV-sharded decode as ONE kernel over peer memory: fold this rank's split
// partials into its [O | LSE] record, store the record into every rank's exchange region (plain
// stores through NVLink into memory the peers exported), flag it, wait for the other ranks' records
// to arrive in this GPU's own region, and merge them into the BF16 output. It replaces three steps
// (the fold kernel, an all-gather collective, the merge kernel) and has no counterpart in the
// reference, which has no multi-GPU path.
//
// Region of a rank (all ranks use the same layout; `bdfp4_exchange_bytes` gives its size):
//   records [2 sets][world sources][rows x heads_q slots][132 floats]   O[128], LSE, 3 floats of padding
//   flags   [2 sets][world sources][rows x heads_q slots] u32           the step number of the record in the slot
// A step uses set (step & 1). A rank can be at most one step ahead of another (it cannot finish a
// step without that rank's record of it), so while one set is being read the records of the next
// step land in the other. One CTA per (row, query head) talks only to the CTAs of the same (row,
// head) on the other GPUs: no grid-wide barrier, no CTA waits for a CTA of its own launch.
//
// Ordering: the record's stores are followed by a system-scope fence and a CTA barrier, then one
// thread writes the flag with release semantics at system scope; the reader acquires the flag at
// system scope and reads the records with loads that bypass L1. Every wait is bounded: a record that
// has not arrived after two seconds is left out and BDFP4_DEV_WAIT_TIMEOUT is set in the error word.
//
// Peer memory is touched with ordinary stores only: no bulk or tensor-map copies, no NVLink reductions.
#include "common.cuh"
#include "host.h"
#include "merge.cuh"

namespace bdfp4 {
namespace exchange {

constexpr int kMaxWorld = 8;
constexpr int kSlotFloats = 132;  // 128 output channels, the LSE, padding to 16 bytes
constexpr uint64_t kWaitLimitNs = 2000000000ull;

struct Params {
  const float* partial_out;
  const float* partial_lse;
  int parts, rows, heads_q, world, rank;
  uint32_t step;
  float* regions[kMaxWorld];
  __nv_bfloat16* out;
  int64_t out_row_stride;
  int32_t* error_word;
};

__host__ __device__ inline int64_t records_floats(int world, int slots) { return 2ll * world * slots * kSlotFloats; }

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void store_release_system(uint32_t* address, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* address) {
  uint32_t value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

__global__ void __launch_bounds__(128) exchange_merge_kernel(const Params p) {
  const int head = blockIdx.x;
  const int row = blockIdx.y;
  const int channel = threadIdx.x;
  const int slots = p.rows * p.heads_q;
  const int slot = row * p.heads_q + head;
  const int set = (int)(p.step & 1u);
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ int arrived[kMaxWorld];

  // the split partials come from the decode launch before this one
  wait_for_prior_kernels();
  dependents_may_launch();

  // ---- this rank's record: its parts folded, in part order (the arithmetic of combine_record) ----
  float my_lse;
  const float mine = fold_parts(p.partial_out + (int64_t)slot * kHeadDim + channel, (int64_t)slots * kHeadDim,
                                p.partial_lse + slot, (int64_t)slots, p.parts, channel, &my_lse);

  // ---- into every rank's region (its own included), then the flag ----------------------------------
  const int64_t record_offset = (((int64_t)set * p.world + p.rank) * slots + slot) * kSlotFloats;
  const int64_t flag_offset = ((int64_t)set * p.world + p.rank) * slots + slot;
  for (int r = 0; r < p.world; ++r) {
    float* record = p.regions[r] + record_offset;
    record[channel] = mine;
    if (channel == 0) record[kHeadDim] = my_lse;
  }
  __threadfence_system();
  __syncthreads();
  if (channel < p.world) {
    uint32_t* flags = reinterpret_cast<uint32_t*>(p.regions[channel] + records_floats(p.world, slots));
    store_release_system(flags + flag_offset, p.step);
  }

  // ---- the other ranks' records of this step, as they land in this GPU's region ---------------------
  float* own = p.regions[p.rank];
  const uint32_t* own_flags = reinterpret_cast<const uint32_t*>(own + records_floats(p.world, slots));
  if (channel < p.world) {
    const uint32_t* flag = own_flags + ((int64_t)set * p.world + channel) * slots + slot;
    bool here = load_acquire_system(flag) == p.step;
    if (!here) {
      const uint64_t start = timer_ns();
      uint32_t spins = 0;
      while (!(here = load_acquire_system(flag) == p.step)) {
        if ((++spins & 63u) == 0 && timer_ns() - start > kWaitLimitNs) break;
      }
    }
    arrived[channel] = here ? 1 : 0;
    if (!here && p.error_word) atomicOr(p.error_word, (int)BDFP4_DEV_WAIT_TIMEOUT);
  }
  __syncthreads();

  // ---- merge in rank order (the arithmetic of the split merge); natural-log LSEs -------------------
  const float* records = own + ((int64_t)set * p.world * slots + slot) * kSlotFloats;
  const int64_t source_stride = (int64_t)slots * kSlotFloats;
  float total_max = -INFINITY;
  for (int r = 0; r < p.world; ++r)
    if (arrived[r]) total_max = fmaxf(total_max, __ldcg(records + r * source_stride + kHeadDim));
  if (total_max == -INFINITY) total_max = 0.0f;
  float total_weight = 0.0f;
  for (int r = 0; r < p.world; ++r)
    if (arrived[r]) total_weight += exp2f(__ldcg(records + r * source_stride + kHeadDim) * kLog2e - total_max * kLog2e);
  const float total_inverse = (total_weight == 0.0f || total_weight != total_weight) ? 0.0f : 1.0f / total_weight;
  float acc = 0.0f;
  for (int r = 0; r < p.world; ++r) {
    if (!arrived[r]) continue;
    const float scale = exp2f(__ldcg(records + r * source_stride + kHeadDim) * kLog2e - total_max * kLog2e) * total_inverse;
    if (scale > 0.0f) acc = acc + scale * __ldcg(records + r * source_stride + channel);
  }
  p.out[(int64_t)row * p.out_row_stride + head * kHeadDim + channel] = __float2bfloat16_rn(acc);
}

}  // namespace exchange
}  // namespace bdfp4

using namespace bdfp4;

extern "C" int64_t bdfp4_exchange_bytes(int32_t world, int32_t rows, int32_t heads_q) {
  if (world < 1 || world > exchange::kMaxWorld || rows < 1 || heads_q < 1) return 0;
  const int64_t slots = (int64_t)rows * heads_q;
  return exchange::records_floats(world, (int)slots) * 4 + 2ll * world * slots * 4;
}

// Set-up calls (they allocate and synchronise; never on the decode path).
extern "C" int bdfp4_peer_alloc(int64_t bytes, void** local, void* handle) {
  if (bytes < 1 || !local || !handle) return BDFP4_E_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed around as 64 bytes");
  void* memory = nullptr;
  cudaError_t e = cudaMalloc(&memory, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(memory, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle), memory);
  if (e != cudaSuccess) {
    if (memory) cudaFree(memory);
    return bdfp4::cuda_status(e);
  }
  *local = memory;
  return BDFP4_OK;
}

extern "C" int bdfp4_peer_open(const void* handle, void** mapped) {
  if (!handle || !mapped) return BDFP4_E_ARG;
  cudaIpcMemHandle_t copy;
  memcpy(&copy, handle, sizeof(copy));
  return bdfp4::cuda_status(cudaIpcOpenMemHandle(mapped, copy, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int bdfp4_peer_close(void* mapped) {
  if (!mapped) return BDFP4_E_ARG;
  return bdfp4::cuda_status(cudaIpcCloseMemHandle(mapped));
}

extern "C" int bdfp4_peer_free(void* local) {
  if (!local) return BDFP4_E_ARG;
  return bdfp4::cuda_status(cudaFree(local));
}

extern "C" int bdfp4_exchange_merge(const bdfp4_exchange_args* a, void* stream) {
  if (!a) return BDFP4_E_ARG;
  if (!a->partial_out || !a->partial_lse || !a->out || a->parts < 1 || a->rows < 1 || a->heads_q < 1) return BDFP4_E_ARG;
  if (a->world < 1 || a->world > exchange::kMaxWorld || a->rank < 0 || a->rank >= a->world) return BDFP4_E_ARG;
  if (a->step == 0) return BDFP4_E_ARG;  // a fresh region's flags are zero
  if (a->out_row_stride < (int64_t)a->heads_q * kHeadDim) return BDFP4_E_ARG;
  if ((int64_t)a->rows > 65535) return BDFP4_E_TOO_LARGE;
  exchange::Params p{};
  p.partial_out = a->partial_out;
  p.partial_lse = a->partial_lse;
  p.parts = a->parts;
  p.rows = a->rows;
  p.heads_q = a->heads_q;
  p.world = a->world;
  p.rank = a->rank;
  p.step = a->step;
  for (int r = 0; r < a->world; ++r) {
    if (!a->regions[r] || (reinterpret_cast<uintptr_t>(a->regions[r]) & 15)) return BDFP4_E_ARG;
    p.regions[r] = static_cast<float*>(a->regions[r]);
  }
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.out_row_stride = a->out_row_stride;
  p.error_word = a->error_word;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(a->heads_q, a->rows);
  config.blockDim = dim3(128);
  config.stream = static_cast<cudaStream_t>(stream);
  config.attrs = &attribute;
  config.numAttrs = 1;
  return bdfp4::cuda_status(cudaLaunchKernelEx(&config, exchange::exchange_merge_kernel, p));
}
