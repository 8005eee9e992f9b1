// Thin inline-PTX wrappers for the sm_100a pieces the decode kernel is built from:
// mbarriers with bounded waits, TMA (tiled and plain bulk copies), tensor-memory allocation,
// tcgen05 block-scaled MMA, tcgen05.cp/ld and the shared-memory / instruction descriptors.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bdfp4 {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// ---- a pair of CTAs (a cluster of two) working through each other's shared memory ------------

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// The address, in the cluster's shared window, of `smem_address` as CTA `cta` of the cluster has it.
__device__ __forceinline__ uint32_t cluster_address(uint32_t smem_address, uint32_t cta) {
  uint32_t mapped;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(smem_address), "r"(cta));
  return mapped;
}

__device__ __forceinline__ void cluster_store_b16(uint32_t cluster_addr, uint16_t v) {
  asm volatile("st.shared::cluster.b16 [%0], %1;" ::"r"(cluster_addr), "h"(v) : "memory");
}

__device__ __forceinline__ void cluster_store_b32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void cluster_store_v2(uint32_t cluster_addr, uint32_t x, uint32_t y) {
  asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(cluster_addr), "r"(x), "r"(y) : "memory");
}

// One arrival on an mbarrier of another CTA of the cluster; releases this thread's earlier writes
// (its own shared memory's and the peer's) to whoever acquires the barrier's phase at cluster scope.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void mbar_arrive_release_cluster(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bulk copy from this CTA's shared memory into a peer's (both 16-byte aligned, size a multiple of
// 16); the bytes are counted on an mbarrier of the peer. Source and destination are accessed by the
// async proxy: generic-proxy writes of the source need a proxy fence before the copy is issued.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t peer_dst, const void* src, uint32_t bytes, uint32_t peer_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(peer_dst),
               "r"(smem_u32(src)), "r"(bytes), "r"(peer_bar)
               : "memory");
}

// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait for `parity` of `bar`, giving up after about two seconds or as soon as another thread of
// the CTA has given up (`*abort_flag` != 0). Returns false when it gave up; the caller then
// skips its work and heads for the kernel's common exit, so a lost arrival can never hang the GPU.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t start = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (start == 0) start = now;
      if (now - start > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Generic-proxy shared-memory writes -> visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA ------------------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* global_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(global_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------

// Whole-warp calls. `columns` is a power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld4(uint32_t address, float* v) {
  uint32_t r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(address)
               : "memory");
  v[0] = __uint_as_float(r0);
  v[1] = __uint_as_float(r1);
  v[2] = __uint_as_float(r2);
  v[3] = __uint_as_float(r3);
}

__device__ __forceinline__ void tmem_ld8(uint32_t address, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(address)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld16(uint32_t address, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Sixteen columns of this thread's lane back into tensor memory.
__device__ __forceinline__ void tmem_st16(uint32_t address, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};" ::"r"(address),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}

__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t address, float* v) {
  static_assert(N == 4 || N == 8 || N == 16, "supported tcgen05.ld widths");
  if (N == 4) tmem_ld4(address, v);
  if (N == 8) tmem_ld8(address, v);
  if (N == 16) tmem_ld16(address, v);
}

// ---- descriptors ----------------------------------------------------------------------------

// Shared-memory matrix descriptor (64-bit): start address >> 4 in [0,14), leading byte offset >> 4
// in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), swizzle mode in
// [61,64) (0 none, 2 128B, 4 64B, 6 32B).
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;

__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_address, uint64_t swizzle, uint32_t stride_bytes,
                                              uint32_t leading_bytes) {
  uint64_t d = (uint64_t)((smem_address & 0x3FFFFu) >> 4);
  d |= (uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= swizzle << 61;
  return d;
}

// K-major FP4 operand tile: rows of 64 bytes (128 E2M1 values), 64-byte swizzle, eight-row groups
// 512 bytes apart. `k_step` selects the 64-value slice one MMA consumes (32 bytes).
__device__ __forceinline__ uint64_t fp4_tile_desc(uint32_t smem_address, int k_step) {
  return smem_desc(smem_address + k_step * 32, kSwizzle64B, 512, 16);
}

// K-major FP4 operand tile of 32-byte rows (64 E2M1 values, exactly one MMA's K slice), 32-byte
// swizzle, eight-row groups 256 bytes apart.
__device__ __forceinline__ uint64_t fp4_half_tile_desc(uint32_t smem_address) {
  return smem_desc(smem_address, kSwizzle32B, 256, 16);
}

// K-major BF16 operand tile: rows of 128 bytes (64 values), 128-byte swizzle, eight-row groups
// 1024 bytes apart. `k_step` selects the 16-value slice one kind::f16 MMA consumes (32 bytes).
__device__ __forceinline__ uint64_t bf16_tile_desc(uint32_t smem_address, int k_step) {
  return smem_desc(smem_address + k_step * 32, kSwizzle128B, 1024, 16);
}

// One 512-byte scale-factor atom (32 rows x 16 bytes) as the source of tcgen05.cp 32x128b.
__device__ __forceinline__ uint64_t sf_atom_desc(uint32_t smem_address) {
  return smem_desc(smem_address, kSwizzleNone, 128, 0);
}

// Instruction descriptor of kind::mxf4nvf4 (block-scaled, E2M1 x E2M1, UE4M3 scales, FP32
// accumulate, both operands K-major): a/b format E2M1 = 1 at [7,10)/[10,13), N >> 3 at [17,23),
// scale format 0 at bit 23, M >> 4 at [24,29); scale-factor ids stay 0 because one 32-bit TMEM
// column already holds the four scales a 64-value K slice needs.
__host__ __device__ constexpr uint32_t nvf4_idesc(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Instruction descriptor of kind::mxf4 (E2M1 x E2M1, UE8M0 scales per 32 values, scale_vec::2X): as
// above with the scale format bit 23 set. One 32-bit TMEM column holds a row's scales of two 64-value
// K slices, two bytes each; mxf4_sf_ids names the first byte (0 or 2) the instruction uses for B in
// bits [4,6) and for A in bits [29,31).
__host__ __device__ constexpr uint32_t mxf4_idesc(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t mxf4_sf_ids(int a_id, int b_id) {
  return ((uint32_t)b_id << 4) | ((uint32_t)a_id << 29);
}

// Instruction descriptor of kind::f16 with BF16 operands, FP32 accumulate, both K-major:
// D format F32 = 1 at [4,6), A/B format BF16 = 1 at [7,10)/[10,13), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t bf16_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- tcgen05 issue (one thread) ---------------------------------------------------------------

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Arrive on `bar` once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 rows x 128 bits from shared memory into 4 TMEM columns, replicated to the four lane quarters.
__device__ __forceinline__ void cp_sf_atom(uint32_t tmem_address, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address), "l"(desc) : "memory");
}

}  // namespace tc
}  // namespace bdfp4
