// MLA latent-cache decode attention for sm_100a, and the writers around it.
//
// A token is a 512-channel latent (cached in NVFP4) plus a 64-channel BF16 rope key; every query
// head attends over the same cache:
//   score[h, t] = q_latent[h] . latent[t] + q_rope[h] . rope[t]       out[h] = sum_t p[h, t] latent[t]
// The latent is cached twice, as four 128-channel pseudo heads of 64-token pages: once with scales
// along channels (the K-side regions of the paged cache) and once with scales along tokens (the
// V-side regions), because a block-scaled MMA wants its scales along the contraction axis.
//
// A pair of CTAs (a cluster of two) serves (row, 128 query heads[, split]) and walks the row's pages
// two at a time (128 tokens per step). The pair shares the step's work both ways:
//   - CTA c scores the step's page c: it alone fetches that page's K-side copy and rope keys, forms
//     S[head, 64 tokens], and turns them into FP4 probabilities;
//   - CTA c accumulates output channels [256 c, 256 c + 256) over all 128 tokens of the step (128
//     heads x 512 FP32 is the whole of an SM's tensor memory), so it needs the other CTA's
//     probabilities too: each CTA forms its half of the step's P operand (the K block of its page)
//     in its own shared memory and sends it, as one bulk copy, into the peer's. (Plain stores into
//     the peer's shared memory followed by the proxy fence the tensor core needs cost about 1 us a
//     step; a bulk copy is written by the async proxy, which the tensor core reads with no fence.)
// Per step and CTA that is half the score products, half the exponentials and half the K-side bytes
// of a CTA that scored the whole step by itself. Query heads are the M rows of every MMA, so a head
// is a lane of tensor memory:
//   S[head, token]  = sum over 4 chunks  Q_chunk[head, :] . K_chunk[token, :]   8 x mxf4nvf4 (N = 64, K = 64)
//                   + q_rope[head, :] . rope[token, :]                           4 x kind::f16  (N = 64, K = 16)
//   O[head, chan]  += P[head, :] . V^T[chan, :]                                  2 x mxf4nvf4 (N = 256, K = 64)
// Each head has four softmax threads per CTA, in two teams that take the steps in turns (team = step
// parity): a thread forms 32 tokens of every other step, the group of sixteen in its own registers
// (no shuffles), and looks at the outcome of EVERY step. A thread reads its scores from tensor
// memory, forms the probabilities against the stale maximum and quantizes them. A warp that saw a
// probability large enough that a maximum may have to move (the stale-maximum rule tolerates 2^8)
// stamps the step's number into a request word that travels with the half. The last warp of a team
// to finish a half sends it (the PV issuer only waits for both halves: the crossing, about 650
// cycles, stays out of its loop). The walk is pipelined by one step: a thread forms step i (if it
// is its team's), then looks at how step i - 1 came out (both halves in place, no request: almost
// always), then announces step i; so the halves cross between the CTAs while the next ones are
// formed. On a requested step the threads that formed it publish their maxima (stores into both
// CTAs' shared memory), all threads of the pair apply the exact rule identically and rescale their
// share of O in place in tensor memory, steps i - 1 and i are formed again by their teams, and the
// PV issuers wait for the second copy. O (256 columns) stays in tensor memory for the whole walk.
// Three P buffers: one being multiplied, one crossing, one being formed.
// Tensor memory: S 2 x 64 (the scores of the next step are formed while this step's are still being
// read) + O 256 + scale factors 112 columns (K scales in two sets, so that the next step's can be
// copied in while this step's are in use).
//
// Warps: 0 issues the bulk copies from global memory (lane 0 the K side of the CTA's page, lane 1 the
// V side of both pages); 1, 2 and 3 issue the tensor work, one thread each for QK, for PV, and for
// the K scale atoms (which the whole of warp 3 first regroups
// from the page's 8-byte rows to the 16-byte rows of an atom); 4-19 are the softmax. Every mbarrier
// wait is bounded and reports its site in bits [8,16) of the error word; a CTA whose peer gave up
// runs into its own limit and gives up too.
#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "host.h"
#include "tcgen05.cuh"

namespace bdfp4 {
namespace mla {

constexpr int kHeads = 128;   // query heads per CTA pair: M of every MMA
constexpr int kChunks = 4;    // 128-channel chunks of the latent
constexpr int kLatent = 512;
constexpr int kHalf = 256;    // output channels per CTA
constexpr int kRope = 64;
constexpr int kStep = 128;    // tokens per step (two 64-token pages)
constexpr int kOwn = 64;      // tokens of a step one CTA scores (its page)
constexpr int kStages = 3;   // K side (the CTA's page of a step)
constexpr int kVStages = 2;  // V side (both pages of a step)
constexpr int kPBuffers = 3;  // P operands: one being multiplied, one under way between the CTAs, one being formed
constexpr int kSoftmaxGroups = 4;                   // softmax threads per head in a CTA
constexpr int kTeams = 2;                           // the softmax warps take the steps in turns: team = step % kTeams
constexpr int kTeamGroups = kSoftmaxGroups / kTeams;  // softmax threads per head that form a given step
constexpr int kRun = kOwn / kTeamGroups;            // tokens of a step one of them owns
constexpr int kRunGroups = kRun / 16;
constexpr int kShare = kHalf / kSoftmaxGroups;      // output columns one softmax thread rescales and writes
constexpr int kSoftmaxThreads = 128 * kSoftmaxGroups;
constexpr int kSoftmaxWarps = kSoftmaxThreads / 32;
constexpr int kTeamWarps = kSoftmaxWarps / kTeams;
constexpr int kSlots = 2 * kSoftmaxGroups;          // softmax threads per head in the pair
constexpr int kStepSlots = 2 * kTeamGroups;         // ... of which these form a given step
constexpr int kThreads = 128 + kSoftmaxThreads;  // producer, QK, PV and K-scale warps, then the softmax warps
constexpr float kRescaleThreshold = 8.0f;

constexpr int kColS = 0;       // two buffers of 64 columns
constexpr int kColO = 128;     // 256 columns
constexpr int kColSFQ = 384;   // 8 atoms x 4
constexpr int kColSFK = 416;   // 2 buffers x 4 atoms x 4 (an atom: a chunk's two K blocks, two columns each)
constexpr int kColSFV = 448;   // 2 buffers x 2 pages x 2 atoms x 4
constexpr int kColSFP = 480;   // 2 buffers x 2 atoms x 4
constexpr int kTmemColumns = 512;

constexpr uint32_t kKeyBytes = kChunks * 4096 + 8192;      // one page: codes of four chunks + its rope block
constexpr uint32_t kKeyScaleBytes = 2048;
constexpr uint32_t kValueBytes = 2 * (8192 + 1024);        // this CTA's two chunks of two pages

struct Params {
  int rows, heads_q, head_blocks;
  const uint8_t* q_codes;
  const uint8_t* q_scales;
  const __nv_bfloat16* q_rope;
  const uint8_t* k_codes;
  const uint8_t* k_scales;
  const uint8_t* v_codes;
  const uint8_t* v_scales;
  const uint8_t* rope;
  int64_t k_codes_pitch, k_scales_pitch, v_codes_pitch, v_scales_pitch, rope_pitch;
  int pages;
  const int32_t* page_table;
  int64_t page_table_stride;
  const int32_t* seq_lens;
  float scale_log2;
  int p_mode;
  float tau;
  __nv_bfloat16* out;
  int num_splits;
  float* partial_out;
  float* partial_lse;
  int32_t* error_word;
};

// One CTA's contribution to a step's P operand: the K block (64 tokens) of the page it scored. It
// forms it in its own copy and sends that, as one bulk copy, into the peer's.
struct alignas(1024) PHalf {
  uint8_t codes[kHeads * 32];  // 128 heads x 32 B, 32 B swizzle
  uint8_t sf[512];             // the K block's scale atom
  int examine;                 // step number + 1 of the last step on which the forming CTA asked for the examination
  int pad[3];
};
constexpr uint32_t kPHalfBytes = kHeads * 32 + 512 + 16;

struct Smem {
  alignas(1024) uint8_t k_codes[kStages][kChunks][4096];  // [chunk][64 tokens x 64 B], 64 B swizzle
  alignas(1024) uint8_t rope[kStages][8192];              // 64 tokens x 128 B, 128 B swizzle
  alignas(1024) uint8_t v_codes[kVStages][2][8192];        // [page][256 ch x 32 B], 32 B swizzle
  alignas(1024) uint8_t k_sf[kStages][2048];              // the page's block, regrouped in place into 4 atoms
  alignas(1024) uint8_t v_sf[kVStages][2][1024];           // [page][2 atoms]
  alignas(1024) uint8_t q_tile[kChunks][kHeads * 64];
  alignas(1024) uint8_t q_rope[kHeads * 128];
  alignas(1024) uint8_t q_sf[kChunks * 2][512];
  PHalf p[kPBuffers][2];                                        // [buffer][page = the CTA that forms it]
  float red[2][kStepSlots][kHeads];  // maxima exchanged between the threads of the pair that formed a step
  float sums[kSlots][kHeads];     // their partial sums, at the end
  uint64_t k_full[kStages], ksf_full[kStages], k_empty[kStages], v_full[kVStages], v_empty[kVStages];
  uint64_t s_full[2], s_empty[2], sfk_ready[2];
  uint64_t o_done[2];  // PV products of even and of odd steps: the walk looks at them up to two steps late
  uint64_t p_local[kPBuffers];   // every softmax warp of this CTA has formed its part of the step's P half
  uint64_t p_remote[kPBuffers];  // the peer's P half of the step has landed here
  uint64_t again_local, again_remote;  // the same, after a step on which the maxima were examined
  uint64_t exchange;     // every softmax warp of the pair has stored its maxima (if it formed the step) or its sums
  int formed[kPBuffers], formed_again;  // softmax warps that have finished a half: the last one sends it
  int page_ids[2][32];
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(Smem) + 1024 <= 232448, "one CTA's shared memory (227 KB opt-in limit)");

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A bounded wait that leaves its own number in the abort flag when it is the one that ran out of
// time; the kernel reports it in bits [8,16) of the error word, so a lost arrival can be located.
// CLUSTER: the barrier also takes arrivals from the peer CTA, whose writes the wait must acquire.
template <bool CLUSTER = false>
__device__ __forceinline__ bool wait_at(int site, uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  auto done = [&]() { return CLUSTER ? tc::mbar_try_wait_cluster(bar, parity) : tc::mbar_try_wait(bar, parity); };
  if (done()) return true;
  uint64_t start = 0;
  uint32_t spins = 0;
  while (true) {
    if (done()) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = tc::global_timer_ns();
      if (start == 0) start = now;
      if (now - start > tc::kWaitLimitNs) {
        atomicCAS(const_cast<int*>(abort_flag), 0, site);
        return false;
      }
    }
  }
}

__device__ __forceinline__ int swizzle64(int offset) { return offset ^ (((offset >> 7) & 3) << 4); }

// Scale of one group of sixteen probabilities from its maximum (the rule of the GQA kernel).
__device__ __forceinline__ float probability_scale(float maximum, int p_mode, float tau) {
  float scale = __fmul_rn(maximum, (float)(1.0 / 6.0));
  if (p_mode != BDFP4_P_AMAX6 && maximum <= tau) scale = __fmul_rn(maximum, 0.5f);
  return scale;
}

__global__ void __launch_bounds__(kThreads, 1) decode_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic window starts at the same offset in both CTAs, so the aligned struct does too
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which work ---------------------------------------------------------------------------
  const int cta = (int)tc::cluster_cta_rank();  // 0 or 1: the page of every step it scores, the output half it owns
  const int pair = blockIdx.x >> 1;
  const int head_block = pair % p.head_blocks;
  const int row = (pair / p.head_blocks) % p.rows;
  const int part = pair / (p.head_blocks * p.rows);
  const int head0 = head_block * kHeads;
  const int valid_heads = min(kHeads, p.heads_q - head0);
  // a length the row's page-table entries cannot cover is cut to what they cover
  const int64_t covered = p.page_table_stride * 64;
  const int seq_len = (int)min((int64_t)max(p.seq_lens[row], 0), covered);
  const int entries = (seq_len + 63) / 64;
  const int total_steps = (seq_len + kStep - 1) / kStep;
  const int chunk = (total_steps + p.num_splits - 1) / p.num_splits;
  const int first_step = min(part * chunk, total_steps);
  const int last_step = min(first_step + chunk, total_steps);
  const int num_steps = last_step - first_step;

  // this CTA's shared memory as the peer sees its own: same layout, another window of the cluster
  const uint32_t local_base = tc::smem_u32(&sm);
  const uint32_t peer_base = tc::cluster_address(local_base, (uint32_t)(cta ^ 1));
  auto in_peer = [&](const void* mine) { return tc::smem_u32(mine) - local_base + peer_base; };

  // ---- set-up -------------------------------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&sm.k_full[s], 1);
      tc::mbar_init(&sm.ksf_full[s], 1);
      tc::mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      tc::mbar_init(&sm.v_full[s], 1);
      tc::mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&sm.s_full[b], 1);
      tc::mbar_init(&sm.s_empty[b], kTeamWarps);  // one arrival per softmax warp of the step's team
    }
    tc::mbar_init(&sm.o_done[0], 1);
    tc::mbar_init(&sm.o_done[1], 1);
    tc::mbar_init(&sm.sfk_ready[0], 1);
    tc::mbar_init(&sm.sfk_ready[1], 1);
    for (int b = 0; b < kPBuffers; ++b) {
      tc::mbar_init(&sm.p_local[b], kTeamWarps);
      tc::mbar_init(&sm.p_remote[b], 1);
      sm.p[b][0].examine = sm.p[b][1].examine = 0;
      sm.formed[b] = 0;
    }
    tc::mbar_init(&sm.again_local, kTeamWarps);
    sm.formed_again = 0;
    tc::mbar_init(&sm.again_remote, 1);
    tc::mbar_init(&sm.exchange, 2 * kSoftmaxWarps);
    sm.abort_flag = 0;
    tc::fence_barrier_init();
  }
  // Everything up to here reads only the batch's metadata. The query operands come from the launch
  // before this one (the query quantizer): with programmatic dependent launch this kernel may have
  // started while that one was still running, so wait for it here, then let the launch after this
  // one (the merge, or the next step's quantizer) start its own preamble.
  wait_for_prior_kernels();
  dependents_may_launch();
  // query operands: codes (16 chunks of 16 bytes per head), scales (8 words per head), rope (8
  // chunks); rows past the last head stay zero
  {
    const int64_t head_base = (int64_t)row * p.heads_q + head0;
    for (int i = tid; i < kHeads * 16; i += kThreads) {
      const int h = i >> 4, c = i & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h < valid_heads) v = __ldg(reinterpret_cast<const uint4*>(p.q_codes + (head_base + h) * 256) + c);
      *reinterpret_cast<uint4*>(sm.q_tile[c >> 2] + swizzle64(h * 64 + (c & 3) * 16)) = v;
    }
    for (int i = tid; i < kHeads * 8; i += kThreads) {
      const int h = i >> 3, a = i & 7;
      uint32_t v = 0;
      if (h < valid_heads) v = __ldg(reinterpret_cast<const uint32_t*>(p.q_scales + (head_base + h) * 32) + a);
      *reinterpret_cast<uint32_t*>(sm.q_sf[a] + (h & 31) * 16 + (h >> 5) * 4) = v;
    }
    for (int i = tid; i < kHeads * 8; i += kThreads) {
      const int h = i >> 3, c = i & 7;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h < valid_heads) v = __ldg(reinterpret_cast<const uint4*>(p.q_rope + (head_base + h) * kRope) + c);
      *reinterpret_cast<uint4*>(sm.q_rope + h * 128 + ((c ^ (h & 7)) << 4)) = v;
    }
  }
  if (warp == 1) {
    tc::tmem_alloc(&sm.tmem_base, kTmemColumns);
    tc::tmem_relinquish();
  }
  tc::fence_proxy_async_smem();
  tc::fence_before_sync();
  // both CTAs: the peer's barriers exist before anything is stored into its shared memory
  tc::cluster_sync_all();
  tc::fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;

  auto page_of = [&](int i, int which) {  // page of the i-th step this pair walks (newest first)
    const int step = last_step - 1 - i;
    int entry = 2 * step + which;
    if (entry >= entries) entry = 2 * step;  // an odd page count: the second half is masked anyway
    int page = p.page_table[(int64_t)row * p.page_table_stride + entry];
    if (page < 0 || page >= p.pages) {
      if (p.error_word) atomicOr(p.error_word, (int)BDFP4_DEV_BAD_PAGE);
      page = min(max(page, 0), p.pages - 1);
    }
    return page;
  };

  if (warp == 0) {
    // ---- copy producer ----------------------------------------------------------------------
    int issued = 0;
    bool ok = true;
    for (int base = 0; base < num_steps && ok; base += 32) {
      const int count = min(32, num_steps - base);
      if (lane < count) {
        sm.page_ids[0][lane] = page_of(base + lane, 0);
        sm.page_ids[1][lane] = page_of(base + lane, 1);
      }
      __syncwarp();
      if (lane < 2) {
        for (int j = 0; j < count && ok; ++j) {
          const int i = base + j;
          const int page[2] = {sm.page_ids[0][j], sm.page_ids[1][j]};
          if (lane == 0) {
            const int s = i % kStages;
            ok = wait_at(1, &sm.k_empty[s], ((i / kStages) & 1) ^ 1, abort_flag);
            if (ok) {
              const int64_t mine = page[cta];
              tc::mbar_expect_tx(&sm.ksf_full[s], kKeyScaleBytes);
              tc::mbar_expect_tx(&sm.k_full[s], kKeyBytes);
              tc::bulk_load(sm.k_sf[s], p.k_scales + mine * p.k_scales_pitch, kKeyScaleBytes, &sm.ksf_full[s]);
#pragma unroll
              for (int c = 0; c < kChunks; ++c)
                tc::bulk_load(sm.k_codes[s][c], p.k_codes + mine * p.k_codes_pitch + c * 4096, 4096, &sm.k_full[s]);
              tc::bulk_load(sm.rope[s], p.rope + mine * p.rope_pitch, 8192, &sm.k_full[s]);
            }
          } else {
            const int s = i % kVStages;
            ok = wait_at(2, &sm.v_empty[s], ((i / kVStages) & 1) ^ 1, abort_flag);
            if (ok) {
              tc::mbar_expect_tx(&sm.v_full[s], kValueBytes);
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                tc::bulk_load(sm.v_codes[s][e], p.v_codes + (int64_t)page[e] * p.v_codes_pitch + cta * 8192, 8192,
                              &sm.v_full[s]);
                tc::bulk_load(sm.v_sf[s][e], p.v_scales + (int64_t)page[e] * p.v_scales_pitch + cta * 1024, 1024,
                              &sm.v_full[s]);
              }
            }
          }
          if (ok) issued = i + 1;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    // After a give-up, wait (bounded) until every copy already in flight has landed, so that no
    // bulk copy can write into this CTA's shared memory after it exits.
    if (lane < 2 && *abort_flag) {
      const uint64_t start = tc::global_timer_ns();
      const int depth = lane == 0 ? kStages : kVStages;
      for (int i = max(0, issued - depth); i < issued; ++i) {
        const int s = i % depth;
        const uint32_t parity = (i / depth) & 1;
        if (lane == 0) {
          while (!tc::mbar_try_wait(&sm.k_full[s], parity) && tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
          while (!tc::mbar_try_wait(&sm.ksf_full[s], parity) && tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
        } else {
          while (!tc::mbar_try_wait(&sm.v_full[s], parity) && tc::global_timer_ns() - start < tc::kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- score products: one thread ---------------------------------------------------------------
    // Issuing is what bounds the tensor side of a step (a tcgen05.cp holds its thread for about 50 ns,
    // an MMA for 40), so the three strands of tensor work are issued by three threads: QK here, PV in
    // warp 2, the K scale atoms in warp 3. The tensor pipe runs what they issue in arrival order; the
    // strands touch different accumulators and hand over through mbarriers fed by tcgen05.commit.
    if (lane == 0 && num_steps > 0) {
      constexpr uint32_t idesc_qk = tc::nvf4_idesc(128, kOwn);
      constexpr uint32_t idesc_rope = tc::bf16_idesc(128, kOwn);
#pragma unroll
      for (int a = 0; a < kChunks * 2; ++a)
        tc::cp_sf_atom(tmem + kColSFQ + 4 * a, tc::sf_atom_desc(tc::smem_u32(sm.q_sf[a])));
      bool ok = true;
      for (int i = 0; i < num_steps && ok; ++i) {
        const int s = i % kStages;
        ok = wait_at(6, &sm.k_full[s], (i / kStages) & 1, abort_flag);
        if (ok) ok = wait_at(14, &sm.sfk_ready[i & 1], (i >> 1) & 1, abort_flag);
        // the scores of two steps ago, which this buffer held, have been read
        if (ok) ok = wait_at(7, &sm.s_empty[i & 1], ((i >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc::fence_after_sync();
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int k = 0; k < 2; ++k)
            tc::mma_nvf4(tmem + kColS + kOwn * (i & 1), tc::fp4_tile_desc(tc::smem_u32(sm.q_tile[c]), k),
                         tc::fp4_tile_desc(tc::smem_u32(sm.k_codes[s][c]), k), idesc_qk,
                         tmem + kColSFQ + 4 * (2 * c + k), tmem + kColSFK + 16 * (i & 1) + 4 * c + 2 * k, (c | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < kRope / 16; ++k)
          tc::mma_bf16(tmem + kColS + kOwn * (i & 1), tc::bf16_tile_desc(tc::smem_u32(sm.q_rope), k),
                       tc::bf16_tile_desc(tc::smem_u32(sm.rope[s]), k), idesc_rope, true);
        tc::commit(&sm.s_full[i & 1]);
        tc::commit(&sm.k_empty[s]);
      }
    }
  } else if (warp == 2) {
    // ---- output products: one thread --------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_pv = tc::nvf4_idesc(128, kHalf);
      bool ok = true;
      int examined = 0;  // steps so far on which the maxima were examined: the phase of the `again` barriers
      for (int m = 0; m < num_steps && ok; ++m) {
        const int s = m % kVStages;
        const int b = m % kPBuffers;
        const uint32_t p_phase = (m / kPBuffers) & 1;
        const int t = m & 1;  // which set of scale columns in tensor memory
        ok = wait_at(3, &sm.v_full[s], (m / kVStages) & 1, abort_flag);
        // both halves of the step's P operand: this CTA's (formed here) and the peer's (sent by the last
        // of its warps to finish forming it)
        if (ok) ok = wait_at(4, &sm.p_local[b], p_phase, abort_flag);
        if (ok) ok = wait_at(17, &sm.p_remote[b], p_phase, abort_flag);
        if (ok && (m == 0 || *const_cast<volatile int*>(&sm.p[b][0].examine) == m + 1 ||
                   *const_cast<volatile int*>(&sm.p[b][1].examine) == m + 1)) {
          // the halves are formed again and sent again
          ok = wait_at(13, &sm.again_local, examined & 1, abort_flag);
          if (ok) ok = wait_at(18, &sm.again_remote, examined & 1, abort_flag);
          ++examined;
        }
        if (!ok) break;
        tc::fence_after_sync();
#pragma unroll
        for (int a = 0; a < 4; ++a)  // [page][atom of chunk 0, atom of chunk 1]
          tc::cp_sf_atom(tmem + kColSFV + 16 * t + 4 * a, tc::sf_atom_desc(tc::smem_u32(sm.v_sf[s][0]) + a * 512));
#pragma unroll
        for (int e = 0; e < 2; ++e)
          tc::cp_sf_atom(tmem + kColSFP + 8 * t + 4 * e, tc::sf_atom_desc(tc::smem_u32(sm.p[b][e].sf)));
#pragma unroll
        for (int e = 0; e < 2; ++e)
          tc::mma_nvf4(tmem + kColO, tc::fp4_half_tile_desc(tc::smem_u32(sm.p[b][e].codes)),
                       tc::fp4_half_tile_desc(tc::smem_u32(sm.v_codes[s][e])), idesc_pv, tmem + kColSFP + 8 * t + 4 * e,
                       tmem + kColSFV + 16 * t + 8 * e, m > 0 || e > 0);
        tc::commit(&sm.o_done[m & 1]);
        tc::commit(&sm.v_empty[s]);
      }
    }
  } else if (warp == 3) {
    // ---- K scale atoms: the warp spreads them, one thread copies to tensor memory ------------------
    bool ok = true;
    for (int i = 0; i < num_steps && ok; ++i) {
      const int s = i % kStages;
      ok = wait_at(5, &sm.ksf_full[s], (i / kStages) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      {
        // The page's scale block arrived as [chunk][K block][32 rows][8 B] (64 tokens: two row quads
        // of four group scales). An atom row is 16 bytes, with room for four quads, and an N = 64
        // product reads only two: so one atom carries both K blocks of a chunk, the first in the low
        // half of every row (tensor-memory columns 0-1 of the atom), the second in the high half
        // (columns 2-3). Every lane reads all its pieces before any lane writes: done in place.
        uint8_t* sf = sm.k_sf[s];
        uint2 low[kChunks], high[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          low[c] = *reinterpret_cast<const uint2*>(sf + c * 512 + lane * 8);
          high[c] = *reinterpret_cast<const uint2*>(sf + c * 512 + 256 + lane * 8);
        }
        __syncwarp();
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          *reinterpret_cast<uint4*>(sf + c * 512 + lane * 16) = make_uint4(low[c].x, low[c].y, high[c].x, high[c].y);
        tc::fence_proxy_async_smem();
        __syncwarp();
      }
      if (lane == 0) {
        // this set of K scale columns is free once the score product of two steps ago has completed
        if (i > 1) ok = wait_at(15, &sm.s_full[i & 1], ((i - 2) >> 1) & 1, abort_flag);
        if (ok) {
          tc::fence_after_sync();
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tc::cp_sf_atom(tmem + kColSFK + 16 * (i & 1) + 4 * c, tc::sf_atom_desc(tc::smem_u32(sm.k_sf[s]) + c * 512));
          tc::commit(&sm.sfk_ready[i & 1]);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    }
  } else {
    // ---- softmax: kSoftmaxGroups threads per query head, each owning a run of the page's tokens ---
    const int warp_q = warp & 3;            // TMEM lane quarter this warp may read
    const int wg = (warp - 4) >> 2;         // this thread among its head's kSoftmaxGroups threads of the CTA
    const int team = wg / kTeamGroups;      // it forms the steps i with i % kTeams == team ...
    const int member = wg % kTeamGroups;    // ... and of those, this run of kRun tokens of the CTA's page
    const int h = warp_q * 32 + lane;       // head = TMEM lane of S and O
    const int slot = cta * kSoftmaxGroups + wg;  // this thread among its head's threads of the pair
    const uint32_t lane_base = tmem + ((uint32_t)(warp_q * 32) << 16);
    const float shift = p.p_mode == BDFP4_P_AMAX2_OR_AMAX6_C8 ? 3.0f : 0.0f;
    // A probability this large against the stale maximum means the maximum may have to move; the
    // trigger is a little below the rule's 2^8 so that the rule itself is only ever applied to the
    // exact scores (the examination), never to an approximate exponential.
    const float trigger_above = exp2f(kRescaleThreshold - 0.25f + shift);
    float row_max = -INFINITY, row_sum = 0.0f, max_scaled = 0.0f;
    // this thread's bytes of its CTA's P half: groups 2 wg, 2 wg + 1 of the page's four
    // the page's group `n` of a head: 8 bytes of the head's 32-byte row, whose 16-byte halves the swizzle swaps
    auto p_offset = [&](int n) { return h * 32 + (((n >> 1) ^ ((h >> 2) & 1)) << 4) + (n & 1) * 8; };
    const int sf_row = (h & 31) * 16 + (h >> 5) * 4 + member * kRunGroups;
    const int step_slot = cta * kTeamGroups + member;  // this thread among those of the pair that form its steps
    int examined = 0;  // steps so far on which the maxima were examined: the phase of `exchange`

    // arrival of this warp on a barrier of both CTAs, after every lane's stores
    auto warp_arrives = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) {
        tc::mbar_arrive_release_cluster(bar);
        tc::mbar_arrive_cluster(in_peer(bar));
      }
    };
    // This warp has formed (and proxy-fenced) its part of the P half in buffer `b`: it says so on `local`
    // for this CTA's readers, and the last warp of the team to get here sends the whole half into the
    // peer's buffer, counted on the peer's `remote` barrier, after announcing on this CTA's own `remote`
    // barrier that the peer's half is expected. Sending from here, rather than from the PV issuer, keeps
    // the crossing (about 650 cycles) out of that thread's loop.
    auto half_is_formed = [&](int b, uint64_t* local, uint64_t* remote, int* counter) {
      __syncwarp();
      if (lane == 0) {
        tc::mbar_arrive(local);
        __threadfence_block();
        const int before = atomicAdd(counter, 1);
        if (before == kTeamWarps - 1) {
          __threadfence_block();
          *counter = 0;
          tc::mbar_expect_tx(remote, kPHalfBytes);
          tc::bulk_copy_to_peer(in_peer(&sm.p[b][cta]), &sm.p[b][cta], kPHalfBytes, in_peer(remote));
        }
      }
    };

    // The walk is pipelined by one step: iteration i reads the scores of step i and forms its P half
    // against the maximum in force, and only then looks at how step i - 1 came out in the pair (both
    // halves in place, nobody asked for the examination: almost always), so the time the halves take
    // to cross between the CTAs is spent forming. Step i's half is announced after that look; if
    // step i - 1 had to be examined, both halves are formed again first, in order. The scores of the
    // step awaiting its outcome stay in registers.
    float s_own[kRun];   // the scores of the last step this thread formed, until its outcome is known
    float sum_own = 0.0f, largest = 0.0f;

    auto load_scores = [&](int i, float* s) {
      const int sb = i & 1;
      wait_at(8, &sm.s_full[sb], (i >> 1) & 1, abort_flag);
      tc::fence_after_sync();
#pragma unroll
      for (int q = 0; q < kRunGroups; ++q) tc::tmem_ld16(lane_base + kColS + kOwn * sb + member * kRun + 16 * q, s + 16 * q);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      // one lane arrives for the warp: hundreds of per-thread arrivals on one barrier serialise
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sm.s_empty[sb]);
      const int step = last_step - 1 - i;
      const int valid = seq_len - step * kStep - cta * kOwn - member * kRun;  // only the row's last step can be short
      if (valid < kRun) {
#pragma unroll
        for (int k = 0; k < kRun; ++k) s[k] = k < valid ? s[k] : -INFINITY;
      }
    };

    // Probabilities of this thread's run of step i against `max_scaled`, quantized sixteen at a time
    // and stored into this CTA's P half with their scale bytes. Forming and quantizing are one loop so
    // that the exponentials of one group overlap the conversions of the one before. Returns the run's
    // sum; `largest` becomes its largest probability.
    auto form_and_store = [&](int i, const float* s) -> float {
      PHalf& half = sm.p[i % kPBuffers][cta];
      float run_sum = 0.0f;
      uint32_t scale_bytes = 0;
      largest = 0.0f;
#pragma unroll
      for (int g = 0; g < kRunGroups; ++g) {
        float prob[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) prob[k] = ex2_approx(fmaf(s[16 * g + k], p.scale_log2, -max_scaled));
        // sums and maxima as trees: few warps share a scheduler, so a serial chain is paid in full
        float sum4[4], max4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          sum4[k] = (prob[k] + prob[k + 4]) + (prob[k + 8] + prob[k + 12]);
          max4[k] = fmaxf(fmaxf(prob[k], prob[k + 4]), fmaxf(prob[k + 8], prob[k + 12]));
        }
        run_sum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        const float group_max = fmaxf(fmaxf(max4[0], max4[1]), fmaxf(max4[2], max4[3]));
        largest = fmaxf(largest, group_max);
        const float scale = probability_scale(group_max, p.p_mode, p.tau);
        const float inverse = rcp_approx(fmaxf(scale, 1e-20f));
        uint32_t words[2] = {0, 0};
#pragma unroll
        for (int k = 0; k < 8; ++k)
          words[k >> 2] |= cvt_e2m1x2(prob[2 * k] * inverse, prob[2 * k + 1] * inverse) << (8 * (k & 3));
        *reinterpret_cast<uint2*>(half.codes + p_offset(member * kRunGroups + g)) = make_uint2(words[0], words[1]);
        scale_bytes |= (uint32_t)cvt_e4m3(scale) << (8 * g);
      }
      static_assert(kRunGroups == 1 || kRunGroups == 2, "one or two scale bytes per thread and step");
      if constexpr (kRunGroups == 1) half.sf[sf_row] = (uint8_t)scale_bytes;
      if constexpr (kRunGroups == 2) *reinterpret_cast<uint16_t*>(half.sf + sf_row) = (uint16_t)scale_bytes;
      return run_sum;
    };

    for (int i = 0; i <= num_steps; ++i) {
      const bool mine = i < num_steps && i % kTeams == team;  // this thread's team forms step i
      if (mine) {
        load_scores(i, s_own);
        // The P buffer of three steps ago is free: this CTA's PV product of that step was observed an
        // iteration ago, and the peer had seen that half before it announced the step after it,
        // which the last look waited for. (Step 0 is always examined: nothing to form yet.)
        sum_own = i > 0 ? form_and_store(i, s_own) : 0.0f;
      }
      if (i > 0) {
        // ---- how step j = i - 1 came out (every thread looks at every step, whoever formed it)
        const int j = i - 1, bj = j % kPBuffers;
        const bool formed_j = j % kTeams == team;
        // PV products complete in order; every completion is observed in turn (a parity wait can only
        // tell the current phase from the one before it, and the product of step j may be done already:
        // hence one barrier for even steps and one for odd)
        if (j > 0) wait_at(11, &sm.o_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag);
        wait_at(9, &sm.p_local[bj], (j / kPBuffers) & 1, abort_flag);
        wait_at(19, &sm.p_remote[bj], (j / kPBuffers) & 1, abort_flag);
        if (j == 0 || *const_cast<volatile int*>(&sm.p[bj][0].examine) == j + 1 ||
            *const_cast<volatile int*>(&sm.p[bj][1].examine) == j + 1) {
          // ---- the examination: the stale-maximum rule on the exact scores of all 128 tokens of
          // step j, identically in every thread of a head in both CTAs. The threads that formed the
          // step still hold its scores and publish their maxima; all threads read them.
          if (formed_j) {
            float run_max = s_own[0];
#pragma unroll
            for (int k = 1; k < kRun; ++k) run_max = fmaxf(run_max, s_own[k]);
            float* slot_of_mine = &sm.red[examined & 1][step_slot][h];
            *slot_of_mine = run_max;
            tc::cluster_store_b32(in_peer(slot_of_mine), __float_as_uint(run_max));
          }
          // every warp arrives, also those with nothing to publish: a phase of this barrier can then
          // not complete before every warp has seen the one before it
          warp_arrives(&sm.exchange);
          wait_at<true>(10, &sm.exchange, examined & 1, abort_flag);
          float block_max = sm.red[examined & 1][0][h];
#pragma unroll
          for (int w = 1; w < kStepSlots; ++w) block_max = fmaxf(block_max, sm.red[examined & 1][w][h]);
          ++examined;
          float acc = 1.0f;
          if (j == 0) {
            row_max = block_max;
            acc = 0.0f;
          } else if (block_max > row_max) {
            const float safe = block_max == -INFINITY ? 0.0f : block_max;
            const float growth = (row_max - safe) * p.scale_log2;
            if (growth < -kRescaleThreshold) {
              acc = ex2_approx(growth);
              row_max = block_max;
            }
          }
          max_scaled = (row_max == -INFINITY ? 0.0f : row_max) * p.scale_log2 - shift;
          if (j > 0 && __any_sync(0xffffffffu, acc != 1.0f)) {
            // O so far is rescaled in tensor memory, each thread of a head taking its share of its
            // CTA's columns. The PV product of step j - 1 has completed (observed above), and step
            // j's is not issued before both halves have been formed again.
            tc::fence_after_sync();
#pragma unroll 1
            for (int q = 0; q < kShare / 16; ++q) {
              float o[16];
              tc::tmem_ld16(lane_base + kColO + wg * kShare + 16 * q, o);
              tc::tmem_wait_ld();
#pragma unroll
              for (int k = 0; k < 16; ++k) o[k] *= acc;
              tc::tmem_st16(lane_base + kColO + wg * kShare + 16 * q, o);
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
          }
          row_sum *= acc;
          if (formed_j) {
            // Step j again, against the maximum now in force. (The first copy of this half has been
            // seen by the peer's threads before they passed the exchange, so it is no longer being read.)
            sum_own = form_and_store(j, s_own);
            tc::fence_proxy_async_smem();
            half_is_formed(bj, &sm.again_local, &sm.again_remote, &sm.formed_again);
          }
          if (mine) sum_own = form_and_store(i, s_own);  // and step i, formed above but not announced yet
        }
        if (formed_j) row_sum += sum_own;
      }
      if (mine) {
        if (i > 0 && __any_sync(0xffffffffu, largest > trigger_above) && lane == 0)
          *const_cast<volatile int*>(&sm.p[i % kPBuffers][cta].examine) = i + 1;
        tc::fence_proxy_async_smem();
        half_is_formed(i % kPBuffers, &sm.p_local[i % kPBuffers], &sm.p_remote[i % kPBuffers], &sm.formed[i % kPBuffers]);
      }
    }

    // ---- normalise and write ------------------------------------------------------------------
    sm.sums[slot][h] = row_sum;
    tc::cluster_store_b32(in_peer(&sm.sums[slot][h]), __float_as_uint(row_sum));
    warp_arrives(&sm.exchange);
    wait_at<true>(16, &sm.exchange, examined & 1, abort_flag);
    float total = sm.sums[0][h];
#pragma unroll
    for (int w = 1; w < kSlots; ++w) total += sm.sums[w][h];
    const bool empty = num_steps == 0 || total == 0.0f || total != total;
    const float inverse = empty ? 0.0f : 1.0f / total;
    const int64_t head = (int64_t)row * p.heads_q + head0 + h;
    if (p.out == nullptr && slot == 0 && h < valid_heads) {
      const float safe = row_max == -INFINITY ? 0.0f : row_max;
      p.partial_lse[(int64_t)part * p.rows * p.heads_q + head] =
          empty ? -INFINITY : (safe * p.scale_log2 + log2f(total) - shift) * 0.6931471805599453f;
    }
    if (num_steps > 0) {  // the loop observed every completion but the last step's
      wait_at(12, &sm.o_done[(num_steps - 1) & 1], ((num_steps - 1) >> 1) & 1, abort_flag);
      tc::fence_after_sync();
    }
#pragma unroll 1
    for (int q = 0; q < kShare / 16; ++q) {
      float o[16];
      if (num_steps > 0) {
        tc::tmem_ld16(lane_base + kColO + wg * kShare + 16 * q, o);
        tc::tmem_wait_ld();
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) o[k] = empty ? 0.0f : o[k] * inverse;
      if (h < valid_heads) {
        const int channel = cta * kHalf + wg * kShare + 16 * q;
        if (p.out != nullptr) {
          uint4 lo, hi;
          lo.x = pack_bf16x2(o[0], o[1]);
          lo.y = pack_bf16x2(o[2], o[3]);
          lo.z = pack_bf16x2(o[4], o[5]);
          lo.w = pack_bf16x2(o[6], o[7]);
          hi.x = pack_bf16x2(o[8], o[9]);
          hi.y = pack_bf16x2(o[10], o[11]);
          hi.z = pack_bf16x2(o[12], o[13]);
          hi.w = pack_bf16x2(o[14], o[15]);
          uint4* dst = reinterpret_cast<uint4*>(p.out + head * kLatent + channel);
          dst[0] = lo;
          dst[1] = hi;
        } else {
          float4* dst = reinterpret_cast<float4*>(p.partial_out + ((int64_t)part * p.rows * p.heads_q + head) * kLatent +
                                                  channel);
#pragma unroll
          for (int k = 0; k < 4; ++k) dst[k] = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
        }
      }
    }
    tc::fence_before_sync();
  }

  // ---- teardown -------------------------------------------------------------------------------
  // Neither CTA leaves while the other may still write into its shared memory or arrive on its
  // barriers: all threads of the pair meet here (every wait above is bounded, so both get here).
  // Every copy between the two has been waited for by its receiver, unless that gave up: then a copy
  // may still be under way, so the pair lingers a little and meets once more.
  tc::fence_before_sync();
  tc::cluster_sync_all();
  if (sm.abort_flag) __nanosleep(20000);
  tc::cluster_sync_all();
  if (tid == 0 && sm.abort_flag && p.error_word)
    atomicOr(p.error_word, (int)BDFP4_DEV_WAIT_TIMEOUT | ((sm.abort_flag & 0xff) << 8));
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemColumns);
  }
}

// ---- writers ------------------------------------------------------------------------------------

// One thread per 16-channel group of the absorbed query: codes at [row][head][256], scale byte at
// [row][head][32].
__global__ void __launch_bounds__(256) quantize_query_kernel(const __nv_bfloat16* query, int64_t row_pitch, int rows,
                                                             int heads_q, ScaleCandidates cand, uint8_t* codes,
                                                             uint8_t* scales) {
  wait_for_prior_kernels();  // the buffers written here may still be read by the launch before
  dependents_may_launch();
  const int64_t index = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t total = (int64_t)rows * heads_q * 32;
  if (index >= total) return;
  const int group = (int)(index & 31);
  const int64_t head = index >> 5;
  const int64_t row = head / heads_q;
  const int h = (int)(head % heads_q);
  float v[16];
  load_bf16x16(query + row * row_pitch + (int64_t)h * kLatent + group * 16, v);
  const GroupCodes q = quantize_group16(v, cand);
  *reinterpret_cast<uint2*>(codes + head * 256 + group * 8) = make_uint2(q.lo, q.hi);
  scales[head * 32 + group] = (uint8_t)cvt_e4m3(q.scale);
}

// One CTA per work item: 64 tokens x 128 bytes into the page's swizzled block.
__global__ void __launch_bounds__(256) rope_page_kernel(const __nv_bfloat16* rope, int64_t token_pitch,
                                                        const int32_t* source_tokens, const int32_t* destination_pages,
                                                        uint8_t* pages, int64_t rope_pitch) {
  const int page = destination_pages[blockIdx.x];
  if (page < 0) return;
  const int64_t source = source_tokens[blockIdx.x];
  for (int i = threadIdx.x; i < 64 * 8; i += 256) {
    const int token = i >> 3, c = i & 7;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(rope + (source + token) * token_pitch) + c);
    *reinterpret_cast<uint4*>(pages + (int64_t)page * rope_pitch + token * 128 + ((c ^ (token & 7)) << 4)) = v;
  }
}

// One CTA per row: the row's new token into its open page of the staging buffers, and the row's
// entry of the page writers' work table.
__global__ void __launch_bounds__(128) append_kernel(const __nv_bfloat16* new_latent, const __nv_bfloat16* new_rope,
                                                     __nv_bfloat16* staging_latent, __nv_bfloat16* staging_rope,
                                                     const int32_t* seq_lens, const int32_t* page_table,
                                                     int64_t page_table_stride, int page_table_columns, int pages,
                                                     int32_t* source_tokens, int32_t* destination_pages,
                                                     int32_t* error_word) {
  wait_for_prior_kernels();
  dependents_may_launch();
  const int row = blockIdx.x;
  const int length = max(seq_lens[row], 0);
  const int position = length & 63;
  uint4* latent = reinterpret_cast<uint4*>(staging_latent + (int64_t)row * 64 * kLatent);  // 64 chunks per token
  uint4* rope = reinterpret_cast<uint4*>(staging_rope + (int64_t)row * 64 * kRope);        // 8 chunks per token
  const int t = threadIdx.x;
  if (position == 0) {  // a page starts: nothing of the previous one may remain
    for (int i = t; i < 64 * 64; i += 128) latent[i] = make_uint4(0, 0, 0, 0);
    for (int i = t; i < 64 * 8; i += 128) rope[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }
  if (t < 64) latent[position * 64 + t] = __ldg(reinterpret_cast<const uint4*>(new_latent + (int64_t)row * kLatent) + t);
  if (t >= 64 && t < 72)
    rope[position * 8 + (t - 64)] = __ldg(reinterpret_cast<const uint4*>(new_rope + (int64_t)row * kRope) + (t - 64));
  if (t == 0) {
    // a row that has filled every column of its table has no open page: reading one column further
    // would return the next row's first entry, a valid page of another sequence
    const int column = length >> 6;
    int page = column < page_table_columns ? page_table[(int64_t)row * page_table_stride + column] : -1;
    if (page < 0 || page >= pages) {
      if (error_word) atomicOr(error_word, (int)BDFP4_DEV_BAD_PAGE);
      page = -1;
    }
    source_tokens[row] = row * 64;
    destination_pages[row] = page;
  }
}

// Merge of split partials: one CTA per (row, head), one thread per 4 channels.
__global__ void __launch_bounds__(128) combine_kernel(const float* partial_out, const float* partial_lse, int parts,
                                                      int64_t part_stride_heads, __nv_bfloat16* out) {
  constexpr float kLog2e = 1.4426950408889634f;
  const int64_t head = blockIdx.x;
  wait_for_prior_kernels();
  dependents_may_launch();
  float lse_max = -INFINITY;
  for (int s = 0; s < parts; ++s) lse_max = fmaxf(lse_max, partial_lse[s * part_stride_heads + head]);
  if (lse_max == -INFINITY) lse_max = 0.0f;
  float weight_sum = 0.0f;
  for (int s = 0; s < parts; ++s) weight_sum += exp2f(partial_lse[s * part_stride_heads + head] * kLog2e - lse_max * kLog2e);
  const float inverse = (weight_sum == 0.0f || weight_sum != weight_sum) ? 0.0f : 1.0f / weight_sum;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < parts; ++s) {
    const float scale = exp2f(partial_lse[s * part_stride_heads + head] * kLog2e - lse_max * kLog2e) * inverse;
    if (scale > 0.0f) {
      const float4 v = *reinterpret_cast<const float4*>(partial_out + (s * part_stride_heads + head) * kLatent +
                                                        threadIdx.x * 4);
      acc.x = acc.x + scale * v.x;
      acc.y = acc.y + scale * v.y;
      acc.z = acc.z + scale * v.z;
      acc.w = acc.w + scale * v.w;
    }
  }
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + head * kLatent + threadIdx.x * 4);
  dst[0] = __floats2bfloat162_rn(acc.x, acc.y);
  dst[1] = __floats2bfloat162_rn(acc.z, acc.w);
}

// Launch with programmatic stream serialization: after a kernel that signals early the CTAs come
// up and run their preamble while it still runs; after any other kernel this is an ordinary launch.
// `cluster` > 1 groups that many neighbouring CTAs of the grid into a cluster.
template <typename... Params, typename... Args>
static cudaError_t launch_overlapped_clusters(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, unsigned cluster, Args... args) {
  cudaLaunchAttribute attributes[2] = {};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = cluster;
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  config.attrs = attributes;
  config.numAttrs = cluster > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
static cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  return launch_overlapped_clusters(kernel, grid, block, smem, stream, 1u, args...);
}

}  // namespace mla
}  // namespace bdfp4

using namespace bdfp4;


extern "C" int bdfp4_mla_quantize_query(const void* query, int64_t row_pitch, int32_t rows, int32_t heads_q,
                                        int32_t scale_mode, void* codes, void* scales, void* stream) {
  if (!query || !codes || !scales || rows < 1 || heads_q < 1) return BDFP4_E_ARG;
  if (scale_mode < 0 || scale_mode > 2) return BDFP4_E_ARG;
  if (row_pitch < (int64_t)heads_q * mla::kLatent || row_pitch % 8) return BDFP4_E_ARG;
  if ((reinterpret_cast<uintptr_t>(query) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7)) return BDFP4_E_ARG;
  const int64_t groups = (int64_t)rows * heads_q * 32;
  return bdfp4::cuda_status(mla::launch_overlapped(
      mla::quantize_query_kernel, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(query), row_pitch, rows, heads_q, scale_candidates(scale_mode),
      static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales)));
}

extern "C" int bdfp4_mla_write_rope(const void* rope, int64_t token_pitch, const int32_t* source_tokens,
                                    const int32_t* destination_pages, int32_t work_items, void* rope_pages,
                                    int64_t rope_pitch, void* stream) {
  if (!rope || !source_tokens || !destination_pages || !rope_pages || work_items < 0) return BDFP4_E_ARG;
  if (token_pitch < mla::kRope || token_pitch % 8 || rope_pitch < 8192 || rope_pitch % 16) return BDFP4_E_ARG;
  if ((reinterpret_cast<uintptr_t>(rope) & 15) || (reinterpret_cast<uintptr_t>(rope_pages) & 15)) return BDFP4_E_ARG;
  if (work_items == 0) return BDFP4_OK;
  mla::rope_page_kernel<<<work_items, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(rope), token_pitch, source_tokens, destination_pages,
      static_cast<uint8_t*>(rope_pages), rope_pitch);
  return bdfp4::cuda_status(cudaGetLastError());
}

extern "C" int bdfp4_mla_append(const void* new_latent, const void* new_rope, void* staging_latent, void* staging_rope,
                                const int32_t* seq_lens, const int32_t* page_table, int64_t page_table_stride,
                                int32_t page_table_columns, int32_t rows, int32_t pages, int32_t* source_tokens,
                                int32_t* destination_pages, int32_t* error_word, void* stream) {
  if (!new_latent || !new_rope || !staging_latent || !staging_rope || !seq_lens || !page_table || !source_tokens ||
      !destination_pages)
    return BDFP4_E_ARG;
  if (rows < 1 || pages < 1 || page_table_columns < 1 || page_table_stride < page_table_columns) return BDFP4_E_ARG;
  auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (misaligned(new_latent) || misaligned(new_rope) || misaligned(staging_latent) || misaligned(staging_rope))
    return BDFP4_E_ARG;
  return bdfp4::cuda_status(mla::launch_overlapped(
      mla::append_kernel, dim3((unsigned)rows), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(new_latent), static_cast<const __nv_bfloat16*>(new_rope),
      static_cast<__nv_bfloat16*>(staging_latent), static_cast<__nv_bfloat16*>(staging_rope), seq_lens, page_table,
      page_table_stride, (int)page_table_columns, (int)pages, source_tokens, destination_pages, error_word));
}

extern "C" int bdfp4_mla_decode(const bdfp4_mla_decode_args* a, void* stream_handle) {
  if (!a) return BDFP4_E_ARG;
  if (a->rows < 1 || a->heads_q < 1) return BDFP4_E_ARG;
  if (a->heads_q % 64) return BDFP4_E_UNSUPPORTED;
  if (!a->query_codes || !a->query_scales || !a->query_rope) return BDFP4_E_ARG;
  if (!a->key_codes || !a->key_scales || !a->value_codes || !a->value_scales || !a->rope_pages) return BDFP4_E_ARG;
  if (a->pages < 1 || !a->page_table || !a->seq_lens || a->page_table_stride < 1) return BDFP4_E_ARG;
  auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (misaligned(a->query_codes) || misaligned(a->query_scales) || misaligned(a->query_rope) ||
      misaligned(a->key_codes) || misaligned(a->key_scales) || misaligned(a->value_codes) ||
      misaligned(a->value_scales) || misaligned(a->rope_pages))
    return BDFP4_E_ARG;
  if (a->key_codes_pitch % 16 || a->key_scales_pitch % 16 || a->value_codes_pitch % 16 ||
      a->value_scales_pitch % 16 || a->rope_pitch % 16)
    return BDFP4_E_ARG;
  if (a->key_codes_pitch < 16384 || a->value_codes_pitch < 16384 || a->key_scales_pitch < 2048 ||
      a->value_scales_pitch < 2048 || a->rope_pitch < 8192)
    return BDFP4_E_ARG;
  if (!(a->softmax_scale > 0.0f) || !isfinite(a->softmax_scale)) return BDFP4_E_ARG;
  if (a->p_scale_mode < 0 || a->p_scale_mode > 2 || a->num_splits < 1) return BDFP4_E_ARG;
  const bool writes_out = a->num_splits == 1 && a->out != nullptr;
  if (!writes_out && (!a->partial_out || !a->partial_lse)) return BDFP4_E_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);

  mla::Params p{};
  p.rows = a->rows;
  p.heads_q = a->heads_q;
  p.head_blocks = (a->heads_q + mla::kHeads - 1) / mla::kHeads;
  p.q_codes = static_cast<const uint8_t*>(a->query_codes);
  p.q_scales = static_cast<const uint8_t*>(a->query_scales);
  p.q_rope = static_cast<const __nv_bfloat16*>(a->query_rope);
  p.k_codes = static_cast<const uint8_t*>(a->key_codes);
  p.k_scales = static_cast<const uint8_t*>(a->key_scales);
  p.v_codes = static_cast<const uint8_t*>(a->value_codes);
  p.v_scales = static_cast<const uint8_t*>(a->value_scales);
  p.rope = static_cast<const uint8_t*>(a->rope_pages);
  p.k_codes_pitch = a->key_codes_pitch;
  p.k_scales_pitch = a->key_scales_pitch;
  p.v_codes_pitch = a->value_codes_pitch;
  p.v_scales_pitch = a->value_scales_pitch;
  p.rope_pitch = a->rope_pitch;
  p.pages = a->pages;
  p.page_table = a->page_table;
  p.page_table_stride = a->page_table_stride;
  p.seq_lens = a->seq_lens;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.p_mode = a->p_scale_mode;
  p.tau = a->p_scale_tau;
  p.out = writes_out ? static_cast<__nv_bfloat16*>(a->out) : nullptr;
  p.num_splits = a->num_splits;
  p.partial_out = a->partial_out;
  p.partial_lse = a->partial_lse;
  p.error_word = a->error_word;

  const int smem = (int)sizeof(mla::Smem) + 1024;
  static PerDeviceOnce configured;
  const int slot = current_device_slot();
  if (slot < 0 || !configured.done[slot]) {
    cudaError_t e = cudaFuncSetAttribute(mla::decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return bdfp4::cuda_status(e);
    if (slot >= 0) configured.done[slot] = true;
  }
  const int64_t grid = (int64_t)a->rows * p.head_blocks * a->num_splits * 2;
  if (grid > 0x7fffffff) return BDFP4_E_TOO_LARGE;
  return bdfp4::cuda_status(mla::launch_overlapped_clusters(mla::decode_kernel, dim3((unsigned)grid),
                                                            dim3(mla::kThreads), smem, stream, 2u, p));
}

extern "C" int bdfp4_mla_combine(const float* partial_out, const float* partial_lse, int32_t parts, int32_t rows,
                                 int32_t heads_q, void* out, void* stream) {
  if (!partial_out || !partial_lse || !out || parts < 1 || rows < 1 || heads_q < 1) return BDFP4_E_ARG;
  const int64_t heads = (int64_t)rows * heads_q;
  if (heads > 0x7fffffff) return BDFP4_E_TOO_LARGE;
  return bdfp4::cuda_status(mla::launch_overlapped(mla::combine_kernel, dim3((unsigned)heads), dim3(128), 0,
                                                   static_cast<cudaStream_t>(stream), partial_out, partial_lse,
                                                   (int)parts, (int64_t)heads, static_cast<__nv_bfloat16*>(out)));
}
