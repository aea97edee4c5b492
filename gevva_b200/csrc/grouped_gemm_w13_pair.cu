// Fused w13 GEMM + GeGLU + NVFP4 requantisation run by CTA pairs, weights on the MMA's M side.
//
// Why this shape.  An SM takes in at most about 140 GB/s through TMA (measured with all SMs
// streaming from L2), and one K block of 256 elements of a 128 x 256 tile needs 54 KiB for 512
// tensor-pipe cycles: the one-CTA kernel (grouped_gemm.cu) is bound by that intake, not by the
// tensor pipe.  Here a CTA pair (tcgen05 cta_group::2, M = 256) holds 256 weight rows, 128 per
// CTA, against up to 256 token rows of one expert on the N side, half of them loaded by each CTA:
// at most 38 KiB per CTA and K block.  And because the tokens sit on N, which may be any multiple
// of 16, a group of 300 rows costs 304 rows of tensor work instead of three 128-row tiles.
//
// Work.  A chunk is one entry of the route plan's tile-pair list: up to 256 consecutive rows of
// one expert starting at a 128-row tile (so its activation scales are whole 128-row blocks).  The
// intermediate width 704 is cut into 11 units of 64 columns; a CTA computes one unit as 128 MMA
// rows, the unit's 64 up rows on lanes 0..63 and its 64 gate rows on lanes 64..127, so that up
// and gate of a column end in the same CTA.  A work item is (chunk, two units); the second CTA of
// the sixth item has no unit (its weight scales are zero and its results are dropped).
//
// Protocol.  As in every kernel here: a TMA producer (one warp per CTA) fills a ring of stages,
// all loads of both CTAs complete on the `full` barrier of the first CTA (tensor-map loads in
// their cta_group::2 form, no multicast; the scale atoms travel through tensor maps too).  There
// the MMA thread copies the scale atoms of a landed stage into tensor memory, issues four MMAs
// (copies and MMAs of one thread execute in order) and commits to `empty` of both CTAs.  Spills
// are expensive here (shared memory leaves almost no L1), which is why the epilogue holds one
// 32-column load at a time.  The 16 epilogue warps of each CTA copy the accumulator (lanes = weight
// rows, columns = tokens) to registers as bf16(alpha * acc), release it, transpose it through
// shared memory and then, one thread per (token, 16 columns), apply erf-GELU(gate) * up and
// quantise exactly like the two-kernel form.  Every wait is bounded.
#include "gv_common.cuh"
#include "gv_gemm_parts.cuh"
#include "gv_launchers.h"

namespace gv {

namespace {

constexpr int kWpStages = 5;
constexpr int kWpThreads = (2 + 4 * kEpilogueWarpsPerQuarter) * 32;     // 576: leaves 112 registers per thread
constexpr uint32_t kWpTmemColumns = 512;
constexpr uint32_t kWpSfColumn = 256;          // accumulator: columns [0, 256)
constexpr uint32_t kWpSfColumnsPerStage = 48;  // per MMA j: weights at +12j, tokens 0..127 at +12j+4, 128..255 at +12j+8
constexpr int kWpTileBytes = 128 * kTileKBytes;  // 16 KiB
constexpr int kWpUnits = kInter / 64;            // 11
constexpr int kWpUnitSlots = 12;                 // the re-tiled scales carry a twelfth, all-zero unit
constexpr int kWpItemsPerChunk = kWpUnitSlots / 2;
constexpr int kWpStagePitch = 256;               // one token of the transposed tile: 128 lanes x bf16
constexpr int kWpStagingBytes = 32 * kWpStagePitch;

struct alignas(1024) WpSmem {
  uint8_t w[kWpStages][kWpTileBytes];          // this CTA's 64 up + 64 gate weight rows
  uint8_t x[kWpStages][kWpTileBytes];          // this CTA's half of the chunk's token rows
  uint8_t sfw[kWpStages][kSfStageBytes];       // scales of this CTA's weight rows
  uint8_t sfx[kWpStages][2 * kSfStageBytes];   // scales of the chunk's one or two 128-row blocks
  uint8_t staging[4][kWpStagingBytes];         // per token group of the epilogue: 32 tokens x 128 lanes, bf16
  uint64_t full[kWpStages];    // leader: the stage's bytes have landed in both CTAs
  uint64_t empty[kWpStages];   // both CTAs: the MMAs that read the stage have completed
  uint64_t acc_full;           // both CTAs: the item's accumulator is complete
  uint64_t acc_empty;          // leader: both CTAs' epilogues have copied the accumulator out
  uint32_t tmem_base;
  volatile int abort;
  int group_left[4];
  alignas(16) float erf_table[GV_ERF_TABLE_FLOATS];
};

constexpr size_t kWpSmemBytes = sizeof(WpSmem) + 1024;
static_assert(kWpSmemBytes <= 232448, "shared memory budget");
static_assert(kWpSfColumn + kWpSfColumnsPerStage * kWpStages <= kWpTmemColumns, "tensor memory budget");

__device__ __forceinline__ void wp_arrive_remote(uint64_t* local_bar, uint32_t target_cta) {
  const uint32_t remote = cluster_map_shared(smem_u32(local_bar), target_cta);
  // Relaxed: the arrive announces that tensor-memory reads have completed (tcgen05.wait::ld came
  // before it); no memory written by this thread has to be visible to the leader, and a release
  // here would first wait for the thread's earlier global stores.
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once every
// tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void wp_commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

// Tensor-map load into this CTA's shared memory that completes on a barrier of either CTA of the
// pair (`barrier` is a shared::cluster address).  No multicast: every CTA loads its own bytes.
__device__ __forceinline__ void wp_load(void* smem_dst, const void* tensor_map, uint32_t barrier, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(barrier)
      : "memory");
}

__device__ __forceinline__ void wp_load_3d(void* smem_dst, const void* tensor_map, uint32_t barrier, int x, int y,
                                           int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(smem_dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(barrier)
      : "memory");
}

// Asks for a box to be brought into L2 (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void wp_prefetch_3d(const void* tensor_map, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(tensor_map), "r"(x), "r"(y),
               "r"(z)
               : "memory");
}
__device__ __forceinline__ void wp_prefetch_2d(const void* tensor_map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tensor_map), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void wp_copy_sf(uint32_t tmem_address, uint32_t hi, uint32_t lo) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address),
               "l"((static_cast<uint64_t>(hi) << 32) | lo)
               : "memory");
}

__device__ __forceinline__ void wp_mma(uint32_t tmem_d, uint32_t hi, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                       uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"((static_cast<uint64_t>(hi) << 32) | a_lo), "l"((static_cast<uint64_t>(hi) << 32) | b_lo), "r"(idesc),
      "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// Scale copies of one K block (four MMAs of K = 64) for both CTAs: per MMA j the atom of the
// weight rows and the atoms of the chunk's one or two 128-row blocks of tokens.
template <bool kTwoBlocks>
__device__ __forceinline__ void wp_issue_sf_copies(uint32_t tmem_sf, uint32_t sfw_lo, uint32_t sfx_lo) {
  constexpr uint32_t hi_sf = (128u >> 4) | (1u << 14);                // 8 rows x 16 B, no swizzle
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) {
    wp_copy_sf(tmem_sf + 12 * j, hi_sf, sfw_lo + 32 * j);
    wp_copy_sf(tmem_sf + 12 * j + 4, hi_sf, sfx_lo + 32 * j);
    if (kTwoBlocks) wp_copy_sf(tmem_sf + 12 * j + 8, hi_sf, sfx_lo + 128 + 32 * j);
  }
}

__device__ __forceinline__ void wp_issue_mmas(uint32_t tmem_acc, uint32_t tmem_sf, uint32_t w_lo, uint32_t x_lo,
                                              uint32_t idesc, uint32_t accumulate) {
  constexpr uint32_t hi_ab = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8 rows x 128 B, 128B swizzle
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j)
    wp_mma(tmem_acc, hi_ab, w_lo + 2 * j, x_lo + 2 * j, idesc, tmem_sf + 12 * j, tmem_sf + 12 * j + 4,
           j == 0 ? accumulate : 1u);
}

struct WpItem {
  int first;     // first 128-row tile of the chunk
  int expert;
  int row0;      // first sorted row of the chunk
  int valid;     // rows of the chunk, 1..256
  int n;         // MMA N: valid rounded up to 16
  int unit_pair; // 0..5
};

struct WpPlan {
  const int* pair_tile;
  const int* tile_expert;
  const int* expert_offsets;
  const int* scale_row_offsets;
  int pair_begin;
  int total_items;
  int rounds;
};

// Items in snake order over the pairs of the grid: the unit pairs of a chunk go to neighbouring
// clusters, which then read the same token rows from L2 at about the same time.
__device__ __forceinline__ bool wp_item(const WpPlan& plan, int round, WpItem& item) {
  const int slots = static_cast<int>(gridDim.x) >> 1;
  const int mine = static_cast<int>(blockIdx.x) >> 1;
  const int slot = (round & 1) ? slots - 1 - mine : mine;
  const int index = round * slots + slot;
  if (index >= plan.total_items) return false;
  const int chunk = index / kWpItemsPerChunk;
  item.unit_pair = index - chunk * kWpItemsPerChunk;
  item.first = plan.pair_tile[plan.pair_begin + chunk] >> 1;
  item.expert = plan.tile_expert[item.first];
  const int local0 = item.first * kTileM - plan.scale_row_offsets[item.expert];
  item.row0 = plan.expert_offsets[item.expert] + local0;
  const int rows_after = plan.expert_offsets[item.expert + 1] - item.row0;
  item.valid = rows_after < 2 * kTileM ? rows_after : 2 * kTileM;
  item.n = (item.valid + 15) & ~15;
  return true;
}

__device__ __forceinline__ int wp_lower_bound(const int* __restrict__ pair_tile, int count, int tile) {
  int lo = 0, hi = count;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if ((pair_tile[mid] >> 1) < tile) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float wp_bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float wp_bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

// GeGLU and block quantisation of 16 columns of one token from values already rounded to bf16
// (what the reference's GEMM stores and its GeGLU kernel reads back, src/nvfp4_cutlass.cu:582-583).
__device__ __forceinline__ uint32_t wp_geglu_block(const uint4& u0, const uint4& u1, const uint4& g0, const uint4& g1,
                                                   float multiplier, const float* erf_table, uint32_t& codes_lo,
                                                   uint32_t& codes_hi) {
  const uint32_t up[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  const uint32_t gate[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  float values[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    values[2 * i] = __fmul_rn(gv_gelu_erf(wp_bf16_lo(gate[i]), erf_table), wp_bf16_lo(up[i]));
    values[2 * i + 1] = __fmul_rn(gv_gelu_erf(wp_bf16_hi(gate[i]), erf_table), wp_bf16_hi(up[i]));
  }
  return quantize_block16(values, multiplier, codes_lo, codes_hi);
}

struct WpTokenMaps {
  CUtensorMap rows[16];   // boxes of 8, 16, ... 128 token rows x 128 bytes
};

struct WpParams {
  const float* alpha;          // [experts] g1 output scale
  uint8_t* next_codes;         // [row capacity, 352] w2 operand codes
  uint8_t* next_scales;        // scale regions of the w2 operand
  const float* next_scale_q;   // [experts] g2.input_scale_quant
  const int* tile_expert;
  const int* expert_offsets;
  const int* scale_row_offsets;
  const int* num_m_tiles;
  const int* tile_first;       // optional: the launch covers tiles [tile_first, tile_first + num_m_tiles)
  const int* pair_tile;
  const int* num_pairs;
  int* status;
};

__global__ void __launch_bounds__(kWpThreads, 1)
w13_geglu_pair_kernel(const __grid_constant__ WpTokenMaps map_x, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_x_sf, const __grid_constant__ CUtensorMap map_w_sf,
                      const WpParams p) {
  extern __shared__ uint8_t smem_raw[];
  WpSmem* smem = reinterpret_cast<WpSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();   // 0 = leader
  const bool is_leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWpStages; ++s) {
      mbar_init(&smem->full[s], 1);   // the leader's producer announces both CTAs' byte count
      mbar_init(&smem->empty[s], 1);
    }
    mbar_init(&smem->acc_full, 1);
    mbar_init(&smem->acc_empty, kEpilogueThreads + kEpilogueThreads / 32);  // leader's threads + the second CTA's warps
    smem->abort = 0;
    for (int s = 0; s < 4; ++s) smem->group_left[s] = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_w);
    prefetch_tensor_map(&map_x_sf);
    prefetch_tensor_map(&map_w_sf);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kWpTmemColumns);  // the whole tensor memory: both CTAs get address 0
    tmem_relinquish();
  }
  load_erf_table(smem->erf_table);
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // Barriers of both CTAs exist before either CTA arrives on the other's.
  cluster_sync_all();
  const uint32_t tmem_base = smem->tmem_base;
  grid_dependency_wait();

  WpPlan plan;
  plan.pair_tile = p.pair_tile;
  plan.tile_expert = p.tile_expert;
  plan.expert_offsets = p.expert_offsets;
  plan.scale_row_offsets = p.scale_row_offsets;
  plan.pair_begin = 0;
  int pair_count = p.num_pairs[0];
  if (p.tile_first) {
    const int first = p.tile_first[0];
    plan.pair_begin = wp_lower_bound(p.pair_tile, pair_count, first);
    pair_count = wp_lower_bound(p.pair_tile, pair_count, first + p.num_m_tiles[0]) - plan.pair_begin;
  }
  plan.total_items = pair_count * kWpItemsPerChunk;
  const int slots = static_cast<int>(gridDim.x) >> 1;
  plan.rounds = (plan.total_items + slots - 1) / slots;
  constexpr int k_blocks = kHidden / 2 / kTileKBytes;   // 11

  if (warp == 0) {
    // ---------------- TMA producer (one warp in each CTA) ----------------
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int round = 0; ok && round < plan.rounds; ++round) {
      WpItem item;
      if (!wp_item(plan, round, item)) continue;
      const int unit = 2 * item.unit_pair + static_cast<int>(rank);
      const bool unit_exists = unit < kWpUnits;
      const int half = item.n >> 1;                            // token rows per CTA, a multiple of 8
      const int token_row = item.row0 + static_cast<int>(rank) * half;
      const bool second_exists = 2 * item.unit_pair + 1 < kWpUnits;
      // per K block and CTA: the weight scales (2 KiB), the scales of two 128-row blocks of tokens
      // (4 KiB; the second block is fetched, and ignored, also when the chunk has one), the token rows,
      // and the unit's weight rows
      const uint32_t both_bytes = 2 * (3 * kSfStageBytes + static_cast<uint32_t>(half) * kTileKBytes) + kWpTileBytes +
                                  (second_exists ? kWpTileBytes : 0);
      const CUtensorMap* token_map = &map_x.rows[(half >> 3) - 1];
      const int w_sf_row = ((item.expert * kWpUnitSlots + unit) * k_blocks) * 4;
      // While this item streams, the bytes of this CTA's next item are asked into L2, K block by K
      // block: the ring holds at most five stages, too few to cover the latency of a load that
      // misses L2 (the weights are read from HBM about once per chunk).
      WpItem next;
      const bool has_next = round + 1 < plan.rounds && wp_item(plan, round + 1, next);
      const int next_unit = has_next ? 2 * next.unit_pair + static_cast<int>(rank) : kWpUnits;
      const int next_half = has_next ? next.n >> 1 : 8;
      const CUtensorMap* next_token_map = &map_x.rows[(next_half >> 3) - 1];
      const int next_token_row = has_next ? next.row0 + static_cast<int>(rank) * next_half : 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, wait_or_abort<true>(&smem->empty[stage], phase ^ 1u, smem, p.status));
        if (!ok) break;
        if (elect_one()) {
          const int x = kb * kTileKBytes;
          const uint32_t bar = is_leader ? smem_u32(&smem->full[stage])
                                         : cluster_map_shared(smem_u32(&smem->full[stage]), 0);
          if (is_leader) mbar_arrive_expect_tx(&smem->full[stage], both_bytes);
          if (unit_exists) wp_load_3d(smem->w[stage], &map_w, bar, x, unit * 64, item.expert * 2);
          wp_load(smem->x[stage], token_map, bar, x, token_row);
          wp_load(smem->sfw[stage], &map_w_sf, bar, 0, w_sf_row + 4 * kb);
          wp_load_3d(smem->sfx[stage], &map_x_sf, bar, 0, 4 * kb, item.first);
          if (has_next) {
            if (next_unit < kWpUnits) wp_prefetch_3d(&map_w, x, next_unit * 64, next.expert * 2);
            wp_prefetch_2d(next_token_map, x, next_token_row);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == kWpStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok && lane == 0 && is_leader) {
      // Unwinding: let the copies already issued (by either CTA) land before shared memory is
      // given up; the second CTA stays resident until the cluster barrier at the end.
      const int pending = issued < kWpStages ? issued : kWpStages;
      int s = stage;
      uint32_t ph = phase;
      for (int i = 0; i < pending; ++i) {
        if (--s < 0) {
          s = kWpStages - 1;
          ph ^= 1u;
        }
        mbar_wait_bounded(&smem->full[s], ph, 40000000ll);
      }
    }
  } else if (warp == 1) {
    if (is_leader) {
      // ---------------- leader: scale copies and MMAs for both CTAs ----------------
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      const uint32_t w_lo0 = (smem_u32(smem->w[0]) & 0x3ffffu) >> 4;
      const uint32_t x_lo0 = (smem_u32(smem->x[0]) & 0x3ffffu) >> 4;
      const uint32_t sfw_lo0 = (smem_u32(smem->sfw[0]) & 0x3ffffu) >> 4;
      const uint32_t sfx_lo0 = (smem_u32(smem->sfx[0]) & 0x3ffffu) >> 4;
      const bool leader_lane = elect_one();
      for (int round = 0; round < plan.rounds; ++round) {
        WpItem item;
        if (!wp_item(plan, round, item)) continue;
        const bool two_blocks = item.n > kTileM;
        // E2M1 x E2M1, both K-major, UE4M3 scales; N at [17,23) in units of 8, M = 256 at [24,29) in units of 16
        const uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(item.n >> 3) << 17) |
                               (static_cast<uint32_t>(256 >> 4) << 24);
        if (!__all_sync(0xffffffffu, wait_or_abort<false>(&smem->acc_empty, acc_phase ^ 1u, smem, p.status))) break;
        acc_phase ^= 1u;
        bool ok = true;
        tc_fence_after_sync();
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = wait_or_abort<false>(&smem->full[stage], phase, smem, p.status);
          if (!ok) break;
          tc_fence_after_sync();
          if (leader_lane) {
            const uint32_t w_lo = w_lo0 + static_cast<uint32_t>(stage) * (kWpTileBytes >> 4);
            const uint32_t x_lo = x_lo0 + static_cast<uint32_t>(stage) * (kWpTileBytes >> 4);
            const uint32_t sfw_lo = sfw_lo0 + static_cast<uint32_t>(stage) * (kSfStageBytes >> 4);
            const uint32_t sfx_lo = sfx_lo0 + static_cast<uint32_t>(stage) * (2 * kSfStageBytes >> 4);
            const uint32_t tmem_sf = tmem_base + kWpSfColumn + kWpSfColumnsPerStage * stage;
            // copies and MMAs of one thread execute in order in the tensor pipe
            if (two_blocks) wp_issue_sf_copies<true>(tmem_sf, sfw_lo, sfx_lo);
            else wp_issue_sf_copies<false>(tmem_sf, sfw_lo, sfx_lo);
            wp_issue_mmas(tmem_base, tmem_sf, w_lo, x_lo, idesc, kb != 0 ? 1u : 0u);
            wp_commit_both(&smem->empty[stage]);   // both CTAs may refill the stage
            if (kb + 1 == k_blocks) wp_commit_both(&smem->acc_full);
          }
          if (++stage == kWpStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else {
    // ---------------- epilogue: 16 warps in each CTA ----------------
    // A warp may touch only the tensor-memory lanes 32*(warp%4)..+31 (here: 32 of the CTA's 128
    // weight rows); the four warps with the same `group` take the same 32 tokens of a pass and
    // share one staging tile.
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;  // 0..3
    uint32_t acc_phase = 0;
    uint8_t* staging = smem->staging[group];
    const int in_group = quarter * 32 + lane;       // 0..127: this thread's weight row, later its (token, block)
    for (int round = 0; round < plan.rounds; ++round) {
      WpItem item;
      if (!wp_item(plan, round, item)) continue;
      const int unit = 2 * item.unit_pair + static_cast<int>(rank);
      const bool unit_exists = unit < kWpUnits;
      const float alpha = p.alpha[item.expert];
      const float multiplier = p.next_scale_q[item.expert];
      const bool acc_ready = wait_or_abort<true>(&smem->acc_full, acc_phase, smem, p.status);
      acc_phase ^= 1u;
      if (!acc_ready) smem->group_left[group] = 1;
      named_barrier(1 + group, 4 * 32);
      if (*reinterpret_cast<volatile int*>(&smem->group_left[group])) break;
      tc_fence_after_sync();
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      // pass 0: tokens [32 group, +32); pass 1: tokens [128 + 32 group, +32)
      const bool has0 = unit_exists && 32 * group < item.valid;
      const bool has1 = unit_exists && 128 + 32 * group < item.valid;
      uint32_t packed[2][16];
      {
        uint32_t r[32];
        if (has0) {
          tmem_load_32x32(tmem_row + 32 * group, r);
          tmem_load_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[0][i] = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[2 * i])), __fmul_rn(alpha, __uint_as_float(r[2 * i + 1])));
        }
        if (has1) {
          tmem_load_32x32(tmem_row + 128 + 32 * group, r);
          tmem_load_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[1][i] = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[2 * i])), __fmul_rn(alpha, __uint_as_float(r[2 * i + 1])));
        }
      }
      tc_fence_before_sync();
      if (is_leader) {
        mbar_arrive(&smem->acc_empty);
      } else {
        __syncwarp();
        if (lane == 0) wp_arrive_remote(&smem->acc_empty, 0);
      }
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        if (!(pass == 0 ? has0 : has1)) continue;
        // transposed write: token i of the pass, this thread's weight row; the 16-byte chunk c of a
        // token lives at chunk position c ^ (token & 7)
        const int chunk = in_group >> 3;
        const int within = (in_group & 7) * 2;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint32_t pair = packed[pass][i >> 1];
          const uint16_t value = static_cast<uint16_t>((i & 1) ? pair >> 16 : pair & 0xffffu);
          *reinterpret_cast<uint16_t*>(staging + i * kWpStagePitch + ((chunk ^ (i & 7)) << 4) + within) = value;
        }
        named_barrier(1 + group, 4 * 32);
        // one thread per (token, 16 columns): lanes [16 b, +16) are up, [64 + 16 b, +16) gate
        const int t = in_group >> 2;
        const int b = in_group & 3;
        const uint8_t* row = staging + t * kWpStagePitch;
        const int swz = t & 7;
        const uint4 u0 = *reinterpret_cast<const uint4*>(row + (((2 * b) ^ swz) << 4));
        const uint4 u1 = *reinterpret_cast<const uint4*>(row + (((2 * b + 1) ^ swz) << 4));
        const uint4 g0 = *reinterpret_cast<const uint4*>(row + (((8 + 2 * b) ^ swz) << 4));
        const uint4 g1 = *reinterpret_cast<const uint4*>(row + (((8 + 2 * b + 1) ^ swz) << 4));
        uint2 codes;
        uint32_t scale = wp_geglu_block(u0, u1, g0, g1, multiplier, smem->erf_table, codes.x, codes.y);
        const int token = 128 * pass + 32 * group + t;
        const bool valid = token < item.valid;
        if (valid)
          *reinterpret_cast<uint2*>(p.next_codes + static_cast<size_t>(item.row0 + token) * (kInter / 2) + unit * 32 + b * 8) = codes;
        // the four scale bytes of a token's unit are one aligned word of the w2 operand's scale atom
        scale <<= 8 * b;
        scale |= __shfl_xor_sync(0xffffffffu, scale, 1);
        scale |= __shfl_xor_sync(0xffffffffu, scale, 2);
        if (valid && b == 0) {
          constexpr int groups = kInter / 16;
          const int tile = item.first + (token >> 7);
          *reinterpret_cast<uint32_t*>(p.next_scales + static_cast<size_t>(tile) * kTileM * groups +
                                       sf_offset(token & 127, 4 * unit, groups)) = scale;
        }
        named_barrier(1 + group, 4 * 32);  // the staging tile is rewritten by the next pass or item
      }
    }
  }

  tc_fence_before_sync();
  // Both CTAs stay until neither can still receive a remote arrive, a copy or a multicast commit.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, kWpTmemColumns);
  }
}

// Re-tiles the w13 block scales for this kernel: unit u of an expert (intermediate columns
// [64u, 64u+64)) is 128 MMA rows, up rows on 0..63 and gate rows on 64..127.  Per expert, unit
// (twelve slots, the last all zero) and K block of 256 the copy holds [MMA 0..3][512-byte atom],
// the atom being (n%32)*16 + (n/32)*4 + k over the 128 rows n.  One thread per byte.
__global__ void retile_w13_unit_scales_kernel(const uint8_t* __restrict__ sidecar, uint8_t* __restrict__ tiled,
                                              int experts) {
  constexpr int groups = kHidden / 16;          // 176
  constexpr int k_blocks = kHidden / 256;       // 11
  const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(experts) * kWpUnitSlots * k_blocks * 4 * kSfAtomBytes;
  if (index >= total) return;
  const int byte = static_cast<int>(index % kSfAtomBytes);
  size_t rest = index / kSfAtomBytes;
  const int mma = static_cast<int>(rest % 4);
  rest /= 4;
  const int k_block = static_cast<int>(rest % k_blocks);
  rest /= k_blocks;
  const int unit = static_cast<int>(rest % kWpUnitSlots);
  const int expert = static_cast<int>(rest / kWpUnitSlots);
  const int n = ((byte & 15) >> 2) * 32 + (byte >> 4);  // MMA row of this byte
  const int k = byte & 3;
  uint8_t value = 0;
  if (unit < kWpUnits) {
    const int source_row = n < 64 ? unit * 64 + n : kInter + unit * 64 + (n - 64);
    value = sidecar[static_cast<size_t>(expert) * kW13Out * groups +
                    sf_offset(source_row, (k_block * 4 + mma) * 4 + k, groups)];
  }
  tiled[index] = value;
}

}  // namespace

size_t w13_unit_scale_bytes(int experts) {
  return static_cast<size_t>(experts) * kWpUnitSlots * (kHidden / 256) * 4 * kSfAtomBytes;
}

void launch_retile_w13_unit_scales(const uint8_t* sidecar_scales, uint8_t* tiled, int experts, cudaStream_t stream) {
  const size_t total = w13_unit_scale_bytes(experts);
  retile_w13_unit_scales_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(sidecar_scales, tiled,
                                                                                                 experts);
}

int prepare_w13_pairs() {
  return static_cast<int>(cudaFuncSetAttribute(w13_geglu_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kWpSmemBytes)));
}

void launch_w13_pairs(const W13PairOperands& op, const RoutePlan& plan, int sm_count, cudaStream_t stream) {
  WpParams p{};
  p.alpha = op.alpha;
  p.next_codes = op.next_codes;
  p.next_scales = op.next_scales;
  p.next_scale_q = op.next_scale_q;
  p.tile_expert = plan.tile_expert;
  p.expert_offsets = plan.expert_offsets;
  p.scale_row_offsets = plan.scale_row_offsets;
  p.num_m_tiles = plan.num_m_tiles;
  p.tile_first = plan.tile_first;
  p.pair_tile = plan.pair_tile;
  p.num_pairs = plan.num_pairs;
  p.status = plan.status;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(sm_count & ~1));
  config.blockDim = dim3(kWpThreads);
  config.dynamicSmemBytes = kWpSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = op.serial_launch ? 1 : 2;
  WpTokenMaps token_maps;
  for (int i = 0; i < 16; ++i) token_maps.rows[i] = op.map_x[i];
  cudaLaunchKernelEx(&config, w13_geglu_pair_kernel, token_maps, op.map_w, op.map_x_sf, op.map_w_sf, p);
}

}  // namespace gv
