// Grouped block-scaled NVFP4 GEMM run by CTA pairs: tcgen05.mma.cta_group::2, M = 256 per pair.
//
// Why pairs.  With one CTA per 128 x 256 tile (grouped_gemm.cu) every K block of 256 elements
// brings 16 KiB of activations, 32 KiB of weights and 6 KiB of scales into the SM for 528 cycles
// of tensor work, and an SM takes in about 64 bytes per cycle from L2: the loads need about 840
// cycles, which is what a K block is measured to take there.  A CTA pair works on two 128-row
// tiles of the same expert against the same 256 weight rows; each CTA loads only its own half
// of the weight rows (the tensor cores of both SMs read both halves through the pair's shared
// memory), so an SM takes in 38 KiB per K block, and one MMA instruction drives both SMs.
//
// Work.  The route sort lists, beside the 128-row tiles, the tile pairs of every expert
// (plan.pair_tile); an expert with an odd number of tiles ends in a pair with one tile, whose
// second CTA loads its weight half and nothing else.  A work item is (pair, 256 weight rows);
// pairs of persistent CTAs (a cluster of two) take items in the order of grouped_gemm.cu.
//
// Protocol, per pipeline stage.  Every CTA runs its own two TMA producers into its own shared
// memory (tensor-map loads in their cta_group::2 form, no multicast), and all of them complete on
// the `full` barrier of the first CTA (the leader), whose producers announce the byte count of both
// CTAs' loads; the scale atoms travel through tensor maps too, because an untiled bulk copy can
// only signal a barrier of its own CTA.  The leader's MMA thread waits for `full`, copies the scale
// atoms of both CTAs into tensor memory (tcgen05.cp.cta_group::2 copies in each CTA from its own
// shared memory; copies and MMAs of one thread execute in order), issues the four MMAs and commits
// to `empty` of both CTAs (the commit's multicast form), and after the last K block to both
// `acc_full`.  The epilogue warps of both CTAs drain their own 128 accumulator rows exactly as in
// the single-CTA kernel and release the accumulator to the leader (the second CTA by remote
// arrives).  Tensor memory is allocated by each CTA for itself (all 512 columns, so both get the
// same addresses).  Every wait is bounded; a CTA that gives up still reaches the cluster barrier
// at the end, which keeps both CTAs resident until no remote arrive or copy can be in flight.
#include "gv_common.cuh"
#include "gv_gemm_parts.cuh"
#include "gv_launchers.h"

namespace gv {

namespace {

constexpr int kPairStages = 5;
constexpr int kPairWeightProducerWarp = 2 + 4 * kEpilogueWarpsPerQuarter;  // 18
constexpr int kPairThreads = (kPairWeightProducerWarp + 1) * 32;           // 608
constexpr uint32_t kPairTmemColumns = 512;
constexpr uint32_t kPairSfColumn = 256;        // accumulator: columns [0, 256)
constexpr uint32_t kPairSfColumnsPerStage = 48;  // per MMA j: A at +12j, B rows 0..127 at +12j+4, 128..255 at +12j+8
constexpr int kPairTileBytes = kTileM * kTileKBytes;  // 16 KiB

template <int kMode>
struct alignas(1024) PairSmem {
  uint8_t a[kPairStages][kPairTileBytes];        // this CTA's 128 activation rows
  uint8_t b[kPairStages][kPairTileBytes];        // this CTA's half (128) of the item's 256 weight rows
  uint8_t sfa[kPairStages][kSfStageBytes];       // scales of this CTA's rows
  uint8_t sfb[kPairStages][2 * kSfStageBytes];   // scales of all 256 weight rows
  uint8_t staging[4][kMode != kGeglu ? kStagingBytesPerWarp : 16];
  uint64_t full[kPairStages];       // leader: the stage's bytes have landed in both CTAs
  uint64_t empty[kPairStages];      // both CTAs: the MMAs that read the stage have completed
  uint64_t acc_full;                // both CTAs: the item's accumulator is complete
  uint64_t acc_empty;               // leader: both CTAs' epilogues have copied the accumulator out
  uint32_t tmem_base;
  volatile int abort;
  int quarter_left[4];
  alignas(16) float erf_table[GV_ERF_TABLE_FLOATS];
};

template <int kMode> constexpr size_t pair_smem_bytes() { return sizeof(PairSmem<kMode>) + 1024; }
static_assert(pair_smem_bytes<kPlain>() <= 232448 && pair_smem_bytes<kGeglu>() <= 232448, "shared memory budget");
static_assert(kPairSfColumn + kPairSfColumnsPerStage * kPairStages <= kPairTmemColumns, "tensor memory budget");

// Instruction descriptor of the pair MMA: E2M1 x E2M1, both K-major, UE4M3 scales, N = 256 at
// [17,23) in units of 8, M = 256 at [24,29) in units of 16, K = 64.
constexpr uint32_t kPairInstrDesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(256 >> 3) << 17) |
                                    (static_cast<uint32_t>(256 >> 4) << 24);

// ---- cluster-scope barrier operations ----------------------------------------------------
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* local_bar, uint32_t target_cta) {
  const uint32_t remote = cluster_map_shared(smem_u32(local_bar), target_cta);
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once every
// tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

// Tensor-map load into this CTA's shared memory that completes on a barrier of either CTA of the
// pair (`barrier` is a shared::cluster address).  No multicast: every CTA loads its own bytes.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tensor_map, uint32_t barrier, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(barrier)
      : "memory");
}

// Scale copies of one K block for both CTAs (each from its own shared memory at these offsets
// into its own tensor memory): per MMA j the A atom, and the two weight halves.
template <int kMmas>
__device__ __forceinline__ void issue_pair_sf_copies(uint32_t tmem_sf, uint32_t sfa_lo, uint32_t sfb_lo,
                                                     uint32_t hi_sf) {
#define GV_PSF_OPERANDS ::"r"(tmem_sf), "r"(sfa_lo), "r"(sfb_lo), "r"(hi_sf) : "memory"
#define GV_PSF_PROLOGUE "{\n\t.reg .b32 lo, ta;\n\t.reg .b64 d0;\n\t"
#define GV_PSF_ONE(source, source_offset, column)                            \
  "add.u32 lo, " source ", " source_offset ";\n\t"                           \
  "mov.b64 d0, {lo, %3};\n\t"                                                \
  "add.u32 ta, %0, " column ";\n\t"                                          \
  "tcgen05.cp.cta_group::2.32x128b.warpx4 [ta], d0;\n\t"
#define GV_PSF_COPY(j)                                                           \
  GV_PSF_ONE("%1", #j "*32", #j "*12") GV_PSF_ONE("%2", #j "*32", "4+" #j "*12") \
  GV_PSF_ONE("%2", "128+" #j "*32", "8+" #j "*12")
  asm volatile(GV_PSF_PROLOGUE GV_PSF_COPY(0) "}" GV_PSF_OPERANDS);
  if constexpr (kMmas >= 2) asm volatile(GV_PSF_PROLOGUE GV_PSF_COPY(1) "}" GV_PSF_OPERANDS);
  if constexpr (kMmas >= 3) asm volatile(GV_PSF_PROLOGUE GV_PSF_COPY(2) "}" GV_PSF_OPERANDS);
  if constexpr (kMmas >= 4) asm volatile(GV_PSF_PROLOGUE GV_PSF_COPY(3) "}" GV_PSF_OPERANDS);
#undef GV_PSF_COPY
#undef GV_PSF_ONE
#undef GV_PSF_PROLOGUE
#undef GV_PSF_OPERANDS
}

template <int kMmas>
__device__ __forceinline__ void issue_pair_mmas(uint32_t tmem_acc, uint32_t tmem_sf, uint32_t a_lo, uint32_t b_lo,
                                                uint32_t hi_ab, uint32_t accumulate) {
#define GV_PM_OPERANDS                                                                                    \
  ::"r"(tmem_acc), "r"(tmem_sf), "r"(a_lo), "r"(b_lo), "r"(hi_ab), "r"(kPairInstrDesc), "r"(accumulate) \
  : "memory"
#define GV_PM_PROLOGUE "{\n\t.reg .pred p, pt;\n\t.reg .b32 lo, ta, tb;\n\t.reg .b64 d0, d1;\n\t" \
                       "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
#define GV_PM_MMA(j, pred)                                                 \
  "add.u32 lo, %2, " #j "*2;\n\t"                                          \
  "mov.b64 d0, {lo, %4};\n\t"                                              \
  "add.u32 lo, %3, " #j "*2;\n\t"                                          \
  "mov.b64 d1, {lo, %4};\n\t"                                              \
  "add.u32 ta, %1, " #j "*12;\n\t"                                         \
  "add.u32 tb, %1, " #j "*12+4;\n\t"                                       \
  "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"      \
  " [%0], d0, d1, %5, [ta], [tb], " pred ";\n\t"
  asm volatile(GV_PM_PROLOGUE GV_PM_MMA(0, "p") "}" GV_PM_OPERANDS);
  if constexpr (kMmas >= 2) asm volatile(GV_PM_PROLOGUE GV_PM_MMA(1, "pt") "}" GV_PM_OPERANDS);
  if constexpr (kMmas >= 3) asm volatile(GV_PM_PROLOGUE GV_PM_MMA(2, "pt") "}" GV_PM_OPERANDS);
  if constexpr (kMmas >= 4) asm volatile(GV_PM_PROLOGUE GV_PM_MMA(3, "pt") "}" GV_PM_OPERANDS);
#undef GV_PM_MMA
#undef GV_PM_PROLOGUE
#undef GV_PM_OPERANDS
}

// An epilogue thread has its share of the accumulator in registers: the leader's threads arrive
// on the leader's barrier themselves, a warp of the second CTA sends one remote arrive.
template <class Smem>
__device__ __forceinline__ void release_accumulator(Smem* smem, bool is_leader, int lane) {
  if (is_leader) {
    mbar_arrive(&smem->acc_empty);
  } else {
    __syncwarp();
    if (lane == 0) mbar_arrive_remote(&smem->acc_empty, 0);
  }
}

struct PairItem {
  int first;     // the pair's first tile (always exists; names the expert)
  int tile;      // this CTA's 128-row tile, or -1 (second CTA of a pair with one tile)
  int n_tile;
};

// Items in snake order over the pairs of the grid (see work_item in grouped_gemm.cu).
__device__ __forceinline__ bool pair_item(int round, int total_items, int n_tiles, int pair_begin,
                                          const int* __restrict__ pair_tile, uint32_t rank, PairItem& item) {
  const int slots = static_cast<int>(gridDim.x) >> 1;
  const int mine = static_cast<int>(blockIdx.x) >> 1;
  const int slot = (round & 1) ? slots - 1 - mine : mine;
  const int index = round * slots + slot;
  if (index >= total_items) return false;
  const int pair = index / n_tiles;
  item.n_tile = index - pair * n_tiles;
  const int entry = pair_tile[pair_begin + pair];
  const int first = entry >> 1;
  item.first = first;
  item.tile = rank == 0 ? first : ((entry & 1) ? first + 1 : -1);
  return true;
}

__device__ __forceinline__ int pair_lower_bound(const int* __restrict__ pair_tile, int count, int tile) {
  int lo = 0, hi = count;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if ((pair_tile[mid] >> 1) < tile) lo = mid + 1; else hi = mid;
  }
  return lo;
}

template <int kMode>
__global__ void __launch_bounds__(kPairThreads, 1)
grouped_nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a32,
                               const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b64,
                               const __grid_constant__ CUtensorMap map_a_sf,
                               const __grid_constant__ CUtensorMap map_b_sf, const GemmParams p, const int* __restrict__ pair_tile,
                               const int* __restrict__ num_pairs) {
  using Smem = PairSmem<kMode>;
  extern __shared__ uint8_t smem_raw[];
  Smem* smem = reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();   // 0 = leader
  const bool is_leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&smem->full[s], 2);       // one arrival (with both CTAs' byte count) per producer warp of the leader
      mbar_init(&smem->empty[s], 1);
    }
    mbar_init(&smem->acc_full, 1);
    mbar_init(&smem->acc_empty, kEpilogueThreads + kEpilogueThreads / 32);  // leader's threads + the second CTA's warps
    smem->abort = 0;
    for (int s = 0; s < 4; ++s) smem->quarter_left[s] = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_a32);
    prefetch_tensor_map(&map_b);
    if (kMode == kGeglu) prefetch_tensor_map(&map_b64);
    prefetch_tensor_map(&map_a_sf);
    prefetch_tensor_map(&map_b_sf);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kPairTmemColumns);  // the whole tensor memory: both CTAs get address 0
    tmem_relinquish();
  }
  if (kMode == kGeglu) load_erf_table(smem->erf_table);
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // Barriers of both CTAs exist before either CTA arrives on the other's.
  cluster_sync_all();
  const uint32_t tmem_base = smem->tmem_base;
  grid_dependency_wait();

  int pair_begin = 0, pair_count = num_pairs[0];
  if (p.tile_first) {
    const int first = p.tile_first[0];
    pair_begin = pair_lower_bound(pair_tile, pair_count, first);
    pair_count = pair_lower_bound(pair_tile, pair_count, first + p.num_m_tiles[0]) - pair_begin;
  }
  const int total_items = pair_count * p.n_tiles;
  const int slots = static_cast<int>(gridDim.x) >> 1;
  const int rounds = (total_items + slots - 1) / slots;

  if (warp == 0 || warp == kPairWeightProducerWarp) {
    // ---------------- TMA producers (both CTAs) ----------------
    const bool weight_side = warp == kPairWeightProducerWarp;
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    const int atoms_per_block = p.groups >> 2;  // 512-byte scale atoms of one 128-row block
    for (int round = 0; ok && round < rounds; ++round) {
      PairItem item;
      if (!pair_item(round, total_items, p.n_tiles, pair_begin, pair_tile, rank, item)) continue;
      const int n_tile = item.n_tile;
      const int expert = p.tile_expert[item.first];
      int row = 0, sf_row = 0, sf_row2 = 0;
      uint32_t my_bytes = 0, both_bytes = 0;   // per K block: this CTA's loads; the leader's and the second CTA's
      bool short_tile = false, half_item = false;
      if (!weight_side) {
        // activation rows: tile `first` in the leader, `first + 1` (if the pair has it) in the second CTA
        const int local0 = item.first * kTileM - p.scale_row_offsets[expert];
        const int rows_after = p.expert_offsets[expert + 1] - p.expert_offsets[expert] - local0;  // from the first tile on
        const bool second_exists = rows_after > kTileM;
        const uint32_t leader_bytes = (rows_after <= 32 ? kPairTileBytes / 4 : kPairTileBytes) + kSfStageBytes;
        const uint32_t second_bytes =
            second_exists ? (rows_after - kTileM <= 32 ? kPairTileBytes / 4 : kPairTileBytes) + kSfStageBytes : 0u;
        both_bytes = leader_bytes + second_bytes;
        my_bytes = is_leader ? leader_bytes : second_bytes;
        if (item.tile >= 0) {
          row = p.expert_offsets[expert] + (item.tile * kTileM - p.scale_row_offsets[expert]);
          short_tile = p.expert_offsets[expert + 1] - row <= 32;
          sf_row = item.tile * atoms_per_block;
        }
      } else if (kMode == kGeglu) {
        // leader: up rows [128 j, +128); second CTA: gate rows [704 + 128 j, +128); the sixth item
        // of a row tile has 64 of each left (64-row box; the rest of the half keeps stale bytes,
        // its scales are zero in the re-tiled copy and the epilogue drops its columns)
        row = expert * kW13Out + n_tile * 128 + (is_leader ? 0 : kInter);
        half_item = (n_tile + 1) * 128 > kInter;
        sf_row = (expert * p.n_tiles + n_tile) * 2 * atoms_per_block;  // 8 atoms per K block
        my_bytes = (half_item ? kPairTileBytes / 2 : kPairTileBytes) + 2 * kSfStageBytes;
        both_bytes = 2 * my_bytes;
      } else {
        row = expert * p.n_out + n_tile * 256 + (is_leader ? 0 : 128);
        sf_row = ((expert * p.n_out + n_tile * 256) >> 7) * atoms_per_block;
        sf_row2 = sf_row + atoms_per_block;
        my_bytes = kPairTileBytes + 2 * kSfStageBytes;
        both_bytes = 2 * my_bytes;
      }
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, wait_or_abort<true>(&smem->empty[stage], phase ^ 1u, smem, p.status));
        if (!ok) break;
        if (elect_one()) {
          const int x = kb * kTileKBytes;
          const uint32_t bar = is_leader ? smem_u32(&smem->full[stage])
                                         : cluster_map_shared(smem_u32(&smem->full[stage]), 0);
          if (is_leader) mbar_arrive_expect_tx(&smem->full[stage], both_bytes);
          if (my_bytes == 0) {
            // second CTA of a pair with one tile: no activation rows
          } else if (!weight_side) {
            tma_load_2d_pair(smem->a[stage], short_tile ? &map_a32 : &map_a, bar, x, row);
            tma_load_2d_pair(smem->sfa[stage], &map_a_sf, bar, 0, sf_row + 4 * kb);
          } else if (kMode == kGeglu) {
            tma_load_2d_pair(smem->b[stage], half_item ? &map_b64 : &map_b, bar, x, row);
            // re-tiled scales: [rows 0..127 | rows 128..255] x four MMAs, 4 KiB per K block
            tma_load_2d_pair(smem->sfb[stage], &map_b_sf, bar, 0, sf_row + 8 * kb);
          } else {
            tma_load_2d_pair(smem->b[stage], &map_b, bar, x, row);
            tma_load_2d_pair(smem->sfb[stage], &map_b_sf, bar, 0, sf_row + 4 * kb);
            tma_load_2d_pair(smem->sfb[stage] + kSfStageBytes, &map_b_sf, bar, 0, sf_row2 + 4 * kb);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok && lane == 0 && is_leader) {
      // Unwinding: let the copies already issued (by either CTA) land before shared memory is
      // given up; the second CTA stays resident until the cluster barrier at the end.
      const int pending = issued < kPairStages ? issued : kPairStages;
      int s = stage;
      uint32_t ph = phase;
      for (int i = 0; i < pending; ++i) {
        if (--s < 0) {
          s = kPairStages - 1;
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
      const uint32_t a_lo0 = (smem_u32(smem->a[0]) & 0x3ffffu) >> 4;
      const uint32_t b_lo0 = (smem_u32(smem->b[0]) & 0x3ffffu) >> 4;
      const uint32_t sfa_lo0 = (smem_u32(smem->sfa[0]) & 0x3ffffu) >> 4;
      const uint32_t sfb_lo0 = (smem_u32(smem->sfb[0]) & 0x3ffffu) >> 4;
      constexpr uint32_t hi_ab = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8 rows x 128 B, 128B swizzle
      constexpr uint32_t hi_sf = (128u >> 4) | (1u << 14);                // 8 rows x 16 B, no swizzle
      const bool full_last = p.last_mmas == 4;
      const bool leader_lane = elect_one();
      for (int round = 0; round < rounds; ++round) {
        PairItem item;
        if (!pair_item(round, total_items, p.n_tiles, pair_begin, pair_tile, rank, item)) continue;
        if (!__all_sync(0xffffffffu, wait_or_abort<false>(&smem->acc_empty, acc_phase ^ 1u, smem, p.status))) break;
        acc_phase ^= 1u;
        bool ok = true;
        tc_fence_after_sync();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = wait_or_abort<false>(&smem->full[stage], phase, smem, p.status);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (kPairTileBytes >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (kPairTileBytes >> 4);
          const uint32_t sfa_lo = sfa_lo0 + static_cast<uint32_t>(stage) * (kSfStageBytes >> 4);
          const uint32_t sfb_lo = sfb_lo0 + static_cast<uint32_t>(stage) * (2 * kSfStageBytes >> 4);
          const uint32_t tmem_sf = tmem_base + kPairSfColumn + kPairSfColumnsPerStage * stage;
          if (leader_lane) {
            const uint32_t accumulate = kb != 0 ? 1u : 0u;
            if (kb != p.k_blocks - 1 || full_last) {
              issue_pair_sf_copies<4>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
              issue_pair_mmas<4>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
            } else if (p.last_mmas == 3) {
              issue_pair_sf_copies<3>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
              issue_pair_mmas<3>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
            } else if (p.last_mmas == 2) {
              issue_pair_sf_copies<2>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
              issue_pair_mmas<2>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
            } else {
              issue_pair_sf_copies<1>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
              issue_pair_mmas<1>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
            }
            tc_commit_pair(&smem->empty[stage]);   // both CTAs may refill the stage
            if (kb + 1 == p.k_blocks) tc_commit_pair(&smem->acc_full);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else {
    // ---------------- epilogue: 16 warps in each CTA, its own 128 accumulator rows ----------------
    const int quarter = warp & 3;
    const int sub = (warp - 2) >> 2;  // 0..3
    uint32_t acc_phase = 0;
    uint8_t* staging = smem->staging[quarter];
    for (int round = 0; round < rounds; ++round) {
      PairItem item;
      if (!pair_item(round, total_items, p.n_tiles, pair_begin, pair_tile, rank, item)) continue;
      const int m_tile = item.tile;
      const int n_tile = item.n_tile;
      int expert = 0, row0 = 0, rows_valid = 0;
      float alpha = 0.0f;
      if (m_tile >= 0) {
        expert = p.tile_expert[m_tile];
        const int local0 = m_tile * kTileM - p.scale_row_offsets[expert];
        row0 = p.expert_offsets[expert] + local0;
        rows_valid = p.expert_offsets[expert + 1] - row0;  // may exceed 128
        alpha = p.alpha[expert];
      }
      const bool acc_ready = wait_or_abort<true>(&smem->acc_full, acc_phase, smem, p.status);
      acc_phase ^= 1u;
      if constexpr (kMode != kGeglu) {
        if (!acc_ready) smem->quarter_left[quarter] = 1;
        named_barrier(1 + quarter, kEpilogueWarpsPerQuarter * 32);
        if (*reinterpret_cast<volatile int*>(&smem->quarter_left[quarter])) break;
      } else {
        if (!acc_ready) break;
      }
      tc_fence_after_sync();
      const int row_local = quarter * 32 + lane;
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (kMode != kGeglu) {
        uint32_t r0[32], r1[32];
        if (m_tile >= 0) {
          tmem_load_32x32(tmem_row + sub * 32, r0);
          tmem_load_32x32(tmem_row + kStoreColumns + sub * 32, r1);
          tmem_load_wait();
        }
        tc_fence_before_sync();
        release_accumulator(smem, is_leader, lane);
        if (m_tile >= 0 && quarter * 32 < rows_valid) {
          stage_and_store(r0, alpha, staging, quarter, sub, lane, rows_valid, row0, n_tile * 256, p);
          stage_and_store(r1, alpha, staging, quarter, sub, lane, rows_valid, row0, n_tile * 256 + kStoreColumns, p);
        }
      } else {
        // accumulator columns [0,128) are up and [128,256) gate of intermediate columns
        // [128 n_tile, +128); this warp owns the 16-column blocks 2 sub and 2 sub + 1 of them
        uint32_t up0[16], gate0[16], up1[16], gate1[16];
        if (m_tile >= 0) {
          tmem_load_32x16(tmem_row + sub * 32, up0);
          tmem_load_32x16(tmem_row + 128 + sub * 32, gate0);
          tmem_load_32x16(tmem_row + sub * 32 + 16, up1);
          tmem_load_32x16(tmem_row + 128 + sub * 32 + 16, gate1);
          tmem_load_wait();
        }
        tc_fence_before_sync();
        release_accumulator(smem, is_leader, lane);
        const bool columns_exist = n_tile * 128 + sub * 32 < kInter;  // the last item is half empty
        if (m_tile >= 0 && row_local < rows_valid && columns_exist) {
          const float multiplier = p.next_scale_q[expert];
          uint4 codes;
          const uint32_t scale0 = geglu_block(up0, gate0, alpha, multiplier, smem->erf_table, codes.x, codes.y);
          const uint32_t scale1 = geglu_block(up1, gate1, alpha, multiplier, smem->erf_table, codes.z, codes.w);
          *reinterpret_cast<uint4*>(p.next_codes + static_cast<size_t>(row0 + row_local) * (kInter / 2) +
                                    n_tile * 64 + sub * 16) = codes;
          constexpr int groups = kInter / 16;
          *reinterpret_cast<uint16_t*>(p.next_scales + static_cast<size_t>(m_tile) * kTileM * groups +
                                       sf_offset(row_local, 8 * n_tile + 2 * sub, groups)) =
              static_cast<uint16_t>(scale0 | (scale1 << 8));
        }
      }
    }
  }

  tc_fence_before_sync();
  // Both CTAs stay until neither can still receive a remote arrive or a multicast commit.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, kPairTmemColumns);
  }
}

template <int kMode>
cudaError_t launch_pair_variant(const GemmOperands& op, const GemmParams& p, const RoutePlan& plan, int sm_count,
                                cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(sm_count & ~1));
  config.blockDim = dim3(kPairThreads);
  config.dynamicSmemBytes = pair_smem_bytes<kMode>();
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
  return cudaLaunchKernelEx(&config, grouped_nvfp4_gemm_pair_kernel<kMode>, op.map_a, op.map_a32, op.map_b,
                            op.map_b64, op.map_a_sf, op.map_b_sf, p, static_cast<const int*>(plan.pair_tile),
                            static_cast<const int*>(plan.num_pairs));
}

}  // namespace

int prepare_grouped_gemm_pairs() {
  cudaError_t e = cudaFuncSetAttribute(grouped_nvfp4_gemm_pair_kernel<kPlain>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(pair_smem_bytes<kPlain>()));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(grouped_nvfp4_gemm_pair_kernel<kGeglu>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(pair_smem_bytes<kGeglu>()));
  return static_cast<int>(e);
}

void launch_grouped_gemm_pairs(const GemmOperands& op, const RoutePlan& plan, int sm_count, cudaStream_t stream) {
  GemmParams p{};
  p.a_scales = op.a_scales;
  p.b_scales = op.b_scales;
  p.alpha = op.alpha;
  p.out = static_cast<__nv_bfloat16*>(op.out);
  p.row_dest = op.row_dest;
  p.next_codes = op.next_codes;
  p.next_scales = op.next_scales;
  p.next_scale_q = op.next_scale_q;
  p.tile_expert = plan.tile_expert;
  p.expert_offsets = plan.expert_offsets;
  p.scale_row_offsets = plan.scale_row_offsets;
  p.num_m_tiles = plan.num_m_tiles;
  p.tile_first = plan.tile_first;
  p.status = plan.status;
  p.n_out = op.n_out;
  const int k_bytes = op.k_in / 2;
  p.groups = op.k_in / 16;
  p.k_blocks = (k_bytes + kTileKBytes - 1) / kTileKBytes;
  p.last_mmas = (k_bytes - (p.k_blocks - 1) * kTileKBytes) / 32;
  if (op.fused_geglu) {
    p.n_tiles = kFusedItems;
    launch_pair_variant<kGeglu>(op, p, plan, sm_count, stream);
  } else {
    p.n_tiles = op.n_out / 256;
    launch_pair_variant<kPlain>(op, p, plan, sm_count, stream);
  }
}

}  // namespace gv
