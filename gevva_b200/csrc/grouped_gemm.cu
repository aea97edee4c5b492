// Grouped block-scaled NVFP4 GEMM for sm_100a: tcgen05.mma kind::mxf4nvf4 with
// UE4M3 scales per 16 elements, fp32 accumulators in tensor memory, operands
// brought in by TMA into 128-byte-swizzled shared memory.
//
// Replaces the reference's CUTLASS SM120 grouped GEMM
// (src/nvfp4_cutlass.cu:81-100 traits, :755-962 plan, :913-930 run):
//   D_e[r, n] = bf16(alpha[e] * sum_k A[r,k] sfa[r,k/16] B_e[n,k] sfb_e[n,k/16])
// for the rows r of each expert e, over all 128 experts in one launch, and, in its
// fused form, also the reference's geglu_quantize_sorted_moe (:552-601) applied to
// the accumulators before anything is written.
//
// Mapping.  Tokens (sorted routes) sit on MMA-M, weight rows on MMA-N.  A work
// item is (128-row tile of one expert) x (kN weight rows), kN = 256 for the two expert
// GEMMs and 128 elsewhere.  The main loop is bound by how fast one thread can issue
// tcgen05 instructions (about 90 cycles per MMA with its scale copies, against 64 cycles
// of tensor-pipe time at N = 128), so the wide tile, which does twice the work per
// instruction, is what keeps the tensor pipe fed.  Row tiles are listed
// in device memory by the route sort; CTAs are persistent and take items
// round-robin.  Warps 0 and 18 are the TMA producers (activation side, weight side),
// warp 1 allocates tensor memory and issues the MMAs, warps 2..17 drain accumulators (two
// accumulator stages at N = 128; at N = 256 one, which the epilogue copies to registers and
// releases before it does its arithmetic, so the epilogue of one item still overlaps the
// main loop of the next).  Warps 0 and 1 walk
// their loops as whole warps (warp-uniform addresses) and one elected lane issues.
//
// Two epilogues:
//   kPlain  bf16(alpha*acc), staged through shared memory so that every global
//           store instruction writes two full 256-byte row segments;
//   kGeglu  the 256 weight rows of an item are up rows [128j,128j+128) and gate rows
//           [704+128j, 704+128j+128) of w13 (the sixth item of a row tile is half empty),
//           so a thread holds up and gate of the same columns: v = gelu_erf(bf16(gate)) *
//           bf16(up), two 16-value blocks per thread -> 16 code bytes and two scale bytes,
//           written straight into the w2 operand buffers.  The bf16 w13 output never
//           exists in memory.
//
// Scale factors.  Both operands keep scales in the 128-row x 4-scale atoms of
// 512 bytes (row%32)*16 + (row/32)*4 + k that the reference writes
// (src/nvfp4_cutlass.cu:321-323); one atom is exactly what one MMA (K = 64)
// consumes and what tcgen05.cp 32x128b.warpx4 moves, so a K block of 256 needs a
// contiguous 2 KiB per operand, fetched with one untiled bulk copy.  For kGeglu the
// weight scales come from a copy re-tiled once at runner creation so that the
// [128 up | 128 gate] rows of an item form such atoms (retile_w13_scales_kernel below).
//
// Every wait is bounded: on expiry the kernel records kWaitTimeout in the status
// word, all roles leave their loops, tensor memory is released and the CTA exits.
#include "gv_common.cuh"
#include "gv_gemm_parts.cuh"
#include "gv_launchers.h"

namespace gv {

namespace {

// Warp roles: 0 = producer of the activation side (A + its scales), 1 = MMA issuer,
// 2..17 = epilogue, 18 = producer of the weight side (B + its scales), 19 = scale-factor
// copier.  Two producers because one thread cannot issue a K block's copies in the time its
// MMAs take; a copier of its own because a thread needs about 34 cycles per tcgen05
// instruction: the twelve shared -> tensor memory scale copies of a K block plus its four
// MMAs in one thread take longer than the 528 cycles the tensor pipe needs for them, whereas
// four MMAs in one thread and twelve copies in another both fit.
constexpr int kWeightProducerWarp = 2 + 4 * kEpilogueWarpsPerQuarter;
constexpr int kScaleCopyWarp = kWeightProducerWarp + 1;
constexpr int kGemmThreads = (kScaleCopyWarp + 1) * 32;
constexpr uint32_t kTmemColumns = 512;
// Accumulators take tensor-memory columns [0, 256) in every configuration (2 x 128 or
// 1 x 256); scale factors follow, per pipeline stage and K block: a copy for the next K
// block must not wait for the MMAs of the previous one to finish reading theirs.
constexpr uint32_t kSfColumn = 256;
constexpr int kOperandStageBytes = kTileM * kTileKBytes;  // 16 KiB: 128 rows of one K block
// A pipeline stage holds kAtoms K blocks of 256 elements (one 128-byte swizzle row each) of
// 128 activation rows and kN weight rows.  At N = 256 a stage is 54 KiB, so four stages fit
// (three beside the store staging of the plain epilogue); at N = 128 five.
template <int kMode, int kAtomsPerStage, int kN> struct StageShape {
  static_assert(kN == 128 || kN == 256, "weight rows per item");
  static_assert(kN == 128 || kAtomsPerStage == 1, "wide tiles take one K block per stage");
  static constexpr int kAtoms = kAtomsPerStage;
  static constexpr int kStages =
      kN == 256 ? (kMode == kGeglu ? 4 : 3) : 5;
  static constexpr int kAccStages = kN == 256 ? 1 : 2;
  static constexpr int kWeightBytes = kN * kTileKBytes;        // per K block
  static constexpr int kWeightSfBytes = (kN / 128) * kSfStageBytes;
  // Scale-factor columns per K block: at N = 128 sixteen for A then sixteen for B; at N = 256
  // sixteen per MMA (A at +0, B rows 0..127 at +4, B rows 128..255 at +8).
  static constexpr uint32_t kSfColumns = kN == 256 ? 64 : 32;
};

template <int kMode, int kAtomsPerStage, int kN>
struct alignas(1024) GemmSmem {
  using Shape = StageShape<kMode, kAtomsPerStage, kN>;
  static constexpr int kAtoms = Shape::kAtoms;
  static constexpr int kStages = Shape::kStages;
  static constexpr int kAccStages = Shape::kAccStages;
  uint8_t a[kStages][kAtoms * kOperandStageBytes];
  uint8_t b[kStages][kAtoms * Shape::kWeightBytes];
  uint8_t sfa[kStages][kAtoms * kSfStageBytes];
  uint8_t sfb[kStages][kAtoms * Shape::kWeightSfBytes];
  uint8_t staging[4][kMode != kGeglu ? kStagingBytesPerWarp : 16];  // plain epilogue only
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t sf_full[kStages];  // the stage's scale factors have reached tensor memory
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint32_t tmem_base;
  volatile int abort;
  int quarter_left[4];  // plain epilogue: a warp of this quarter gave up waiting
  alignas(16) float erf_table[GV_ERF_TABLE_FLOATS];
};

template <int kMode, int kAtoms, int kN> constexpr size_t gemm_smem_bytes() {
  return sizeof(GemmSmem<kMode, kAtoms, kN>) + 1024;
}
static_assert(gemm_smem_bytes<kPlain, 1, 128>() <= 232448 && gemm_smem_bytes<kPlain, 1, 256>() <= 232448 &&
                  gemm_smem_bytes<kGeglu, 1, 256>() <= 232448 && gemm_smem_bytes<kFp8, 1, 128>() <= 232448,
              "shared memory budget of one sm_100 CTA");
static_assert(kSfColumn + 64 * 4 <= kTmemColumns && kSfColumn + 32 * 6 <= kTmemColumns, "tensor memory budget");

// Dense FP8 form of the same: kMmas MMAs of K = 32 E4M3 elements (32 bytes, the same
// descriptor step), no scale factors.  Instruction descriptor: fp32 accumulate (bit 4),
// E4M3 x E4M3 (format 0), both K-major, N and M as above.
constexpr uint32_t kInstrDescFp8 = (1u << 4) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
                                   (static_cast<uint32_t>(kTileM >> 4) << 24);

template <int kMmas>
__device__ __forceinline__ void issue_k_block_fp8(uint32_t tmem_acc, uint32_t a_lo, uint32_t b_lo,
                                                  uint32_t hi_ab, uint32_t accumulate) {
#define GV_MMA8(j, pred)                                                   \
  "add.u32 lo, %1, " #j "*2;\n\t"                                          \
  "mov.b64 d0, {lo, %3};\n\t"                                              \
  "add.u32 lo, %2, " #j "*2;\n\t"                                          \
  "mov.b64 d1, {lo, %3};\n\t"                                              \
  "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], d0, d1, %4, " pred ";\n\t"
#define GV_OPERANDS8 ::"r"(tmem_acc), "r"(a_lo), "r"(b_lo), "r"(hi_ab), "r"(kInstrDescFp8), "r"(accumulate) : "memory"
#define GV_PROLOGUE8 "{\n\t.reg .pred p, pt;\n\t.reg .b32 lo;\n\t.reg .b64 d0, d1;\n\t" \
                     "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
  asm volatile(GV_PROLOGUE8 GV_MMA8(0, "p") "}" GV_OPERANDS8);
  if constexpr (kMmas >= 2) asm volatile(GV_PROLOGUE8 GV_MMA8(1, "pt") "}" GV_OPERANDS8);
  if constexpr (kMmas >= 3) asm volatile(GV_PROLOGUE8 GV_MMA8(2, "pt") "}" GV_OPERANDS8);
  if constexpr (kMmas >= 4) asm volatile(GV_PROLOGUE8 GV_MMA8(3, "pt") "}" GV_OPERANDS8);
#undef GV_MMA8
#undef GV_OPERANDS8
#undef GV_PROLOGUE8
}


// Work distribution.  Items are dealt to the persistent CTAs in snake order: round r goes to
// CTA b as item r*G + b for even r and r*G + (G-1-b) for odd r.  In a short launch of the fused
// wide form (at most eight rounds) the items are numbered with the expensive ones first, the
// half-filled last item of every row tile after all full ones: that is the longest-first
// rule, which is what balances a decode-sized launch (768 items of two sizes over 148 CTAs).
struct WorkItem {
  int m_tile;
  int n_tile;
};

template <int kMode, int kN>
__device__ __forceinline__ bool work_item(int round, int total_items, int m_tiles, int n_tiles,
                                          int tile_first, WorkItem& item) {
  const int grid = static_cast<int>(gridDim.x);
  const int slot = (round & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int index = round * grid + slot;
  if (index >= total_items) return false;
  // Cost order only where balance decides (a few rounds); a long launch keeps the items of a
  // row tile together so that its activation tile is still in L2 for the last one.
  if (kMode == kGeglu && kN == 256 && total_items <= 8 * grid) {
    const int full = m_tiles * (n_tiles - 1);
    if (index < full) {
      item.m_tile = index / (n_tiles - 1);
      item.n_tile = index - item.m_tile * (n_tiles - 1);
    } else {
      item.m_tile = index - full;
      item.n_tile = n_tiles - 1;
    }
  } else {
    item.m_tile = index / n_tiles;
    item.n_tile = index - item.m_tile * n_tiles;
  }
  item.m_tile += tile_first;
  return true;
}

template <int kMode, int kAtomsPerStage, int kN>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_a32,
                          const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_b64, const GemmParams p) {
  using Smem = GemmSmem<kMode, kAtomsPerStage, kN>;
  using Shape = typename Smem::Shape;
  constexpr int kStages = Smem::kStages;
  constexpr int kAtoms = Smem::kAtoms;
  constexpr int kAccStages = Smem::kAccStages;
  constexpr bool kWide = kN == 256;
  static_assert(kMode != kFp8 || !kWide, "the dense path uses 128-row weight tiles");
  static_assert(kMode != kGeglu || kWide, "the fused form exists for 256-row weight tiles only");
  extern __shared__ uint8_t smem_raw[];
  Smem* smem = reinterpret_cast<Smem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&smem->full[s], 2);  // one arrival (with its byte count) per producer warp
      mbar_init(&smem->empty[s], 1);
      mbar_init(&smem->sf_full[s], 1);
    }
    for (int s = 0; s < 4; ++s) smem->quarter_left[s] = 0;
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&smem->acc_full[s], 1);
      mbar_init(&smem->acc_empty[s], kEpilogueThreads);
    }
    smem->abort = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_a32);
    prefetch_tensor_map(&map_b);
    if (kMode == kGeglu) prefetch_tensor_map(&map_b64);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  if (kMode == kGeglu) load_erf_table(smem->erf_table);
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = smem->tmem_base;
  // Everything above touched only this CTA's shared and tensor memory; from here on the
  // kernel reads what earlier kernels of the stream wrote.
  grid_dependency_wait();

  const int m_tiles = p.num_m_tiles[0];
  const int tile_first = p.tile_first ? p.tile_first[0] : 0;
  const int total_items = m_tiles * p.n_tiles;
  const int rounds = (total_items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  if (warp == 0 || warp == kWeightProducerWarp) {
    // ---------------- TMA producers ----------------
    const bool weight_side = warp == kWeightProducerWarp;
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int round = 0; ok && round < rounds; ++round) {
      WorkItem item;
      if (!work_item<kMode, kN>(round, total_items, m_tiles, p.n_tiles, tile_first, item)) continue;
      const int m_tile = item.m_tile;
      const int n_tile = item.n_tile;
      const int expert = p.tile_expert[m_tile];
      int row = 0, row2 = 0;
      const uint8_t* sf_src;
      const uint8_t* sf_src2 = nullptr;  // wide plain tiles: scales of weight rows 128..255
      bool short_tile = false;  // decode-sized groups: fetch 32 activation rows instead of 128
      bool half_item = false;   // fused wide tiles: the last item of a row tile has 64 up and 64 gate rows
      if (!weight_side) {
        row = p.expert_offsets[expert] + (m_tile * kTileM - p.scale_row_offsets[expert]);
        short_tile = p.expert_offsets[expert + 1] - row <= 32;
        sf_src = p.a_scales + static_cast<size_t>(m_tile) * kTileM * p.groups;
      } else if (kMode == kGeglu) {
        // up rows; the gate rows lie kInter further on.  The last item of a row tile has only
        // 64 up and 64 gate rows left: only those are fetched (64-row boxes); the rest of each
        // 128-row half keeps whatever the stage held, its scales are zero in the re-tiled copy
        // and its columns are dropped by the epilogue.
        row = expert * kW13Out + n_tile * (kN / 2);
        row2 = row + kInter;
        half_item = kWide && (n_tile + 1) * (kN / 2) > kInter;
        sf_src = p.b_scales + (static_cast<size_t>(expert) * p.n_tiles + n_tile) * kN * p.groups;
      } else {
        row = expert * p.n_out + n_tile * kN;
        row2 = row + 128;
        sf_src = p.b_scales + static_cast<size_t>(row) * p.groups;
        sf_src2 = sf_src + static_cast<size_t>(128) * p.groups;
      }
      for (int kb = 0; kb < p.k_blocks; kb += kAtoms) {
        ok = __all_sync(0xffffffffu, wait_or_abort<true>(&smem->empty[stage], phase ^ 1u, smem, p.status));
        if (!ok) break;
        if (elect_one()) {
          const int atoms = p.k_blocks - kb < kAtoms ? p.k_blocks - kb : kAtoms;
          const bool has_last = kb + atoms == p.k_blocks;
          const uint32_t sf_bytes =
              kMode == kFp8 ? 0u
                            : static_cast<uint32_t>((atoms - 1) * 4 + (has_last ? p.last_mmas : 4)) * kSfAtomBytes;
          uint32_t expected;
          if (!weight_side)
            expected = atoms * (short_tile ? kOperandStageBytes / 4 : kOperandStageBytes) + sf_bytes;
          else if (kWide && kMode == kGeglu)
            expected = (half_item ? Shape::kWeightBytes / 2 : Shape::kWeightBytes) + Shape::kWeightSfBytes;
          else
            expected = atoms * Shape::kWeightBytes + (kWide ? 2u : 1u) * sf_bytes;
          mbar_arrive_expect_tx(&smem->full[stage], expected);
#pragma unroll
          for (int atom = 0; atom < kAtoms; ++atom) {
            if (atom >= atoms) break;
            const int x = (kb + atom) * kTileKBytes;
            if (!weight_side) {
              tma_load_2d(smem->a[stage] + atom * kOperandStageBytes, short_tile ? &map_a32 : &map_a,
                          &smem->full[stage], x, row);
            } else if (kWide) {
              const CUtensorMap* map = half_item ? &map_b64 : &map_b;
              tma_load_2d(smem->b[stage], map, &smem->full[stage], x, row);
              tma_load_2d(smem->b[stage] + kOperandStageBytes, map, &smem->full[stage], x, row2);
            } else {
              tma_load_2d(smem->b[stage] + atom * kOperandStageBytes, &map_b, &smem->full[stage], x, row);
            }
          }
          if (kMode != kFp8) {
            if (!weight_side) {
              bulk_load_1d(smem->sfa[stage], sf_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes,
                           &smem->full[stage]);
            } else if (kWide && kMode == kGeglu) {
              // re-tiled scales: [rows 0..127 | rows 128..255] x four MMAs, 4 KiB per K block
              bulk_load_1d(smem->sfb[stage], sf_src + static_cast<size_t>(kb) * Shape::kWeightSfBytes,
                           Shape::kWeightSfBytes, &smem->full[stage]);
            } else {
              bulk_load_1d(smem->sfb[stage], sf_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes,
                           &smem->full[stage]);
              if (kWide)
                bulk_load_1d(smem->sfb[stage] + kSfStageBytes, sf_src2 + static_cast<size_t>(kb) * kSfStageBytes,
                             sf_bytes, &smem->full[stage]);
            }
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok && lane == 0) {
      // Unwinding: let the copies already issued land before shared memory is given up.
      const int pending = issued < kStages ? issued : kStages;
      int s = stage;
      uint32_t ph = phase;
      for (int i = 0; i < pending; ++i) {
        if (--s < 0) {
          s = kStages - 1;
          ph ^= 1u;
        }
        mbar_wait_bounded(&smem->full[s], ph, 40000000ll);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop so that every address below is warp-uniform; one
    // elected lane (always the same one) issues the tcgen05 instructions, which keeps
    // their program order.
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    // Descriptor words (sm_100 shared-memory descriptor): low word = address >> 4; high
    // word = stride >> 4 | version 1 at bit 14 | swizzle mode at bits 29..31.
    const uint32_t a_lo0 = (smem_u32(smem->a[0]) & 0x3ffffu) >> 4;
    const uint32_t b_lo0 = (smem_u32(smem->b[0]) & 0x3ffffu) >> 4;
    constexpr uint32_t hi_ab = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8 rows x 128 B, 128B swizzle
    const bool full_last = p.last_mmas == 4;
    const bool leader = elect_one();
    for (int round = 0; round < rounds; ++round) {
      WorkItem item;
      if (!work_item<kMode, kN>(round, total_items, m_tiles, p.n_tiles, tile_first, item)) continue;
      if (!__all_sync(0xffffffffu,
                      wait_or_abort<false>(&smem->acc_empty[acc_stage], acc_phase ^ 1u, smem, p.status)))
        break;
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc_stage * kTileN);
      bool ok = true;
      tc_fence_after_sync();  // the epilogue's tensor-memory loads of this accumulator are done
      for (int kb = 0; kb < p.k_blocks; kb += kAtoms) {
        // All lanes execute the same test on the same barrier, so the result is warp-uniform
        // without a vote.  The operands were written by the async proxy and are read by it;
        // the barrier's transaction count is what orders the two, no tcgen05 fence is needed.
        // With block scales the stage is ready once the copier's scale copies have landed in
        // tensor memory (which implies that the operands have landed in shared memory).
        ok = wait_or_abort<false>(kMode == kFp8 ? &smem->full[stage] : &smem->sf_full[stage], phase, smem, p.status);
        if (!ok) break;
        if (kMode != kFp8) tc_fence_after_sync();
        // Descriptor low words advance by whole stages and K atoms; the K offset of each MMA
        // (+32 bytes inside the swizzle row) is an immediate.
        const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (kAtoms * kOperandStageBytes >> 4);
        const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (kAtoms * Shape::kWeightBytes >> 4);
        const uint32_t tmem_sf = tmem_base + kSfColumn + Shape::kSfColumns * kAtoms * stage;
        if (leader) {
#pragma unroll
          for (int atom = 0; atom < kAtoms; ++atom) {
            const int k = kb + atom;
            if (k >= p.k_blocks) break;
            const uint32_t accumulate = k != 0 ? 1u : 0u;
            const uint32_t aa = a_lo + atom * (kOperandStageBytes >> 4);
            const uint32_t bb = b_lo + atom * (Shape::kWeightBytes >> 4);
            const uint32_t ts = tmem_sf + atom * Shape::kSfColumns;
            if (kMode == kFp8) {
              if (k != p.k_blocks - 1 || full_last) issue_k_block_fp8<4>(tmem_acc, aa, bb, hi_ab, accumulate);
              else if (p.last_mmas == 3) issue_k_block_fp8<3>(tmem_acc, aa, bb, hi_ab, accumulate);
              else if (p.last_mmas == 2) issue_k_block_fp8<2>(tmem_acc, aa, bb, hi_ab, accumulate);
              else issue_k_block_fp8<1>(tmem_acc, aa, bb, hi_ab, accumulate);
            } else if (k != p.k_blocks - 1 || full_last) {
              issue_mmas<4, kN>(tmem_acc, ts, aa, bb, hi_ab, accumulate);
            } else if (p.last_mmas == 3) {
              issue_mmas<3, kN>(tmem_acc, ts, aa, bb, hi_ab, accumulate);
            } else if (p.last_mmas == 2) {
              issue_mmas<2, kN>(tmem_acc, ts, aa, bb, hi_ab, accumulate);
            } else {
              issue_mmas<1, kN>(tmem_acc, ts, aa, bb, hi_ab, accumulate);
            }
          }
          tc_commit(&smem->empty[stage]);  // frees the stage once these MMAs have read it
          if (kb + kAtoms >= p.k_blocks) tc_commit(&smem->acc_full[acc_stage]);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (warp == kScaleCopyWarp) {
    // ---------------- scale-factor copier ----------------
    // Walks the same items and K blocks as the MMA warp, one step ahead of it: when a stage's
    // bytes have landed in shared memory it copies the stage's scale-factor atoms into the
    // tensor-memory columns of that stage and commits them to sf_full.  The columns of a stage
    // are free by then: the producers refill a stage only after the MMAs that read it (and its
    // scale columns) have completed.
    if (kMode != kFp8) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t sfa_lo0 = (smem_u32(smem->sfa[0]) & 0x3ffffu) >> 4;
      const uint32_t sfb_lo0 = (smem_u32(smem->sfb[0]) & 0x3ffffu) >> 4;
      constexpr uint32_t hi_sf = (128u >> 4) | (1u << 14);  // 8 rows x 16 B, no swizzle
      const bool full_last = p.last_mmas == 4;
      const bool leader = elect_one();
      bool ok = true;
      for (int round = 0; ok && round < rounds; ++round) {
        WorkItem item;
        if (!work_item<kMode, kN>(round, total_items, m_tiles, p.n_tiles, tile_first, item)) continue;
        for (int kb = 0; kb < p.k_blocks; kb += kAtoms) {
          ok = wait_or_abort<false>(&smem->full[stage], phase, smem, p.status);
          if (!ok) break;
          const uint32_t sfa_lo = sfa_lo0 + static_cast<uint32_t>(stage) * (kAtoms * kSfStageBytes >> 4);
          const uint32_t sfb_lo = sfb_lo0 + static_cast<uint32_t>(stage) * (kAtoms * Shape::kWeightSfBytes >> 4);
          const uint32_t tmem_sf = tmem_base + kSfColumn + Shape::kSfColumns * kAtoms * stage;
          if (leader) {
#pragma unroll
            for (int atom = 0; atom < kAtoms; ++atom) {
              const int k = kb + atom;
              if (k >= p.k_blocks) break;
              const uint32_t sa = sfa_lo + atom * (kSfStageBytes >> 4);
              const uint32_t sb = sfb_lo + atom * (Shape::kWeightSfBytes >> 4);
              const uint32_t ts = tmem_sf + atom * Shape::kSfColumns;
              if (k != p.k_blocks - 1 || full_last) issue_sf_copies<4, kN>(ts, sa, sb, hi_sf);
              else if (p.last_mmas == 3) issue_sf_copies<3, kN>(ts, sa, sb, hi_sf);
              else if (p.last_mmas == 2) issue_sf_copies<2, kN>(ts, sa, sb, hi_sf);
              else issue_sf_copies<1, kN>(ts, sa, sb, hi_sf);
            }
            tc_commit(&smem->sf_full[stage]);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ---------------- epilogue: 16 warps ----------------
    // A warp may touch only the tensor-memory lanes 32*(warp%4)..+31, so the four warps
    // with the same warp%4 share one 32-row quarter of the tile and split its columns.
    const int quarter = warp & 3;
    const int sub = (warp - 2) >> 2;  // 0..3
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    uint8_t* staging = smem->staging[quarter];
    for (int round = 0; round < rounds; ++round) {
      WorkItem item;
      if (!work_item<kMode, kN>(round, total_items, m_tiles, p.n_tiles, tile_first, item)) continue;
      const int m_tile = item.m_tile;
      const int n_tile = item.n_tile;
      const int expert = p.tile_expert[m_tile];
      const int local0 = m_tile * kTileM - p.scale_row_offsets[expert];
      const int row0 = p.expert_offsets[expert] + local0;
      const int rows_valid = p.expert_offsets[expert + 1] - row0;  // may exceed 128
      const float alpha = p.alpha[expert];
      const bool acc_ready = wait_or_abort<true>(&smem->acc_full[acc_stage], acc_phase, smem, p.status);
      if constexpr (kMode != kGeglu) {
        // The four warps of a quarter meet at named barriers while they store, so they must
        // leave together: a warp whose wait failed says so, and all four read the answer behind
        // a barrier of their own.
        if (!acc_ready) smem->quarter_left[quarter] = 1;
        named_barrier(1 + quarter, kEpilogueWarpsPerQuarter * 32);
        if (*reinterpret_cast<volatile int*>(&smem->quarter_left[quarter])) break;
      } else {
        if (!acc_ready) break;
      }
      tc_fence_after_sync();
      const int row_local = quarter * 32 + lane;
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                static_cast<uint32_t>(acc_stage * kTileN);
      if constexpr (kMode != kGeglu && !kWide) {
        uint32_t r[32];
        tmem_load_32x32(tmem_row + sub * 32, r);
        tmem_load_wait();
        tc_fence_before_sync();
        mbar_arrive(&smem->acc_empty[acc_stage]);  // accumulators are in registers now
        // same decision in all four warps of the quarter
        if (quarter * 32 < rows_valid)
          stage_and_store(r, alpha, staging, quarter, sub, lane, rows_valid, row0, n_tile * kN, p);
      } else if constexpr (kMode != kGeglu) {
        // 256 columns: both halves are taken into registers before the accumulator is released
        uint32_t r0[32], r1[32];
        tmem_load_32x32(tmem_row + sub * 32, r0);
        tmem_load_32x32(tmem_row + kStoreColumns + sub * 32, r1);
        tmem_load_wait();
        tc_fence_before_sync();
        mbar_arrive(&smem->acc_empty[acc_stage]);
        if (quarter * 32 < rows_valid) {
          stage_and_store(r0, alpha, staging, quarter, sub, lane, rows_valid, row0, n_tile * kN, p);
          stage_and_store(r1, alpha, staging, quarter, sub, lane, rows_valid, row0,
                          n_tile * kN + kStoreColumns, p);
        }
      } else {
        // Fused GeGLU + NVFP4 requantise, wide tile.  Accumulator columns [0,128) are up and
        // [128,256) gate of intermediate columns [128*n_tile, 128*n_tile+128); this warp owns
        // the two 16-column blocks 2*sub and 2*sub+1 of them.
        const float multiplier = p.next_scale_q[expert];
        uint32_t up0[16], gate0[16], up1[16], gate1[16];
        tmem_load_32x16(tmem_row + sub * 32, up0);
        tmem_load_32x16(tmem_row + 128 + sub * 32, gate0);
        tmem_load_32x16(tmem_row + sub * 32 + 16, up1);
        tmem_load_32x16(tmem_row + 128 + sub * 32 + 16, gate1);
        tmem_load_wait();
        tc_fence_before_sync();
        mbar_arrive(&smem->acc_empty[acc_stage]);
        const bool columns_exist = n_tile * 128 + sub * 32 < kInter;  // the last item is half empty
        if (row_local < rows_valid && columns_exist) {
          uint4 codes;
          const uint32_t scale0 = geglu_block(up0, gate0, alpha, multiplier, smem->erf_table, codes.x, codes.y);
          const uint32_t scale1 = geglu_block(up1, gate1, alpha, multiplier, smem->erf_table, codes.z, codes.w);
          // the w2 operand: read eleven times by the next launch, so L2 is asked to keep it
          unsigned long long keep_in_l2;
          asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_in_l2));
          asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(
                           p.next_codes + static_cast<size_t>(row0 + row_local) * (kInter / 2) + n_tile * 64 + sub * 16),
                       "r"(codes.x), "r"(codes.y), "r"(codes.z), "r"(codes.w), "l"(keep_in_l2)
                       : "memory");
          // scale groups 8*n_tile+2*sub and the next one (same 4-group word) of row
          // (128*m_tile + row_local) of the w2 operand
          constexpr int groups = kInter / 16;
          *reinterpret_cast<uint16_t*>(p.next_scales + static_cast<size_t>(m_tile) * kTileM * groups +
                                       sf_offset(row_local, 8 * n_tile + 2 * sub, groups)) =
              static_cast<uint16_t>(scale0 | (scale1 << 8));
        }
      }
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// Re-tiles the w13 block scales for the fused epilogue: item j of an expert takes up rows
// [128j, 128j+128) and gate rows [704+128j, 704+128j+128) as its 256 MMA-N rows.  Per item
// and K block of 256 the copy holds [half (up, gate)][MMA 0..3][512-byte atom], the atom
// being (n%32)*16 + (n/32)*4 + k over the 128 rows n of the half; rows past 704 get scale 0.
// One thread per byte.
__global__ void retile_w13_scales_kernel(const uint8_t* __restrict__ sidecar,
                                         uint8_t* __restrict__ tiled, int experts) {
  constexpr int groups = kHidden / 16;          // 176
  constexpr int k_blocks = kHidden / 256;       // 11
  const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(experts) * kFusedItems * k_blocks * 8 * kSfAtomBytes;
  if (index >= total) return;
  const int byte = static_cast<int>(index % kSfAtomBytes);
  size_t rest = index / kSfAtomBytes;
  const int mma = static_cast<int>(rest % 4);
  rest /= 4;
  const int half = static_cast<int>(rest % 2);
  rest /= 2;
  const int k_block = static_cast<int>(rest % k_blocks);
  rest /= k_blocks;
  const int item = static_cast<int>(rest % kFusedItems);
  const int expert = static_cast<int>(rest / kFusedItems);
  const int n = ((byte & 15) >> 2) * 32 + (byte >> 4);  // row of this byte within the half
  const int k = byte & 3;
  const int column = item * 128 + n;                    // intermediate column
  uint8_t value = 0;
  if (column < kInter) {
    const int source_row = half == 0 ? column : kInter + column;
    value = sidecar[static_cast<size_t>(expert) * kW13Out * groups +
                    sf_offset(source_row, (k_block * 4 + mma) * 4 + k, groups)];
  }
  tiled[index] = value;
}

}  // namespace


namespace {
template <int kMode, int kAtoms, int kN> cudaError_t raise_smem_limit() {
  return cudaFuncSetAttribute(grouped_nvfp4_gemm_kernel<kMode, kAtoms, kN>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(gemm_smem_bytes<kMode, kAtoms, kN>()));
}

template <int kMode, int kN>
void launch_variant(const GemmOperands& op, const GemmParams& p, int sm_count, cudaStream_t stream) {
  if (op.serial_launch) {
    grouped_nvfp4_gemm_kernel<kMode, 1, kN><<<sm_count, kGemmThreads, gemm_smem_bytes<kMode, 1, kN>(), stream>>>(
        op.map_a, op.map_a32, op.map_b, op.map_b64, p);
    return;
  }
  launch_chained(grouped_nvfp4_gemm_kernel<kMode, 1, kN>, dim3(sm_count), dim3(kGemmThreads),
                 gemm_smem_bytes<kMode, 1, kN>(), stream, op.map_a, op.map_a32, op.map_b, op.map_b64, p);
}
}  // namespace

int prepare_grouped_gemm() {
  cudaError_t e = raise_smem_limit<kPlain, 1, 128>();
  if (e == cudaSuccess) e = raise_smem_limit<kPlain, 1, 256>();
  if (e == cudaSuccess) e = raise_smem_limit<kGeglu, 1, 256>();
  if (e == cudaSuccess) e = raise_smem_limit<kFp8, 1, 128>();
  if (e == cudaSuccess) e = static_cast<cudaError_t>(prepare_decode_experts());
  if (e == cudaSuccess) return prepare_grouped_gemm_pairs();
  return static_cast<int>(e);
}

size_t retiled_w13_scale_bytes(int experts) {
  return static_cast<size_t>(experts) * kFusedItems * (kHidden / 256) * 8 * kSfAtomBytes;
}

void launch_retile_w13_scales(const uint8_t* sidecar_scales, uint8_t* tiled, int experts,
                              cudaStream_t stream) {
  const size_t total = retiled_w13_scale_bytes(experts);
  retile_w13_scales_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      sidecar_scales, tiled, experts);
}

void launch_grouped_gemm(const GemmOperands& op, const RoutePlan& plan, int sm_count,
                         cudaStream_t stream) {
  if (op.use_pairs && plan.pair_tile && !op.fp8 && (op.fused_geglu || op.n_out % 256 == 0) && sm_count >= 2) {
    launch_grouped_gemm_pairs(op, plan, sm_count, stream);
    return;
  }
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
  const int k_bytes = op.fp8 ? op.k_in : op.k_in / 2;
  p.groups = op.k_in / 16;
  p.k_blocks = (k_bytes + kTileKBytes - 1) / kTileKBytes;
  p.last_mmas = (k_bytes - (p.k_blocks - 1) * kTileKBytes) / 32;
  if (op.fp8) {
    p.n_tiles = op.n_out / kTileN;
    launch_variant<kFp8, 128>(op, p, sm_count, stream);
  } else if (op.fused_geglu) {
    p.n_tiles = kFusedItems;
    launch_variant<kGeglu, 256>(op, p, sm_count, stream);
  } else if (op.n_out % 256 == 0) {
    p.n_tiles = op.n_out / 256;
    launch_variant<kPlain, 256>(op, p, sm_count, stream);
  } else {
    p.n_tiles = op.n_out / kTileN;
    launch_variant<kPlain, 128>(op, p, sm_count, stream);
  }
}

}  // namespace gv
