// Both expert GEMMs of a decode-sized batch in one persistent kernel.
//
// With a few rows per expert the layer is bound by streaming the routed experts' weights from
// HBM once (3.3 MB per expert).  As two launches (grouped_gemm.cu) the stream stops twice: w13's
// last items drain while most SMs idle, w2 ramps up from empty pipelines, and 768 + 1408 items of
// two sizes are dealt to 148 CTAs in two separate, coarse rounds.  Here one grid walks one list,
// all w13 items (fused GeGLU + requantise epilogue) followed by all w2 items, so weight bytes keep
// arriving across the boundary and the tail is that of the whole list.
//
// A w2 item needs the w2 operand rows of its row tile, which the six w13 items of that tile write.
// Every epilogue warp of a w13 item adds one to the tile's counter after its stores (release);
// the activation-side producer of a w2 item waits until the counter says that all 6 x 16 warps
// have done so (bounded acquire spin), then crosses to the async proxy and issues its TMA loads.
// The weight-side producer waits for nothing, which is the point.  No cycle of waits exists:
// every CTA reaches its w2 items only after its own w13 items, and w13 items wait for nothing
// outside their CTA.  The grid is one CTA per SM, all co-resident.
//
// Tile shape, pipeline, roles and epilogue arithmetic are those of the 128 x 256 kernel of
// grouped_gemm.cu, with four stages: the plain epilogue stores its few rows straight from
// registers (64 bytes per thread and half tile), so no staging tile takes shared memory from the
// pipeline.  At most 128 tokens, so every expert has at most one row tile.
//
// In its kFront form the kernel also does what route_sort_quantize_small_kernel does, so a decode
// layer step is three launches (router, this, reduce) and the weights start streaming while the
// input is still being quantised.  Every CTA counts the batch's at most 1024 routes per expert
// and derives the group geometry into its own shared memory (the same redundant counting sort,
// 148 times instead of once per token); CTA t < tokens ranks the eight routes of token t and
// quantises the token with three of its epilogue warps, then adds one to a counter (release).
// The activation-side producer waits (bounded) until the counter has reached `tokens` before
// its first load; the weight side waits for nothing.  The last CTA to finish puts the counters
// back to zero for the next launch: no CTA can still be waiting on them then.
#include "gv_common.cuh"
#include "gv_gemm_parts.cuh"
#include "gv_launchers.h"
#include "gv_quantize.cuh"

namespace gv {

namespace {

constexpr int kDecStages = 4;
constexpr int kDecWeightProducerWarp = 2 + 4 * kEpilogueWarpsPerQuarter;  // 18
constexpr int kDecScaleCopyWarp = kDecWeightProducerWarp + 1;             // 19
constexpr int kDecThreads = (kDecScaleCopyWarp + 1) * 32;                 // 640
constexpr uint32_t kDecTmemColumns = 512;
constexpr uint32_t kDecSfColumn = 256;
constexpr uint32_t kDecSfColumnsPerStage = 64;
constexpr int kDecTileBytes = kTileM * kTileKBytes;  // 16 KiB
constexpr int kW13Items = kFusedItems;               // 6 per row tile
constexpr int kW13KBlocks = kHidden / kTileK;        // 11
constexpr int kW2Items = kHidden / 256;              // 11 per row tile
constexpr int kW2KBlocks = (kInter / 2 + kTileKBytes - 1) / kTileKBytes;             // 3
constexpr int kW2LastMmas = (kInter / 2 - (kW2KBlocks - 1) * kTileKBytes) / 32;      // 3
constexpr int kReadyPerTile = kW13Items * 4 * kEpilogueWarpsPerQuarter;              // 96 warp arrivals

struct alignas(1024) DecodeSmem {
  uint8_t a[kDecStages][kDecTileBytes];
  uint8_t b[kDecStages][2 * kDecTileBytes];
  uint8_t sfa[kDecStages][kSfStageBytes];
  uint8_t sfb[kDecStages][2 * kSfStageBytes];
  uint64_t full[kDecStages];
  uint64_t empty[kDecStages];
  uint64_t sf_full[kDecStages];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  volatile int abort;
  alignas(16) float erf_table[GV_ERF_TABLE_FLOATS];
  // kFront: the group geometry of the batch, computed by this CTA, and the routes of its token
  int expert_offsets[kExperts + 1];
  int scale_row_offsets[kExperts + 1];
  int tile_expert[kExperts];
  int histogram[kExperts];
  int m_tiles;
  int own_expert[kTopK];
  int own_rank[kTopK];
  int route_row[kTopK];
  float route_multiplier[kTopK];
  unsigned long long route_scale_base[kTopK];
};

constexpr int kFrontQuantizeWarps = (kQuantizeThreadsPerToken + 31) / 32;  // epilogue warps 2..4
constexpr size_t kDecSmemBytes = sizeof(DecodeSmem) + 1024;
static_assert(kDecSmemBytes <= 232448, "shared memory budget");
static_assert(kDecSfColumn + kDecSfColumnsPerStage * kDecStages <= kDecTmemColumns, "tensor memory budget");

struct DecodeParams {
  GemmParams w13;   // fused form: next_codes / next_scales / next_scale_q set
  GemmParams w2;    // plain form: out (and optionally row_dest) set
  int* tile_ready;  // [row tiles], zero on entry; zero again on exit where plan.front_sync exists
  RoutePlan plan;   // kFront: written by CTA 0 (geometry) and by each token's CTA (its routes)
  // kFront only
  const __nv_bfloat16* input;   // bf16 [tokens, 2816]
  const int* expert_ids;        // i32 [tokens, 8]
  const float* in_scale_q;      // f32 [128]
  uint8_t* packed;              // w13 operand codes
  uint8_t* scales;              // w13 operand scale factors
  int tokens;
};

struct DecodeItem {
  bool down;   // false: w13 item, true: w2 item
  int m_tile;
  int n_tile;
};

// One list: the w13 items tile by tile (so that the first tiles' w2 operands are complete long
// before the last w13 item ends), then the w2 items; dealt to the CTAs in snake order.
__device__ __forceinline__ bool decode_item(int round, int m_tiles, DecodeItem& item) {
  const int grid = static_cast<int>(gridDim.x);
  const int slot = (round & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  int index = round * grid + slot;
  const int up_items = m_tiles * kW13Items;
  if (index < up_items) {
    item.down = false;
    item.m_tile = index / kW13Items;
    item.n_tile = index - item.m_tile * kW13Items;
    return true;
  }
  index -= up_items;
  if (index >= m_tiles * kW2Items) return false;
  item.down = true;
  item.m_tile = index / kW2Items;
  item.n_tile = index - item.m_tile * kW2Items;
  return true;
}

// 32 accumulator columns of one row, scaled, rounded to bf16 and stored: 64 contiguous bytes.
__device__ __forceinline__ void store_row_piece(const uint32_t (&r)[32], float alpha, __nv_bfloat16* destination) {
  uint4* out = reinterpret_cast<uint4*>(destination);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i])), __fmul_rn(alpha, __uint_as_float(r[8 * i + 1])));
    v.y = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 2])), __fmul_rn(alpha, __uint_as_float(r[8 * i + 3])));
    v.z = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 4])), __fmul_rn(alpha, __uint_as_float(r[8 * i + 5])));
    v.w = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 6])), __fmul_rn(alpha, __uint_as_float(r[8 * i + 7])));
    out[i] = v;
  }
}

__device__ __forceinline__ int load_acquire_gpu(const int* address) {
  int value;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

template <bool kFront>
__global__ void __launch_bounds__(kDecThreads, 1)
decode_experts_kernel(const __grid_constant__ CUtensorMap map_a13, const __grid_constant__ CUtensorMap map_a13_32,
                      const __grid_constant__ CUtensorMap map_b13, const __grid_constant__ CUtensorMap map_b13_64,
                      const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_a2_32,
                      const __grid_constant__ CUtensorMap map_b2, const DecodeParams params) {
  extern __shared__ uint8_t smem_raw[];
  DecodeSmem* smem =
      reinterpret_cast<DecodeSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int* const status = params.w13.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&smem->full[s], 2);
      mbar_init(&smem->empty[s], 1);
      mbar_init(&smem->sf_full[s], 1);
    }
    mbar_init(&smem->acc_full, 1);
    mbar_init(&smem->acc_empty, kEpilogueThreads);
    smem->abort = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a13);
    prefetch_tensor_map(&map_a13_32);
    prefetch_tensor_map(&map_b13);
    prefetch_tensor_map(&map_b13_64);
    prefetch_tensor_map(&map_a2);
    prefetch_tensor_map(&map_a2_32);
    prefetch_tensor_map(&map_b2);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kDecTmemColumns);
    tmem_relinquish();
  }
  load_erf_table(smem->erf_table);
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = smem->tmem_base;
  grid_dependency_wait();

  // The geometry both GEMMs walk: the plan of an earlier launch, or this CTA's own copy.
  const int* tile_expert = params.w13.tile_expert;
  const int* expert_offsets = params.w13.expert_offsets;
  const int* scale_row_offsets = params.w13.scale_row_offsets;
  int m_tiles;
  const bool has_token = kFront && static_cast<int>(blockIdx.x) < params.tokens;
  if constexpr (kFront) {
    constexpr int groups = kHidden / 16;
    const int tid = threadIdx.x;
    const int token = blockIdx.x;
    const int routes = params.tokens * kTopK;
    const RoutePlan& plan = params.plan;
    if (tid < kExperts) smem->histogram[tid] = 0;
    if (tid < kTopK) {
      int expert = kExperts;
      if (has_token) {
        expert = params.expert_ids[token * kTopK + tid];
        if (expert < 0 || expert >= kExperts) expert = kExperts;
        else if (plan.remap) expert = plan.remap[expert];
      }
      smem->own_expert[tid] = expert;
      smem->own_rank[tid] = 0;
    }
    __syncthreads();
    for (int route = tid; route < routes; route += kDecThreads) {
      int expert = params.expert_ids[route];
      if (expert < 0 || expert >= kExperts) {
        if (token == 0) atomicExch(status, static_cast<int>(kBadExpertId));
        continue;
      }
      if (plan.remap) expert = plan.remap[expert];
      atomicAdd(&smem->histogram[expert], 1);
      if (has_token) {
#pragma unroll
        for (int k = 0; k < kTopK; ++k)
          if (expert == smem->own_expert[k] && route < token * kTopK + k) atomicAdd(&smem->own_rank[k], 1);
      }
    }
    __syncthreads();
    if (warp == 0) {
      // lane l scans experts 4l..4l+3: rows and row tiles (one per expert that has rows)
      int counts[4], rows = 0, tiles = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        counts[i] = smem->histogram[4 * lane + i];
        rows += counts[i];
        tiles += (counts[i] + kTileM - 1) / kTileM;
      }
      int rows_inclusive = rows, tiles_inclusive = tiles;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int r = __shfl_up_sync(0xffffffffu, rows_inclusive, offset);
        const int t = __shfl_up_sync(0xffffffffu, tiles_inclusive, offset);
        if (lane >= offset) {
          rows_inclusive += r;
          tiles_inclusive += t;
        }
      }
      int row = rows_inclusive - rows, tile = tiles_inclusive - tiles;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int expert = 4 * lane + i;
        const int expert_tiles = (counts[i] + kTileM - 1) / kTileM;
        smem->expert_offsets[expert] = row;
        smem->scale_row_offsets[expert] = tile * kTileM;
        for (int j = 0; j < expert_tiles; ++j) smem->tile_expert[tile + j] = expert;
        if (token == 0) {
          plan.expert_offsets[expert] = row;
          plan.scale_row_offsets[expert] = tile * kTileM;
          for (int j = 0; j < expert_tiles; ++j) plan.tile_expert[tile + j] = expert;
        }
        row += counts[i];
        tile += expert_tiles;
      }
      if (lane == 31) {
        smem->expert_offsets[kExperts] = row;
        smem->scale_row_offsets[kExperts] = tile * kTileM;
        smem->m_tiles = tile;
        if (token == 0) {
          plan.expert_offsets[kExperts] = row;
          plan.scale_row_offsets[kExperts] = tile * kTileM;
          plan.num_m_tiles[0] = tile;
        }
      }
    }
    __syncthreads();
    if (has_token && tid < kTopK) {
      const int route = token * kTopK + tid;
      const int expert = smem->own_expert[tid];
      int dst = -1;
      if (expert < kExperts) {
        dst = smem->expert_offsets[expert] + smem->own_rank[tid];
        plan.sorted_experts[dst] = expert;
        plan.sorted_routes[dst] = route;
        plan.inverse_routes[route] = dst;
        // the static scale belongs to the expert id as the caller numbers it
        smem->route_multiplier[tid] = params.in_scale_q[params.expert_ids[route]];
        smem->route_scale_base[tid] = static_cast<unsigned long long>(smem->scale_row_offsets[expert]) * groups +
                                      sf_offset(smem->own_rank[tid], 0, groups);
      }
      smem->route_row[tid] = dst;
    }
    __syncthreads();
    tile_expert = smem->tile_expert;
    expert_offsets = smem->expert_offsets;
    scale_row_offsets = smem->scale_row_offsets;
    m_tiles = smem->m_tiles;
  } else {
    m_tiles = params.w13.num_m_tiles[0];
  }
  const int total_items = m_tiles * (kW13Items + kW2Items);
  const int rounds = (total_items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  if (warp == 0 || warp == kDecWeightProducerWarp) {
    // ---------------- TMA producers ----------------
    const bool weight_side = warp == kDecWeightProducerWarp;
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    if (kFront && !weight_side) {
      // the w13 operand exists once every token's CTA has quantised its token and counted itself
      const long long start = clock64();
      bool ready = false;
      for (uint32_t spin = 0; !ready; ++spin) {
        ready = load_acquire_gpu(params.plan.front_sync) >= params.tokens;
        if (!ready) {
          __nanosleep(64);
          if ((spin & 63u) == 63u && (smem->abort || clock64() - start > kWaitLimitCycles)) {
            if (!smem->abort) {
              smem->abort = 1;
              atomicExch(status, static_cast<int>(kWaitTimeout));
            }
            break;
          }
        }
      }
      ok = __all_sync(0xffffffffu, ready);
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    for (int round = 0; ok && round < rounds; ++round) {
      DecodeItem item;
      if (!decode_item(round, m_tiles, item)) continue;
      const GemmParams& p = item.down ? params.w2 : params.w13;
      const int k_blocks = item.down ? kW2KBlocks : kW13KBlocks;
      const int last_mmas = item.down ? kW2LastMmas : 4;
      const int expert = tile_expert[item.m_tile];
      int row = 0, row2 = 0;
      const uint8_t* sf_src;
      const uint8_t* sf_src2 = nullptr;
      bool short_tile = false, half_item = false;
      if (!weight_side) {
        row = expert_offsets[expert] + (item.m_tile * kTileM - scale_row_offsets[expert]);
        short_tile = expert_offsets[expert + 1] - row <= 32;
        sf_src = p.a_scales + static_cast<size_t>(item.m_tile) * kTileM * p.groups;
        if (item.down) {
          // the w2 operand rows of this tile exist once every epilogue warp of its six w13 items
          // has stored and counted itself
          const long long start = clock64();
          bool ready = false;
          for (uint32_t spin = 0; !ready; ++spin) {
            ready = load_acquire_gpu(params.tile_ready + item.m_tile) >= kReadyPerTile;
            if (!ready) {
              __nanosleep(64);
              if ((spin & 63u) == 63u && (smem->abort || clock64() - start > kWaitLimitCycles)) {
                if (!smem->abort) {
                  smem->abort = 1;
                  atomicExch(status, static_cast<int>(kWaitTimeout));
                }
                break;
              }
            }
          }
          ok = __all_sync(0xffffffffu, ready);
          if (!ok) break;
          // the rows were written by ordinary stores of other SMs; the copies below read them
          // through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
      } else if (!item.down) {
        row = expert * kW13Out + item.n_tile * 128;
        row2 = row + kInter;
        half_item = (item.n_tile + 1) * 128 > kInter;
        sf_src = p.b_scales + (static_cast<size_t>(expert) * kW13Items + item.n_tile) * 256 * p.groups;
      } else {
        row = expert * p.n_out + item.n_tile * 256;
        row2 = row + 128;
        sf_src = p.b_scales + static_cast<size_t>(row) * p.groups;
        sf_src2 = sf_src + static_cast<size_t>(128) * p.groups;
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, wait_or_abort<true>(&smem->empty[stage], phase ^ 1u, smem, status));
        if (!ok) break;
        if (elect_one()) {
          const uint32_t sf_bytes = static_cast<uint32_t>(kb + 1 == k_blocks ? last_mmas : 4) * kSfAtomBytes;
          const int x = kb * kTileKBytes;
          if (!weight_side) {
            mbar_arrive_expect_tx(&smem->full[stage], (short_tile ? kDecTileBytes / 4 : kDecTileBytes) + sf_bytes);
            const CUtensorMap* map = item.down ? (short_tile ? &map_a2_32 : &map_a2) : (short_tile ? &map_a13_32 : &map_a13);
            tma_load_2d(smem->a[stage], map, &smem->full[stage], x, row);
            bulk_load_1d(smem->sfa[stage], sf_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes, &smem->full[stage]);
          } else if (!item.down) {
            mbar_arrive_expect_tx(&smem->full[stage], (half_item ? kDecTileBytes : 2 * kDecTileBytes) + 2 * kSfStageBytes);
            const CUtensorMap* map = half_item ? &map_b13_64 : &map_b13;
            tma_load_2d(smem->b[stage], map, &smem->full[stage], x, row);
            tma_load_2d(smem->b[stage] + kDecTileBytes, map, &smem->full[stage], x, row2);
            bulk_load_1d(smem->sfb[stage], sf_src + static_cast<size_t>(kb) * 2 * kSfStageBytes, 2 * kSfStageBytes,
                         &smem->full[stage]);
          } else {
            mbar_arrive_expect_tx(&smem->full[stage], 2 * kDecTileBytes + 2 * sf_bytes);
            tma_load_2d(smem->b[stage], &map_b2, &smem->full[stage], x, row);
            tma_load_2d(smem->b[stage] + kDecTileBytes, &map_b2, &smem->full[stage], x, row2);
            bulk_load_1d(smem->sfb[stage], sf_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes, &smem->full[stage]);
            bulk_load_1d(smem->sfb[stage] + kSfStageBytes, sf_src2 + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes,
                         &smem->full[stage]);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == kDecStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok && lane == 0) {
      const int pending = issued < kDecStages ? issued : kDecStages;
      int s = stage;
      uint32_t ph = phase;
      for (int i = 0; i < pending; ++i) {
        if (--s < 0) {
          s = kDecStages - 1;
          ph ^= 1u;
        }
        mbar_wait_bounded(&smem->full[s], ph, 40000000ll);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0, acc_phase = 0;
    const uint32_t a_lo0 = (smem_u32(smem->a[0]) & 0x3ffffu) >> 4;
    const uint32_t b_lo0 = (smem_u32(smem->b[0]) & 0x3ffffu) >> 4;
    constexpr uint32_t hi_ab = (1024u >> 4) | (1u << 14) | (2u << 29);
    const bool leader = elect_one();
    for (int round = 0; round < rounds; ++round) {
      DecodeItem item;
      if (!decode_item(round, m_tiles, item)) continue;
      const int k_blocks = item.down ? kW2KBlocks : kW13KBlocks;
      if (!__all_sync(0xffffffffu, wait_or_abort<false>(&smem->acc_empty, acc_phase ^ 1u, smem, status))) break;
      acc_phase ^= 1u;
      bool ok = true;
      tc_fence_after_sync();
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = wait_or_abort<false>(&smem->sf_full[stage], phase, smem, status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (kDecTileBytes >> 4);
        const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (2 * kDecTileBytes >> 4);
        const uint32_t tmem_sf = tmem_base + kDecSfColumn + kDecSfColumnsPerStage * stage;
        if (leader) {
          const uint32_t accumulate = kb != 0 ? 1u : 0u;
          if (item.down && kb + 1 == k_blocks) issue_mmas<kW2LastMmas, 256>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
          else issue_mmas<4, 256>(tmem_base, tmem_sf, a_lo, b_lo, hi_ab, accumulate);
          tc_commit(&smem->empty[stage]);
          if (kb + 1 == k_blocks) tc_commit(&smem->acc_full);
        }
        if (++stage == kDecStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
    }
  } else if (warp == kDecScaleCopyWarp) {
    // ---------------- scale-factor copier ----------------
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t sfa_lo0 = (smem_u32(smem->sfa[0]) & 0x3ffffu) >> 4;
    const uint32_t sfb_lo0 = (smem_u32(smem->sfb[0]) & 0x3ffffu) >> 4;
    constexpr uint32_t hi_sf = (128u >> 4) | (1u << 14);
    const bool leader = elect_one();
    bool ok = true;
    for (int round = 0; ok && round < rounds; ++round) {
      DecodeItem item;
      if (!decode_item(round, m_tiles, item)) continue;
      const int k_blocks = item.down ? kW2KBlocks : kW13KBlocks;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = wait_or_abort<false>(&smem->full[stage], phase, smem, status);
        if (!ok) break;
        const uint32_t sfa_lo = sfa_lo0 + static_cast<uint32_t>(stage) * (kSfStageBytes >> 4);
        const uint32_t sfb_lo = sfb_lo0 + static_cast<uint32_t>(stage) * (2 * kSfStageBytes >> 4);
        const uint32_t tmem_sf = tmem_base + kDecSfColumn + kDecSfColumnsPerStage * stage;
        if (leader) {
          if (item.down && kb + 1 == k_blocks) issue_sf_copies<kW2LastMmas, 256>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
          else issue_sf_copies<4, 256>(tmem_sf, sfa_lo, sfb_lo, hi_sf);
          tc_commit(&smem->sf_full[stage]);
        }
        if (++stage == kDecStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------- epilogue: 16 warps ----------------
    const int quarter = warp & 3;
    const int sub = (warp - 2) >> 2;
    uint32_t acc_phase = 0;
    if (kFront && has_token && warp < 2 + kFrontQuantizeWarps) {
      // this CTA's token: quantised once per distinct static scale, stored to its eight sorted rows
      const int part = threadIdx.x - 64;
      if (part < kQuantizeThreadsPerToken) {
        float values[32];
        float maximum[2];
        load_token_columns<2>(params.input, static_cast<int>(blockIdx.x), part, values, maximum);
        quantize_routes_of_token<2>(values, maximum, part, smem->route_row, smem->route_multiplier,
                                    smem->route_scale_base, params.packed, params.scales);
      }
      __threadfence();
      named_barrier(1, kFrontQuantizeWarps * 32);
      if (threadIdx.x == 64) atomicAdd(params.plan.front_sync, 1);
    }
    for (int round = 0; round < rounds; ++round) {
      DecodeItem item;
      if (!decode_item(round, m_tiles, item)) continue;
      const GemmParams& p = item.down ? params.w2 : params.w13;
      const int m_tile = item.m_tile, n_tile = item.n_tile;
      const int expert = tile_expert[m_tile];
      const int row0 = expert_offsets[expert] + (m_tile * kTileM - scale_row_offsets[expert]);
      const int rows_valid = expert_offsets[expert + 1] - row0;
      const float alpha = p.alpha[expert];
      const bool acc_ready = wait_or_abort<true>(&smem->acc_full, acc_phase, smem, status);
      acc_phase ^= 1u;
      if (!acc_ready) break;
      tc_fence_after_sync();
      const int row_local = quarter * 32 + lane;
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      if (item.down) {
        uint32_t r0[32], r1[32];
        tmem_load_32x32(tmem_row + sub * 32, r0);
        tmem_load_32x32(tmem_row + kStoreColumns + sub * 32, r1);
        tmem_load_wait();
        tc_fence_before_sync();
        mbar_arrive(&smem->acc_empty);
        if (row_local < rows_valid) {
          __nv_bfloat16* row = p.row_dest ? reinterpret_cast<__nv_bfloat16*>(p.row_dest[row0 + row_local])
                                          : p.out + static_cast<size_t>(row0 + row_local) * p.n_out;
          store_row_piece(r0, alpha, row + n_tile * 256 + sub * 32);
          store_row_piece(r1, alpha, row + n_tile * 256 + kStoreColumns + sub * 32);
        }
      } else {
        uint32_t up0[16], gate0[16], up1[16], gate1[16];
        tmem_load_32x16(tmem_row + sub * 32, up0);
        tmem_load_32x16(tmem_row + 128 + sub * 32, gate0);
        tmem_load_32x16(tmem_row + sub * 32 + 16, up1);
        tmem_load_32x16(tmem_row + 128 + sub * 32 + 16, gate1);
        tmem_load_wait();
        tc_fence_before_sync();
        mbar_arrive(&smem->acc_empty);
        const bool columns_exist = n_tile * 128 + sub * 32 < kInter;
        if (row_local < rows_valid && columns_exist) {
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
        // this warp's share of the tile's w2 operand is written: publish it
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(params.tile_ready + m_tile, 1);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, kDecTmemColumns);
  }
  if (params.plan.front_sync && threadIdx.x == 0) {
    // The CTA that finishes last puts the counters back for the next launch.  Every wait on
    // them lies before a CTA's end, so nobody reads them any more.
    __threadfence();
    if (atomicAdd(params.plan.front_sync + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      for (int tile = 0; tile < m_tiles; ++tile) params.tile_ready[tile] = 0;
      params.plan.front_sync[0] = 0;
      params.plan.front_sync[1] = 0;
    }
  }
}

void fill_params(GemmParams& p, const GemmOperands& op, const RoutePlan& plan) {
  p = GemmParams{};
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
  p.status = plan.status;
  p.n_out = op.n_out;
  p.groups = op.k_in / 16;
}

}  // namespace

int prepare_decode_experts() {
  cudaError_t e = cudaFuncSetAttribute(decode_experts_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kDecSmemBytes));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(decode_experts_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kDecSmemBytes));
  return static_cast<int>(e);
}

void launch_decode_experts(const GemmOperands& w13_fused, const GemmOperands& w2, const RoutePlan& plan, int sm_count,
                           cudaStream_t stream) {
  DecodeParams params{};
  fill_params(params.w13, w13_fused, plan);
  fill_params(params.w2, w2, plan);
  params.tile_ready = plan.tile_ready;
  params.plan = plan;
  launch_chained(decode_experts_kernel<false>, dim3(sm_count), dim3(kDecThreads), kDecSmemBytes, stream,
                 w13_fused.map_a, w13_fused.map_a32, w13_fused.map_b, w13_fused.map_b64, w2.map_a, w2.map_a32, w2.map_b,
                 params);
}

void launch_decode_layer(const void* input_bf16, const int* expert_ids, const float* in_scale_q, int tokens,
                         uint8_t* packed, uint8_t* scales, const GemmOperands& w13_fused, const GemmOperands& w2,
                         const RoutePlan& plan, int sm_count, cudaStream_t stream) {
  DecodeParams params{};
  fill_params(params.w13, w13_fused, plan);
  fill_params(params.w2, w2, plan);
  params.tile_ready = plan.tile_ready;
  params.input = static_cast<const __nv_bfloat16*>(input_bf16);
  params.expert_ids = expert_ids;
  params.in_scale_q = in_scale_q;
  params.plan = plan;
  params.packed = packed;
  params.scales = scales;
  params.tokens = tokens;
  launch_chained(decode_experts_kernel<true>, dim3(sm_count), dim3(kDecThreads), kDecSmemBytes, stream,
                 w13_fused.map_a, w13_fused.map_a32, w13_fused.map_b, w13_fused.map_b64, w2.map_a, w2.map_a32, w2.map_b,
                 params);
}

}  // namespace gv
