// Group geometry shared by the route sort and the expert-parallel receive side.
#pragma once

#include "gv_common.cuh"
#include "gv_launchers.h"

namespace gv {

// Exclusive scans of the 128 expert counts and tile counts, and the outputs that
// depend only on them.  Called by threads 0..127 with `count` = rows of expert tid.
__device__ __forceinline__ int publish_groups(int count, int routes, const RoutePlan& plan,
                                              int* scan_scratch /* smem [16] */) {
  const int expert = threadIdx.x;
  const int lane = expert & 31, warp = expert >> 5;
  const int tiles = (count + kTileM - 1) / kTileM;
  const int pairs = (tiles + 1) / 2;
  int rows_inclusive = count, tiles_inclusive = tiles, pairs_inclusive = pairs;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const int r = __shfl_up_sync(0xffffffffu, rows_inclusive, offset);
    const int t = __shfl_up_sync(0xffffffffu, tiles_inclusive, offset);
    const int q = __shfl_up_sync(0xffffffffu, pairs_inclusive, offset);
    if (lane >= offset) {
      rows_inclusive += r;
      tiles_inclusive += t;
      pairs_inclusive += q;
    }
  }
  if (lane == 31) {
    scan_scratch[warp] = rows_inclusive;
    scan_scratch[4 + warp] = tiles_inclusive;
    scan_scratch[8 + warp] = pairs_inclusive;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // only the first four warps take part
  int row_base = 0, tile_base = 0, pair_base = 0;
  for (int w = 0; w < warp; ++w) {
    row_base += scan_scratch[w];
    tile_base += scan_scratch[4 + w];
    pair_base += scan_scratch[8 + w];
  }
  const int row_begin = row_base + rows_inclusive - count;
  const int tile_begin = tile_base + tiles_inclusive - tiles;
  if (plan.pair_tile) {
    const int pair_begin = pair_base + pairs_inclusive - pairs;
    for (int i = 0; i < pairs; ++i)
      plan.pair_tile[pair_begin + i] = 2 * (tile_begin + 2 * i) + (2 * i + 1 < tiles ? 1 : 0);
    if (expert == kExperts - 1) plan.num_pairs[0] = pair_begin + pairs;
  }
  plan.expert_offsets[expert] = row_begin;
  plan.scale_row_offsets[expert] = tile_begin * kTileM;
  for (int i = 0; i < tiles; ++i) plan.tile_expert[tile_begin + i] = expert;
  if (expert == kExperts - 1) {
    plan.expert_offsets[kExperts] = row_begin + count;
    plan.scale_row_offsets[kExperts] = (tile_begin + tiles) * kTileM;
    plan.num_m_tiles[0] = tile_begin + tiles;
  }
  (void)routes;
  return row_begin;
}

}  // namespace gv
