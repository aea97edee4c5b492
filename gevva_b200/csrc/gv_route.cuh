// Top-8 of a token's 128 router logits, softmax over the eight, per-expert scale: the body of
// the router kernel, shared by the stand-alone launch and by the fused projection kernel.
// Reference: route_128_top8_kernel, src/cuda/kernels/routing_sampling.cuh:396-431 (a 128-thread
// CTA and a CUB radix sort per token).  Here one warp owns one token: lane l holds the logits of
// experts 4l..4l+3, and eight rounds of redux.sync pick the maxima in the order a stable
// descending radix sort would (ties keep the lower expert index, -0 sorts as +0).
#pragma once

#include "gv_common.cuh"

namespace gv {

__device__ __forceinline__ uint32_t radix_key(float value) {
  uint32_t bits = __float_as_uint(value);
  if (bits == 0x80000000u) bits = 0;  // -0 sorts as +0
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// All 32 lanes of a warp call this with the same row; lanes 0..7 write the row's results.
__device__ __forceinline__ void route_top8_of_row(const float (&value)[4], int lane,
                                                  const __nv_bfloat16* __restrict__ expert_scale,
                                                  float* __restrict__ weights_row, int* __restrict__ ids_row) {
  uint32_t key[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) key[j] = radix_key(value[j]);
  uint32_t taken = 0;
  int my_id = 0;
  float my_key = 0.0f;
#pragma unroll 1
  for (int round = 0; round < kTopK; ++round) {
    uint32_t best_key = 0;
    uint32_t best_index = 0xffffffffu;
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      if (!((taken >> j) & 1u) && key[j] >= best_key) {  // descending j: ties keep the lower index
        best_key = key[j];
        best_index = 4u * lane + j;
      }
    }
    const uint32_t top_key = __reduce_max_sync(0xffffffffu, best_key);
    const uint32_t candidate = (best_index != 0xffffffffu && best_key == top_key) ? best_index
                                                                                  : 0xffffffffu;
    const uint32_t winner = __reduce_min_sync(0xffffffffu, candidate);
    const int owner = static_cast<int>(winner >> 2);
    const int slot = static_cast<int>(winner & 3u);
    float v = value[0];
    v = slot == 1 ? value[1] : v;
    v = slot == 2 ? value[2] : v;
    v = slot == 3 ? value[3] : v;
    v = __shfl_sync(0xffffffffu, v, owner);
    if (lane == owner) taken |= 1u << slot;
    if (lane == round) {
      my_id = static_cast<int>(winner);
      my_key = v;
    }
  }
  const float maximum = __shfl_sync(0xffffffffu, my_key, 0);
  const float e = lane < kTopK ? gv_expf(__fsub_rn(my_key, maximum)) : 0.0f;
  float ek[kTopK];
#pragma unroll
  for (int k = 0; k < kTopK; ++k) ek[k] = __shfl_sync(0xffffffffu, e, k);
  // Same association as the reference's shuffle-down tree over lanes 0..7.
  const float denominator =
      __fadd_rn(__fadd_rn(__fadd_rn(ek[0], ek[4]), __fadd_rn(ek[2], ek[6])),
                __fadd_rn(__fadd_rn(ek[1], ek[5]), __fadd_rn(ek[3], ek[7])));
  if (lane < kTopK) {
    ids_row[lane] = my_id;
    weights_row[lane] = __fmul_rn(__fdiv_rn(e, denominator), __bfloat162float(expert_scale[my_id]));
  }
}

}  // namespace gv
