// Top-8 of a token's 128 router logits, softmax over the eight, per-expert scale: the body of
// the router kernel, shared by the stand-alone launch and by the fused projection kernel.
// Reference: route_128_top8_kernel, src/cuda/kernels/routing_sampling.cuh:396-431 (a 128-thread
// CTA and a CUB radix sort per token).
//
// Here four adjacent lanes (a quad) own one token, 32 logits each.  A lane finds the eight
// largest of its 32 in registers (sorting networks without branches), then the quad exchanges and
// merges its four sorted lists.  Order is that of a stable descending radix sort
// on the float keys: every logit is a bf16 value, so its order is carried by 16 bits, and the
// composite (key16 << 7 | 127 - expert) makes ties fall to the lower expert index and all
// composites distinct; -0 sorts as +0.  (A warp-wide redux.sync arg-max per round, the earlier
// form, cost about 200 cycles per round and token.)
#pragma once

#include "gv_common.cuh"

namespace gv {

// Order-preserving 16-bit key of a bf16 bit pattern (larger value -> larger key).
__device__ __forceinline__ uint32_t route_key16(uint32_t bf16_bits) {
  if (bf16_bits == 0x8000u) bf16_bits = 0;  // -0 sorts as +0
  return (bf16_bits & 0x8000u) ? (~bf16_bits & 0xffffu) : (bf16_bits | 0x8000u);
}

__device__ __forceinline__ float route_value_of_key16(uint32_t key16) {
  const uint32_t bf16_bits = (key16 & 0x8000u) ? (key16 & 0x7fffu) : (~key16 & 0xffffu);
  return __uint_as_float(bf16_bits << 16);
}

// Compare-exchange: afterwards a >= b.
__device__ __forceinline__ void route_order(uint32_t& a, uint32_t& b) {
  const uint32_t hi = max(a, b);
  b = min(a, b);
  a = hi;
}

// The eight largest of two descending lists of eight, descending: max(a[i], b[7-i]) are those
// eight as a bitonic sequence, which three compare-exchange stages sort.
__device__ __forceinline__ void route_merge8(uint32_t (&a)[kTopK], const uint32_t (&b)[kTopK]) {
#pragma unroll
  for (int i = 0; i < kTopK; ++i) a[i] = max(a[i], b[kTopK - 1 - i]);
#pragma unroll
  for (int distance = 4; distance >= 1; distance >>= 1) {
#pragma unroll
    for (int i = 0; i < kTopK; ++i)
      if ((i & distance) == 0) route_order(a[i], a[i + distance]);
  }
}

// The four lanes of a quad (lanes 4q..4q+3 of a warp, `part` = lane & 3) call this together.
// `packed` holds this lane's 32 logits as bf16 pairs: experts 32*part + 2i (low half) and
// 32*part + 2i + 1 (high half) in packed[i].  With `rescale` the key of a logit is
// bf16(logit * rescale) (the FP8 router's per-row scale, routing_sampling.cuh:405-411).
// Every lane of the warp must call (shuffles use the full mask); a quad whose token does not
// exist passes valid = false and writes nothing.  Lane `part` writes results 2*part and 2*part + 1.
//
// Dependent steps are kept few: a lane sorts four groups of eight logits independently (insertion
// networks side by side), merges them pairwise, then the quad exchanges whole lists (xor 1, then
// xor 2) and every lane merges, so all four lanes end with the same eight winners.
__device__ __forceinline__ void route_top8_quad(const uint32_t (&packed)[16], int part, bool use_rescale,
                                                float rescale, bool valid,
                                                const __nv_bfloat16* __restrict__ expert_scale,
                                                float* __restrict__ weights_row, int* __restrict__ ids_row) {
  uint32_t list[4][kTopK];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
#pragma unroll
    for (int i = 0; i < kTopK; ++i) {
      const int e = 8 * g + i;
      uint32_t bits = (e & 1) ? (packed[e >> 1] >> 16) : (packed[e >> 1] & 0xffffu);
      if (use_rescale) {
        const float scaled = __fmul_rn(__uint_as_float(bits << 16), rescale);
        bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(scaled)));
      }
      // composites are distinct (the expert index is part of them) and at least 1
      uint32_t c = ((route_key16(bits) << 7) | static_cast<uint32_t>(127 - (32 * part + e))) + 1u;
      // insert into the descending list of the i elements seen so far
#pragma unroll
      for (int k = 0; k < i; ++k) route_order(list[g][k], c);
      list[g][i] = c;
    }
  }
  route_merge8(list[0], list[1]);
  route_merge8(list[2], list[3]);
  route_merge8(list[0], list[2]);
  uint32_t (&winner)[kTopK] = list[0];
#pragma unroll
  for (int step = 1; step <= 2; ++step) {
    uint32_t other[kTopK];
#pragma unroll
    for (int k = 0; k < kTopK; ++k) other[k] = __shfl_xor_sync(0xffffffffu, winner[k], step);
    route_merge8(winner, other);
  }
  float value[kTopK];
  int id[kTopK];
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    const uint32_t c = winner[k] - 1u;
    id[k] = 127 - static_cast<int>(c & 127u);
    value[k] = route_value_of_key16(c >> 7);
  }
  float e[kTopK];
#pragma unroll
  for (int k = 0; k < kTopK; ++k) e[k] = gv_expf(__fsub_rn(value[k], value[0]));
  // Same association as the reference's shuffle-down tree over lanes 0..7.
  const float denominator = __fadd_rn(__fadd_rn(__fadd_rn(e[0], e[4]), __fadd_rn(e[2], e[6])),
                                      __fadd_rn(__fadd_rn(e[1], e[5]), __fadd_rn(e[3], e[7])));
  if (valid) {
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
      if ((k >> 1) == part) {
        ids_row[k] = id[k];
        weights_row[k] = __fmul_rn(__fdiv_rn(e[k], denominator), __bfloat162float(expert_scale[id[k]]));
      }
    }
  }
}

}  // namespace gv
