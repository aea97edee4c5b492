// Device side of the input quantiser, shared by its own launches (moe_kernels.cu) and by the
// decode kernel that quantises its token itself (grouped_gemm_decode.cu).
#pragma once

#include "gv_common.cuh"

namespace gv {

constexpr int kQuantizeThreadsPerToken = kHidden / 32;  // 88 threads x 32 columns per token

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* out) {
  out[0] = __uint_as_float(raw.x << 16);
  out[1] = __uint_as_float(raw.x & 0xffff0000u);
  out[2] = __uint_as_float(raw.y << 16);
  out[3] = __uint_as_float(raw.y & 0xffff0000u);
  out[4] = __uint_as_float(raw.z << 16);
  out[5] = __uint_as_float(raw.z & 0xffff0000u);
  out[6] = __uint_as_float(raw.w << 16);
  out[7] = __uint_as_float(raw.w & 0xffff0000u);
}

// The per-route part of the input quantiser.  A thread owns kBlocks consecutive 16-value
// blocks of the token (2 or 4): `values` are its columns, `maximum` the block maxima, `part`
// its index along the row; route_* describe the token's eight routes.  With four blocks the
// thread owns one whole 4-byte word of the swizzled scale layout (the launchers use two).
template <int kBlocks>
__device__ __forceinline__ void quantize_routes_of_token(const float (&values)[16 * kBlocks],
                                                         const float (&maximum)[kBlocks], int part,
                                                         const int* route_row, const float* route_multiplier,
                                                         const unsigned long long* route_scale_base,
                                                         uint8_t* __restrict__ packed,
                                                         uint8_t* __restrict__ scales) {
  static_assert(kBlocks == 2 || kBlocks == 4, "two or four blocks per thread");
  unsigned long long keep_in_l2;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_in_l2));
  // scale groups kBlocks*part .. +kBlocks-1 lie in one 4-group word of the swizzled layout
  const unsigned scale_offset = kBlocks == 4
                                    ? static_cast<unsigned>(part) * 512u
                                    : static_cast<unsigned>(part >> 1) * 512u + static_cast<unsigned>(part & 1) * 2u;
  // Codes and scale bytes depend on the route only through its expert's static scale, so a
  // route whose scale equals the previous route's (bit for bit) reuses that result: with one
  // calibration scale shared by all experts the arithmetic runs once per token, with distinct
  // scales eight times.
  uint32_t codes[2 * kBlocks];
#pragma unroll
  for (int i = 0; i < 2 * kBlocks; ++i) codes[i] = 0;
  uint32_t scale_word = 0;
  uint32_t previous_bits = 0;
  bool have_previous = false;
  for (int k = 0; k < kTopK; ++k) {
    const int dst = route_row[k];
    if (dst < 0) continue;
    const float multiplier = route_multiplier[k];
    if (!have_previous || __float_as_uint(multiplier) != previous_bits) {
      have_previous = true;
      previous_bits = __float_as_uint(multiplier);
      scale_word = 0;
#pragma unroll
      for (int block = 0; block < kBlocks; ++block) {
        const float unrounded = __fdiv_rn(__fmul_rn(multiplier, maximum[block]), 6.0f);
        const uint32_t scale = encode_e4m3(unrounded);
        const float rounded = decode_e4m3(scale);
        const float inverse = rounded == 0.0f ? 0.0f : __fdiv_rn(multiplier, rounded);
        scale_word |= scale << (8 * block);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t word = 0;
#pragma unroll
          for (int pair = 0; pair < 4; ++pair)
            word |= encode_e2m1x2(__fmul_rn(values[16 * block + 8 * half + 2 * pair], inverse),
                                  __fmul_rn(values[16 * block + 8 * half + 2 * pair + 1], inverse))
                    << (8 * pair);
          codes[2 * block + half] = word;
        }
      }
    }
    uint4* row = reinterpret_cast<uint4*>(packed + static_cast<size_t>(dst) * (kHidden / 2)) + (kBlocks / 2) * part;
    // the codes are the w13 operand, read six times by the next launch: L2 is asked to keep them
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(row), "r"(codes[0]), "r"(codes[1]),
                 "r"(codes[2]), "r"(codes[3]), "l"(keep_in_l2)
                 : "memory");
    if constexpr (kBlocks == 4) {
      row[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
      *reinterpret_cast<uint32_t*>(scales + route_scale_base[k] + scale_offset) = scale_word;
    } else {
      // two neighbouring threads hold the four scale bytes of one aligned word: one store, kept in L2
      const uint32_t neighbour = __shfl_down_sync(__activemask(), scale_word, 1);
      if ((part & 1) == 0)
        asm volatile("st.global.L2::cache_hint.b32 [%0], %1, %2;" ::"l"(scales + route_scale_base[k] + scale_offset),
                     "r"((scale_word & 0xffffu) | (neighbour << 16)), "l"(keep_in_l2)
                     : "memory");
    }
  }
}

// This thread's 16*kBlocks columns of a token row and the block maxima.
template <int kBlocks>
__device__ __forceinline__ void load_token_columns(const __nv_bfloat16* __restrict__ input, int token, int part,
                                                   float (&values)[16 * kBlocks], float (&maximum)[kBlocks]) {
  const uint4* source =
      reinterpret_cast<const uint4*>(input + static_cast<size_t>(token) * kHidden) + 2 * kBlocks * part;
#pragma unroll
  for (int i = 0; i < 2 * kBlocks; ++i) unpack_bf16x8(__ldg(source + i), values + 8 * i);
#pragma unroll
  for (int block = 0; block < kBlocks; ++block) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(values[16 * block + i]));
    maximum[block] = m;
  }
}

}  // namespace gv
