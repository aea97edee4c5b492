// Pieces shared by the grouped GEMM kernels (grouped_gemm.cu: one CTA per tile;
// grouped_gemm_pair.cu: a CTA pair per tile pair): the launch parameters, the epilogue arithmetic
// and the shared-memory staged store.
#pragma once

#include "gv_common.cuh"
#include "gv_launchers.h"

namespace gv {
namespace {

constexpr int kEpilogueWarpsPerQuarter = 4;  // each takes a quarter of a tile's columns
constexpr int kEpilogueThreads = 4 * kEpilogueWarpsPerQuarter * 32;
constexpr int kStoreColumns = 128;                        // columns per store pass (plain epilogue)
constexpr int kStageRowBytes = kStoreColumns * 2;         // one bf16 row of a store pass
constexpr int kStagingBytesPerWarp = 32 * kStageRowBytes; // 8 KiB

enum GemmMode { kPlain = 0, kGeglu = 1, kFp8 = 2 };  // kFp8: dense E4M3 operands, plain epilogue


struct GemmParams {
  const uint8_t* a_scales;
  const uint8_t* b_scales;   // kPlain: sidecar layout; kGeglu: re-tiled copy
  const float* alpha;
  __nv_bfloat16* out;        // kPlain
  const unsigned long long* row_dest;  // kPlain, optional: address of each output row (may be peer memory)
  uint8_t* next_codes;       // kGeglu: w2 operand codes [rows, 352]
  uint8_t* next_scales;      // kGeglu: w2 operand scale regions
  const float* next_scale_q; // kGeglu: g2.input_scale_quant [128]
  const int* tile_expert;
  const int* expert_offsets;
  const int* scale_row_offsets;
  const int* num_m_tiles;
  const int* tile_first;     // optional: first row tile of this launch
  int* status;
  int n_out;
  int n_tiles;      // work items per row tile
  int groups;       // k_in / 16
  int k_blocks;     // ceil(k_in / 256)
  int last_mmas;    // MMAs (K = 64 each) in the last K block, 1..4
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&pair);
}

// bf16 rounding of alpha*acc, returned as float: the value the reference's GEMM
// epilogue stores and its GeGLU kernel reads back (src/nvfp4_cutlass.cu:582-583).
__device__ __forceinline__ float round_through_bf16(float alpha, uint32_t acc_bits) {
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(acc_bits))));
}

// Plain epilogue, one store pass: this warp's 32 rows x 32 columns (already scaled and
// rounded) go to the quarter's staging tile (32 rows x 256 bytes), then the four warps of the
// quarter write the tile out so that every store instruction covers two full 256-byte row
// segments.  16-byte chunk c of row r lives at chunk position c ^ (r & 15), which keeps the
// row-wise writes and the two-rows-per-instruction reads at the minimum number of bank passes.
__device__ __forceinline__ void stage_and_store(const uint32_t (&r)[32], float alpha, uint8_t* staging,
                                                int quarter, int sub, int lane, int rows_valid,
                                                int row0, int column0, const GemmParams& p) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i])),
                      __fmul_rn(alpha, __uint_as_float(r[8 * i + 1])));
    v.y = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 2])),
                      __fmul_rn(alpha, __uint_as_float(r[8 * i + 3])));
    v.z = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 4])),
                      __fmul_rn(alpha, __uint_as_float(r[8 * i + 5])));
    v.w = pack_bf16x2(__fmul_rn(alpha, __uint_as_float(r[8 * i + 6])),
                      __fmul_rn(alpha, __uint_as_float(r[8 * i + 7])));
    const int c = sub * 4 + i;
    *reinterpret_cast<uint4*>(staging + lane * kStageRowBytes + ((c ^ (lane & 15)) << 4)) = v;
  }
  named_barrier(1 + quarter, kEpilogueWarpsPerQuarter * 32);
  const int c = lane & 15;
  __nv_bfloat16* dst = p.out + static_cast<size_t>(row0 + quarter * 32) * p.n_out + column0 + c * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r2 = 2 * (sub * 4 + i) + (lane >> 4);
    const uint4 v = *reinterpret_cast<const uint4*>(staging + r2 * kStageRowBytes + ((c ^ (r2 & 15)) << 4));
    if (quarter * 32 + r2 < rows_valid) {
      if (p.row_dest) {
        // expert-parallel combine: the row goes straight to its source rank's buffer
        __nv_bfloat16* remote = reinterpret_cast<__nv_bfloat16*>(p.row_dest[row0 + quarter * 32 + r2]);
        *reinterpret_cast<uint4*>(remote + column0 + c * 8) = v;
      } else {
        *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r2) * p.n_out) = v;
      }
    }
  }
  named_barrier(1 + quarter, kEpilogueWarpsPerQuarter * 32);  // staging is rewritten next pass
}

// Fused epilogue arithmetic for one 16-value block of one row.
__device__ __forceinline__ uint32_t geglu_block(const uint32_t (&up)[16], const uint32_t (&gate)[16],
                                                float alpha, float multiplier, const float* erf_table,
                                                uint32_t& codes_lo, uint32_t& codes_hi) {
  float values[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float g = round_through_bf16(alpha, gate[i]);
    const float u = round_through_bf16(alpha, up[i]);
    values[i] = __fmul_rn(gv_gelu_erf(g, erf_table), u);
  }
  return quantize_block16(values, multiplier, codes_lo, codes_hi);
}

constexpr int kFusedItems = (kInter + 127) / 128;  // 6


}  // namespace
}  // namespace gv
