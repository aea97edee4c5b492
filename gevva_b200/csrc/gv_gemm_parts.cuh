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
  unsigned long long keep_in_l2;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_in_l2));
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
        // The rows are read back by the weighted reduce (or the next stage) right after this
        // launch: ask L2 to keep them (without the hint the reduce finds 2 % of them there).
        asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(
                         dst + static_cast<size_t>(r2) * p.n_out),
                     "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(keep_in_l2)
                     : "memory");
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


// Instruction descriptor: E2M1 x E2M1 (format 1 in the mxf4 kinds), both K-major,
// UE4M3 scales (bit 23 clear), N at [17,23) in units of 8, M at [24,29) in units of 16,
// K = 64 (bit 31 clear), scale ids 0.
template <int kN>
constexpr uint32_t kInstrDesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kN >> 3) << 17) |
                                (static_cast<uint32_t>(kTileM >> 4) << 24);

// One K block's worth of tensor-core work, issued by two threads.  The scale copier issues
// kMmas scale-factor atom copies per operand half (shared -> tensor memory, issue_sf_copies); the
// MMA thread, once those have landed, issues kMmas MMAs of K = 64 (issue_mmas).  Everything is
// derived from 32-bit descriptor bases with immediate offsets so that an issuing thread spends
// a handful of integer instructions per tcgen05 instruction.
//   a_lo / b_lo     low words of the operand descriptors of this stage (address >> 4)
//   sfa_lo / sfb_lo low words of the scale-factor descriptors of this stage
//   hi_ab / hi_sf   high words (stride, version, swizzle) shared by all stages
// Scale columns of a K block in tensor memory: at N = 128, A of MMA j at +4j and B at +16+4j;
// at N = 256, A at +16j, B rows 0..127 at +16j+4, B rows 128..255 at +16j+8 (the second half of
// the weight scales lies 2 KiB = 128 descriptor units after the first in shared memory).
template <int kMmas, int kN>
__device__ __forceinline__ void issue_sf_copies(uint32_t tmem_sf, uint32_t sfa_lo, uint32_t sfb_lo, uint32_t hi_sf) {
  static_assert(kMmas >= 1 && kMmas <= 4, "a K block holds one to four MMAs");
#define GV_SF_OPERANDS ::"r"(tmem_sf), "r"(sfa_lo), "r"(sfb_lo), "r"(hi_sf) : "memory"
#define GV_SF_PROLOGUE "{\n\t.reg .b32 lo, ta;\n\t.reg .b64 d0;\n\t"
#define GV_SF_ONE(source, source_offset, column)                             \
  "add.u32 lo, " source ", " source_offset ";\n\t"                           \
  "mov.b64 d0, {lo, %3};\n\t"                                                \
  "add.u32 ta, %0, " column ";\n\t"                                          \
  "tcgen05.cp.cta_group::1.32x128b.warpx4 [ta], d0;\n\t"
  if constexpr (kN == 128) {
#define GV_SF_COPY(j) GV_SF_ONE("%1", #j "*32", #j "*4") GV_SF_ONE("%2", #j "*32", "16+" #j "*4")
    asm volatile(GV_SF_PROLOGUE GV_SF_COPY(0) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 2) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(1) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 3) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(2) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 4) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(3) "}" GV_SF_OPERANDS);
#undef GV_SF_COPY
  } else {
#define GV_SF_COPY(j)                                                        \
  GV_SF_ONE("%1", #j "*32", #j "*16") GV_SF_ONE("%2", #j "*32", "4+" #j "*16") \
  GV_SF_ONE("%2", "128+" #j "*32", "8+" #j "*16")
    asm volatile(GV_SF_PROLOGUE GV_SF_COPY(0) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 2) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(1) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 3) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(2) "}" GV_SF_OPERANDS);
    if constexpr (kMmas >= 4) asm volatile(GV_SF_PROLOGUE GV_SF_COPY(3) "}" GV_SF_OPERANDS);
#undef GV_SF_COPY
  }
#undef GV_SF_ONE
#undef GV_SF_PROLOGUE
#undef GV_SF_OPERANDS
}

template <int kMmas, int kN>
__device__ __forceinline__ void issue_mmas(uint32_t tmem_acc, uint32_t tmem_sf, uint32_t a_lo, uint32_t b_lo,
                                           uint32_t hi_ab, uint32_t accumulate) {
  static_assert(kMmas >= 1 && kMmas <= 4, "a K block holds one to four MMAs");
#define GV_OPERANDS                                                                                  \
  ::"r"(tmem_acc), "r"(tmem_sf), "r"(a_lo), "r"(b_lo), "r"(hi_ab), "r"(kInstrDesc<kN>), "r"(accumulate) \
  : "memory"
#define GV_PROLOGUE "{\n\t.reg .pred p, pt;\n\t.reg .b32 lo, ta, tb;\n\t.reg .b64 d0, d1;\n\t" \
                    "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
#define GV_MMA(j, step, sfb_column, pred)                                  \
  "add.u32 lo, %2, " #j "*2;\n\t"                                          \
  "mov.b64 d0, {lo, %4};\n\t"                                              \
  "add.u32 lo, %3, " #j "*2;\n\t"                                          \
  "mov.b64 d1, {lo, %4};\n\t"                                              \
  "add.u32 ta, %1, " #j "*" #step ";\n\t"                                  \
  "add.u32 tb, %1, " #j "*" #step "+" #sfb_column ";\n\t"                  \
  "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"      \
  " [%0], d0, d1, %5, [ta], [tb], " pred ";\n\t"
  if constexpr (kN == 128) {
    asm volatile(GV_PROLOGUE GV_MMA(0, 4, 16, "p") "}" GV_OPERANDS);
    if constexpr (kMmas >= 2) asm volatile(GV_PROLOGUE GV_MMA(1, 4, 16, "pt") "}" GV_OPERANDS);
    if constexpr (kMmas >= 3) asm volatile(GV_PROLOGUE GV_MMA(2, 4, 16, "pt") "}" GV_OPERANDS);
    if constexpr (kMmas >= 4) asm volatile(GV_PROLOGUE GV_MMA(3, 4, 16, "pt") "}" GV_OPERANDS);
  } else {
    asm volatile(GV_PROLOGUE GV_MMA(0, 16, 4, "p") "}" GV_OPERANDS);
    if constexpr (kMmas >= 2) asm volatile(GV_PROLOGUE GV_MMA(1, 16, 4, "pt") "}" GV_OPERANDS);
    if constexpr (kMmas >= 3) asm volatile(GV_PROLOGUE GV_MMA(2, 16, 4, "pt") "}" GV_OPERANDS);
    if constexpr (kMmas >= 4) asm volatile(GV_PROLOGUE GV_MMA(3, 16, 4, "pt") "}" GV_OPERANDS);
  }
#undef GV_MMA
#undef GV_OPERANDS
#undef GV_PROLOGUE
}


}  // namespace
}  // namespace gv
