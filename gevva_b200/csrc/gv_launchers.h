// Host-callable launchers of the MoE kernels; every one only enqueues on `stream`.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace gv {

// Device-resident description of one launch's routing, written by the route sort
// and read by every later stage without a host round trip.
struct RoutePlan {
  int* sorted_experts;     // [R]   expert of sorted row
  int* sorted_routes;      // [R]   original route (8*token+k) of sorted row
  int* inverse_routes;     // [R]   sorted row of original route
  int* expert_offsets;     // [129] first sorted row of each expert, [128] = R
  int* scale_row_offsets;  // [129] first scale-factor row (128-row padded) of each expert
  int* tile_expert;        // [R/128 + 128] expert of each 128-row tile
  int* num_m_tiles;        // [1]
  int* pair_tile;          // optional [R/128 + 128]: 2 * (first tile of a pair) + (1 if the pair has two
                           // tiles); a pair = two consecutive 128-row tiles of one expert, or its last odd one
  int* num_pairs;          // optional [1]
  int* tile_ready;         // optional [R/128 + 128]: per row tile, epilogue warps of its w13 items that have
                           // stored their share of the w2 operand (merged decode kernel); zeroed by the sort
  const int* tile_first;   // optional [1]: a GEMM launch covers tiles [tile_first, tile_first + num_m_tiles)
  int* chunk_hist;         // [ceil(R/1024) * 128] scratch of the multi-block sort
  int* status;             // [1]   device status word (gv::Status)
  const int* remap;        // optional [128]: sort key = remap[expert id] (expert-parallel placement)
  int* sync;               // optional [2], zero on entry: arrival/departure counters of the one-launch sort
  int* front_sync;         // optional [2], zero on entry and on exit: tokens quantised / CTAs finished, of the
                           // decode kernel that sorts and quantises by itself
};

void launch_route(const void* logits_bf16, int ld, const void* expert_scale_bf16, float* weights,
                  int* ids, int tokens, const float* activation_scales,
                  const float* projection_weight_scale, cudaStream_t stream);

// Router projection fused with routing: x [tokens, 2816] (bf16, or E4M3 with per-row scales) times
// router_w [128, 2816]^T, optional f32 bias, bf16 rounding, top-8 + softmax.  Returns a cudaError_t value.
int launch_route_project(const void* x, const void* router_w, bool fp8, const float* bias,
                         const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                         const float* activation_scales, const float* weight_scale, int tokens, int* status,
                         cudaStream_t stream);

void launch_route_sort(const int* expert_ids, int routes, const RoutePlan& plan,
                       cudaStream_t stream);

// Route sort and input quantiser in one launch; at most 128 tokens (1024 routes).
constexpr int kFusedSortQuantizeMaxTokens = 128;
void launch_route_sort_quantize_small(const void* input_bf16, const int* expert_ids, const float* in_scale_q,
                                      const RoutePlan& plan, int tokens, uint8_t* packed, uint8_t* scales,
                                      cudaStream_t stream);

// bf16 [tokens, 2816] -> codes [R, 1408] (sorted order) + swizzled scale bytes.
void launch_quantize_input(const void* input_bf16, const int* expert_ids, const float* in_scale_q,
                           const RoutePlan& plan, int tokens, uint8_t* packed, uint8_t* scales,
                           cudaStream_t stream);

// bf16 [R, 1408] ([up;gate]) -> codes [R, 352] + swizzled scale bytes.
void launch_geglu_quantize(const void* fused_bf16, const float* in_scale_q, const RoutePlan& plan,
                           int routes, uint8_t* packed, uint8_t* scales, cudaStream_t stream);

void launch_reduce_routes(const void* routed_bf16, const float* route_weights,
                          const int* inverse_routes, int tokens, void* output_bf16,
                          cudaStream_t stream);

// Grouped NVFP4 GEMM: out[r, n] = bf16(alpha[e] * sum_k A[r,k] B[e,n,k]).
struct GemmOperands {
  CUtensorMap map_a;        // [row capacity, K/2] bytes, box 128 x 128 B, 128B swizzle
  CUtensorMap map_a32;      // same matrix through a 32-row box (groups of at most 32 rows)
  CUtensorMap map_b;        // [128*N, K/2] bytes, same box
  CUtensorMap map_b64;      // fused w13 form only: the same matrix through a 64-row box
  CUtensorMap map_a_sf;     // CTA-pair form: a_scales as [atoms of 512 B][128 x u32], box of four atoms
  CUtensorMap map_b_sf;     // CTA-pair form: b_scales likewise; box of eight atoms (fused w13) or four (w2)
  const uint8_t* a_scales;  // activation scale regions
  const uint8_t* b_scales;  // [128, N, K/16] swizzled per expert
  const float* alpha;       // [128]
  void* out;                // bf16 [row capacity, N]
  const unsigned long long* row_dest;  // optional: per-row output address instead of `out`
  int n_out;                // N: 1408 or 2816
  int k_in;                 // K: 2816 or 704
  // Fused w13 form (GeGLU + requantise in the epilogue, no bf16 output): b_scales is the
  // re-tiled copy made by launch_retile_w13_scales, map_b64 serves the last, half-filled item
  // of each row tile, and the results go to the w2 operand buffers below.
  bool fused_geglu;
  bool serial_launch;         // launch the ordinary way: no start before the stream's previous kernel ends
  bool use_pairs;             // NVFP4 forms with 256 weight rows per item: run as CTA pairs (tcgen05 cta_group::2)
                              // when the plan carries a pair list
  bool fp8;                   // dense E4M3 x E4M3 (no block scales); k_in counts bytes = elements
  uint8_t* next_codes;        // [row capacity, 352]
  uint8_t* next_scales;       // scale regions of the w2 operand
  const float* next_scale_q;  // g2.input_scale_quant [128]
};

void launch_grouped_gemm(const GemmOperands& op, const RoutePlan& plan, int sm_count,
                         cudaStream_t stream);

// w13 block scales [128,1408,176] (sidecar layout) -> per-item atoms for the fused form.
size_t retiled_w13_scale_bytes(int experts);
void launch_retile_w13_scales(const uint8_t* sidecar_scales, uint8_t* tiled, int experts,
                              cudaStream_t stream);

// Byte matrix [rows, row_bytes] seen through a box of box_rows x 128 bytes with the 128-byte
// swizzle; bytes out of range read as zero.  False if the driver entry point is missing.
bool make_operand_tensor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                             int box_rows);

// Scale-factor bytes seen as rows of one 512-byte atom each (128 x u32), through a box of
// `box_atoms` consecutive atoms; no swizzle.
bool make_scale_tensor_map(CUtensorMap* map, const void* base, uint64_t bytes, int box_atoms);

// The CTA-pair form (grouped_gemm_pair.cu): fused w13 (op.fused_geglu) or plain w2 (n_out % 256 == 0).
void launch_grouped_gemm_pairs(const GemmOperands& op, const RoutePlan& plan, int sm_count, cudaStream_t stream);
int prepare_grouped_gemm_pairs();

// Fused w13 + GeGLU + requantise run by CTA pairs with the weights on the MMA's M side and up to
// 256 rows of one expert on its N side (grouped_gemm_w13_pair.cu); needs the plan's tile-pair list.
struct W13PairOperands {
  CUtensorMap map_x[16];  // activation codes [row capacity, 1408] bytes through boxes of 8, 16, ... 128 rows x 128 B
  CUtensorMap map_w;      // w13 codes as [experts * 2 halves, 704 rows, 1408] bytes, box 2 x 64 rows x 128 B: the
                          // up rows and the gate rows of one unit in one copy
  CUtensorMap map_x_sf;   // activation scale regions as [128-row blocks, 44 atoms, 512 B], box 2 blocks x 4 atoms
  CUtensorMap map_w_sf;   // unit-tiled weight scales (launch_retile_w13_unit_scales), box of four atoms
  const float* alpha;           // [experts]
  uint8_t* next_codes;          // [row capacity, 352]
  uint8_t* next_scales;         // scale regions of the w2 operand
  const float* next_scale_q;    // [experts]
  bool serial_launch;
};
size_t w13_unit_scale_bytes(int experts);
void launch_retile_w13_unit_scales(const uint8_t* sidecar_scales, uint8_t* tiled, int experts, cudaStream_t stream);
void launch_w13_pairs(const W13PairOperands& op, const RoutePlan& plan, int sm_count, cudaStream_t stream);
int prepare_w13_pairs();

// Both expert GEMMs of a batch of at most 128 tokens in one persistent launch (grouped_gemm_decode.cu):
// the fused w13 form, then w2, with per-tile readiness counters (plan.tile_ready) in between.
void launch_decode_experts(const GemmOperands& w13_fused, const GemmOperands& w2, const RoutePlan& plan,
                           int sm_count, cudaStream_t stream);
// The same with the route sort and the input quantiser inside (needs plan.front_sync and
// tokens <= min(128, sm_count)): a decode layer step without the router and the reduce.
void launch_decode_layer(const void* input_bf16, const int* expert_ids, const float* in_scale_q, int tokens,
                         uint8_t* packed, uint8_t* scales, const GemmOperands& w13_fused, const GemmOperands& w2,
                         const RoutePlan& plan, int sm_count, cudaStream_t stream);
int prepare_decode_experts();

// Must be called once per device before launch_grouped_gemm (sets the dynamic
// shared-memory limit).  Returns a cudaError_t value.
int prepare_grouped_gemm();

// Synthetic-expert packer: fp32 [experts, N, K] -> NVFP4 codes, swizzled scale
// bytes and the per-expert global scale amax/(6*448).
void launch_pack_weights(const float* weights, int experts, int n_out, int k_in, uint8_t* codes,
                         uint8_t* scales, float* global_scales, cudaStream_t stream);

// ---- feed-forward steps around the expert path and the dense FP8 MLP (dense_ff.cu) ------
void launch_ff_prepare(const void* input, const void* dense_weight, const void* expert_weight,
                       const void* router_scale, void* dense_out, void* expert_out, void* router_out,
                       int rows, cudaStream_t stream);
void launch_fp8_quantize_rows(const void* input, uint8_t* out, float* scales, int rows,
                              cudaStream_t stream);
void launch_gelu_quantize_fp8(const void* gate_up, const float* activation_scales, float gate_w_scale,
                              float up_w_scale, uint8_t* out, float* scales, int rows,
                              cudaStream_t stream);
void launch_ff_finalize(const void* dense, const void* dense_weight, const void* expert_routes,
                        const float* route_weights, const int* inverse_routes, const void* expert_weight,
                        const void* combined_weight, const void* residual, const void* layer_scalar,
                        void* output, int rows, const float* dense_activation_scales,
                        const float* dense_projection_scale, cudaStream_t stream);
void launch_dense_plan(int rows, const RoutePlan& plan, cudaStream_t stream);
void launch_pack_fp8(const float* w, size_t count, uint8_t* out, float* scale_out, cudaStream_t stream);

}  // namespace gv
