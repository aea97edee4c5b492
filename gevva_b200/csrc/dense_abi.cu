// C ABI of the dense FP8 GeGLU MLP and of the feed-forward steps before and after the
// expert path (declared in include/gevva_moe.h).  The reference runs the three dense
// projections through cuBLASLt (Fp8LinearRunner::launch_unscaled,
// src/cuda/runtime/fp8_linear.cuh:215-473, called at src/cuda/runtime/prefill.cuh:1211-1230);
// here they are the tcgen05 kernel of grouped_gemm.cu in its FP8 form.
#include <cuda.h>
#include <cuda_runtime.h>

#include <new>

#include "../../include/gevva_moe.h"
#include "gv_common.cuh"
#include "gv_launchers.h"

namespace {
constexpr int kDense = 2112;
}

struct gevva_dense {
  gevva_dense_weights weights{};
  int max_tokens = 0;
  int sm_count = 0;
  gv::RoutePlan plan{};
  gv::GemmOperands gate_up{}, down{};
  uint8_t* act_fp8 = nullptr;     // [T, 2816]
  float* act_scales = nullptr;    // [T]
  void* gate_up_out = nullptr;    // bf16 [T, 4224], unscaled
  uint8_t* prod_fp8 = nullptr;    // [T, 2112]
  float* prod_scales = nullptr;   // [T]
  float* ones = nullptr;          // [128]
  float* down_scale = nullptr;    // [1]: weights.down_scale on the device, for gevva_ff_finalize
  int* ints = nullptr;
};

extern "C" {

void gevva_dense_destroy(gevva_dense* d) {
  if (!d) return;
  cudaFree(d->act_fp8);
  cudaFree(d->act_scales);
  cudaFree(d->gate_up_out);
  cudaFree(d->prod_fp8);
  cudaFree(d->prod_scales);
  cudaFree(d->ones);
  cudaFree(d->down_scale);
  cudaFree(d->ints);
  delete d;
}

int gevva_dense_create(gevva_dense** out, const gevva_dense_weights* weights, int max_tokens) {
  if (!out || !weights || !weights->gate_up || !weights->down || max_tokens < 1) return GEVVA_MOE_BAD_ARGUMENT;
  if (max_tokens > 131072) return GEVVA_MOE_TOO_LARGE;
  cudaDeviceProp prop;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess)
    return GEVVA_MOE_CUDA_ERROR;
  if (prop.major != 10) return GEVVA_MOE_NO_DEVICE;
  if (gv::prepare_grouped_gemm() != 0) return GEVVA_MOE_CUDA_ERROR;
  gevva_dense* d = new (std::nothrow) gevva_dense;
  if (!d) return GEVVA_MOE_CUDA_ERROR;
  d->weights = *weights;
  d->max_tokens = max_tokens;
  d->sm_count = prop.multiProcessorCount;
  const size_t t = static_cast<size_t>(max_tokens);
  const size_t tiles = t / gv::kTileM + gv::kExperts + 1;
  const size_t int_count = 2 * (gv::kExperts + 1) + tiles + 2;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&d->act_fp8), t * gv::kHidden);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->act_scales), t * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&d->gate_up_out, t * 2 * kDense * 2);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->prod_fp8), t * kDense);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->prod_scales), t * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->ones), gv::kExperts * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->down_scale), sizeof(float));
  if (e == cudaSuccess)
    e = cudaMemcpy(d->down_scale, &weights->down_scale, sizeof(float), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->ints), int_count * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(d->ints, 0, int_count * sizeof(int));
  if (e == cudaSuccess) {
    float host_ones[gv::kExperts];
    for (float& v : host_ones) v = 1.0f;
    e = cudaMemcpy(d->ones, host_ones, sizeof(host_ones), cudaMemcpyHostToDevice);
  }
  if (e != cudaSuccess) {
    gevva_dense_destroy(d);
    return GEVVA_MOE_CUDA_ERROR;
  }
  int* cursor = d->ints;
  auto carve = [&](size_t n) { int* p = cursor; cursor += n; return p; };
  d->plan.expert_offsets = carve(gv::kExperts + 1);
  d->plan.scale_row_offsets = carve(gv::kExperts + 1);
  d->plan.tile_expert = carve(tiles);
  d->plan.num_m_tiles = carve(1);
  d->plan.status = carve(1);
  bool ok = true;
  ok = ok && gv::make_operand_tensor_map(&d->gate_up.map_a, d->act_fp8, t, gv::kHidden, gv::kTileM);
  ok = ok && gv::make_operand_tensor_map(&d->gate_up.map_a32, d->act_fp8, t, gv::kHidden, 32);
  ok = ok && gv::make_operand_tensor_map(&d->down.map_a32, d->prod_fp8, t, kDense, 32);
  ok = ok && gv::make_operand_tensor_map(&d->gate_up.map_b, weights->gate_up, 2 * kDense, gv::kHidden, gv::kTileM);
  ok = ok && gv::make_operand_tensor_map(&d->down.map_a, d->prod_fp8, t, kDense, gv::kTileM);
  ok = ok && gv::make_operand_tensor_map(&d->down.map_b, weights->down, gv::kHidden, kDense, gv::kTileM);
  if (!ok) {
    gevva_dense_destroy(d);
    return GEVVA_MOE_CUDA_ERROR;
  }
  d->gate_up.alpha = d->ones;
  d->gate_up.out = d->gate_up_out;
  d->gate_up.n_out = 2 * kDense;
  d->gate_up.k_in = gv::kHidden;
  d->gate_up.fp8 = true;
  d->down.alpha = d->ones;
  d->down.n_out = gv::kHidden;
  d->down.k_in = kDense;
  d->down.fp8 = true;
  *out = d;
  return GEVVA_MOE_OK;
}

int gevva_dense_launch(gevva_dense* d, const void* in, void* out_unscaled, int tokens,
                       gevva_stream_t stream) {
  if (!d || !in || !out_unscaled || tokens < 1 || tokens > d->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_dense_plan(tokens, d->plan, stream);
  gv::launch_fp8_quantize_rows(in, d->act_fp8, d->act_scales, tokens, stream);
  gv::launch_grouped_gemm(d->gate_up, d->plan, d->sm_count, stream);
  gv::launch_gelu_quantize_fp8(d->gate_up_out, d->act_scales, d->weights.gate_scale, d->weights.up_scale,
                               d->prod_fp8, d->prod_scales, tokens, stream);
  gv::GemmOperands down = d->down;
  down.out = out_unscaled;
  gv::launch_grouped_gemm(down, d->plan, d->sm_count, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

const float* gevva_dense_output_scales(const gevva_dense* d) { return d ? d->prod_scales : nullptr; }

const float* gevva_dense_projection_scale(const gevva_dense* d) { return d ? d->down_scale : nullptr; }

int gevva_dense_buffer(const gevva_dense* d, int which, void** ptr, size_t* bytes) {
  if (!d || !ptr || !bytes) return GEVVA_MOE_BAD_ARGUMENT;
  const size_t t = static_cast<size_t>(d->max_tokens);
  switch (which) {
    case 0: *ptr = d->act_fp8; *bytes = t * gv::kHidden; break;
    case 1: *ptr = d->act_scales; *bytes = t * 4; break;
    case 2: *ptr = d->gate_up_out; *bytes = t * 2 * kDense * 2; break;
    case 3: *ptr = d->prod_fp8; *bytes = t * kDense; break;
    case 4: *ptr = d->prod_scales; *bytes = t * 4; break;
    default: return GEVVA_MOE_BAD_ARGUMENT;
  }
  return GEVVA_MOE_OK;
}

int gevva_ff_prepare(const void* input, const void* dense_weight, const void* expert_weight,
                     const void* router_scale, void* dense_out, void* expert_out, void* router_out,
                     int rows, gevva_stream_t stream) {
  if (!input || !dense_weight || !expert_weight || !router_scale || !dense_out || !expert_out ||
      !router_out || rows < 0)
    return GEVVA_MOE_BAD_ARGUMENT;
  if (rows == 0) return GEVVA_MOE_OK;
  gv::launch_ff_prepare(input, dense_weight, expert_weight, router_scale, dense_out, expert_out, router_out,
                        rows, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

int gevva_ff_finalize(const void* dense, const void* dense_weight, const void* expert_routes,
                      const float* route_weights, const int* inverse_routes, const void* expert_weight,
                      const void* combined_weight, const void* residual, const void* layer_scalar,
                      void* output, int rows, const float* dense_activation_scales,
                      const float* dense_projection_scale, gevva_stream_t stream) {
  if (!dense || !dense_weight || !expert_routes || !route_weights || !expert_weight || !combined_weight ||
      !residual || !layer_scalar || !output || rows < 0 ||
      (dense_activation_scales != nullptr && dense_projection_scale == nullptr))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (rows == 0) return GEVVA_MOE_OK;
  gv::launch_ff_finalize(dense, dense_weight, expert_routes, route_weights, inverse_routes, expert_weight,
                         combined_weight, residual, layer_scalar, output, rows, dense_activation_scales,
                         dense_projection_scale, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

int gevva_pack_fp8(const float* weights, size_t count, void* out, float* scale, gevva_stream_t stream) {
  if (!weights || !out || !scale || count == 0) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_pack_fp8(weights, count, static_cast<uint8_t*>(out), scale, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

}  // extern "C"
