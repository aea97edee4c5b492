// TEST INFRASTRUCTURE ONLY.  Host launchers around the reference's own stage kernels
// (route_128_top8_kernel, the route sorts, quantize_bf16_sorted_moe,
// geglu_quantize_sorted_moe, reduce_expert_routes), which the Makefile cuts out of the mounted
// reference tree and hands in through GV_REF_STAGE_KERNELS.  The kernels are compiled as they
// stand; only the four CUTLASS type names in their signatures are given plain stand-ins of the
// same size, and launch shapes follow the reference's call sites
// (src/nvfp4_cutlass.cu:870-912, :1840-1885; src/cuda/runtime/prefill.cuh:420-422).
// Every pointer is a device pointer.  Each call runs `repeats` times on the default stream,
// synchronises and returns the mean time of one run in milliseconds (negative on a CUDA error),
// so a parity test also yields the reference stage's time on the same GPU.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cub/block/block_radix_sort.cuh>
#include <cub/device/device_radix_sort.cuh>

#include <cstddef>
#include <cstdint>

namespace gv_ref {

// Stand-ins for cute::Shape<int,int,int>, cutlass::float_e2m1_t, float_ue4m3_t, bfloat16_t.
struct Shape3 {
  std::int32_t m, n, k;
};
using ElementType = std::uint8_t;
using ElementSF = std::uint8_t;
using ElementD = __nv_bfloat16;
constexpr int kExperts = 128;

#include GV_REF_STAGE_KERNELS

namespace {

// Pointer tables the sort/configure kernels fill for the reference's CUTLASS plan; nothing
// here reads them back.
struct Tables {
  Shape3* shapes = nullptr;
  const ElementType** a = nullptr;
  const ElementSF** sfa = nullptr;
  ElementD** d = nullptr;
  int* route_indices = nullptr;
  void* sort_workspace = nullptr;
  std::size_t sort_workspace_bytes = 0;
  std::size_t route_capacity = 0;
};

Tables& tables() {
  static Tables t;
  if (!t.shapes) {
    cudaMalloc(reinterpret_cast<void**>(&t.shapes), kExperts * sizeof(Shape3));
    cudaMalloc(reinterpret_cast<void**>(&t.a), kExperts * sizeof(void*));
    cudaMalloc(reinterpret_cast<void**>(&t.sfa), kExperts * sizeof(void*));
    cudaMalloc(reinterpret_cast<void**>(&t.d), kExperts * sizeof(void*));
  }
  return t;
}

template <class Launch>
float timed(int repeats, Launch&& launch) {
  if (repeats < 1) repeats = 1;
  cudaEvent_t begin, end;
  cudaEventCreate(&begin);
  cudaEventCreate(&end);
  cudaEventRecord(begin, nullptr);
  for (int i = 0; i < repeats; ++i) launch();
  cudaEventRecord(end, nullptr);
  const cudaError_t error = cudaDeviceSynchronize();
  float ms = 0.0f;
  cudaEventElapsedTime(&ms, begin, end);
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  if (error != cudaSuccess || cudaGetLastError() != cudaSuccess) return -1.0f;
  return ms / repeats;
}

}  // namespace
}  // namespace gv_ref

extern "C" {

// 1 when the library was compiled with --use_fast_math, as the reference's own build is.
int ref_fast_math(void) {
#ifdef __FAST_MATH__
  return 1;
#else
  return 0;
#endif
}

// logits bf16 [rows,128] (contiguous), launch shape of prefill.cuh:420-422.
float ref_route(const void* logits, const void* expert_scale, float* weights, int* ids, int rows,
                const float* activation_scales, const float* projection_weight_scale, int repeats) {
  return gv_ref::timed(repeats, [&] {
    gv_ref::route_128_top8_kernel<<<rows, 128>>>(static_cast<const __nv_bfloat16*>(logits),
                                                static_cast<const __nv_bfloat16*>(expert_scale), weights, ids,
                                                rows, activation_scales, projection_weight_scale);
  });
}

// variant 0: bitonic network (routes <= 128); 1: counting sort (routes <= 320); 2: one-block
// radix sort (routes <= 4096); 3: device-wide radix sort + configure (any size; the inverse map
// is then written by ref_quantize, as in the reference).  Returns < 0 for a size the variant
// does not take.
float ref_sort(const int* expert_ids, int routes, int variant, int* sorted_experts, int* sorted_routes,
               int* inverse_routes, int* offsets, int* scale_row_offsets, int repeats) {
  using namespace gv_ref;
  Tables& t = tables();
  const int limits[4] = {128, 320, 4096, 1 << 30};
  if (variant < 0 || variant > 3 || routes < 1 || routes > limits[variant]) return -2.0f;
  if (variant == 3) {
    if (static_cast<std::size_t>(routes) > t.route_capacity) {
      cudaFree(t.route_indices);
      cudaFree(t.sort_workspace);
      cudaMalloc(reinterpret_cast<void**>(&t.route_indices), sizeof(int) * routes);
      t.sort_workspace_bytes = 0;
      cub::DeviceRadixSort::SortPairs(nullptr, t.sort_workspace_bytes, expert_ids, sorted_experts,
                                      t.route_indices, sorted_routes, routes, 0, 7, nullptr);
      cudaMalloc(&t.sort_workspace, t.sort_workspace_bytes);
      t.route_capacity = routes;
    }
    initialize_route_indices<<<(routes + 255) / 256, 256>>>(t.route_indices, routes);
  }
  return timed(repeats, [&] {
    if (variant == 0)
      sort_and_configure_dynamic_grouped<<<1, kExperts>>>(expert_ids, routes, 1408, 2816, t.shapes, offsets, t.a,
                                                          t.sfa, t.d, nullptr, nullptr, nullptr, scale_row_offsets,
                                                          sorted_experts, sorted_routes, inverse_routes);
    else if (variant == 1)
      count_sort_and_configure_dynamic_grouped<<<1, 512>>>(expert_ids, routes, 1408, 2816, t.shapes, offsets, t.a,
                                                           t.sfa, t.d, nullptr, nullptr, nullptr,
                                                           scale_row_offsets, sorted_experts, sorted_routes,
                                                           inverse_routes);
    else if (variant == 2)
      block_sort_and_configure_dynamic_grouped<<<1, 256>>>(expert_ids, routes, 1408, 2816, t.shapes, offsets, t.a,
                                                           t.sfa, t.d, nullptr, nullptr, nullptr,
                                                           scale_row_offsets, sorted_experts, sorted_routes,
                                                           inverse_routes);
    else {
      std::size_t bytes = t.sort_workspace_bytes;
      cub::DeviceRadixSort::SortPairs(t.sort_workspace, bytes, expert_ids, sorted_experts, t.route_indices,
                                      sorted_routes, routes, 0, 7, nullptr);
      configure_dynamic_grouped<<<1, kExperts>>>(sorted_experts, routes, 1408, 2816, t.shapes, offsets, t.a,
                                                 t.sfa, t.d, nullptr, nullptr, nullptr, scale_row_offsets);
    }
  });
}

// Launch shape of src/nvfp4_cutlass.cu:1869-1873.  inverse_routes may be null.
float ref_quantize(const void* input, const float* input_scale_quant, const int* sorted_experts,
                   const int* sorted_routes, const int* offsets, std::uint8_t* packed,
                   std::uint8_t* scale_factors, const int* scale_row_offsets, int width, int routes,
                   int* inverse_routes, int repeats) {
  return gv_ref::timed(repeats, [&] {
    gv_ref::quantize_bf16_sorted_moe<<<routes, width / 16>>>(static_cast<const __nv_bfloat16*>(input),
                                                            input_scale_quant, sorted_experts, sorted_routes,
                                                            offsets, packed, scale_factors, scale_row_offsets,
                                                            width, routes, inverse_routes);
  });
}

// Launch shape of src/nvfp4_cutlass.cu:908-911.
float ref_geglu(const void* fused, const float* input_scale_quant, const int* sorted_experts,
                const int* offsets, std::uint8_t* packed, std::uint8_t* scale_factors,
                const int* scale_row_offsets, int routes, int repeats) {
  using namespace gv_ref;
  Tables& t = tables();
  return timed(repeats, [&] {
    geglu_quantize_sorted_moe<<<routes, kExperts>>>(static_cast<const __nv_bfloat16*>(fused), input_scale_quant,
                                                    sorted_experts, offsets, packed, scale_factors,
                                                    scale_row_offsets, routes, 2816, t.shapes, t.a, t.sfa, t.d,
                                                    nullptr);
  });
}

// Launch shape of src/nvfp4_cutlass.cu:1882-1884.
float ref_reduce(const void* routes, const float* route_weights, void* output, int tokens,
                 const int* inverse_routes, int repeats) {
  return gv_ref::timed(repeats, [&] {
    gv_ref::reduce_expert_routes<<<tokens, 256>>>(static_cast<const __nv_bfloat16*>(routes), route_weights,
                                                 static_cast<__nv_bfloat16*>(output), tokens, inverse_routes);
  });
}

}  // extern "C"
