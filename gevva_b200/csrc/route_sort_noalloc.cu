// gevva_moe_route_sort_noalloc: the route sort for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs the MoE
// layer.  An inference server may hand every byte of device memory to its own arena
// at start-up (the reference does that with its weight arena and scratch pools,
// src/runtime.cpp:165-184), so nothing is left for a library to take; a serving loop
// may forbid cudaMalloc because it synchronises the whole device; a plug-in may live
// inside a framework that allows device memory only from the framework's allocator.
// The ordinary route sort keeps its working memory (per-chunk histograms, the tile
// list, the tile count) in the scratch a runner allocates at creation.  This variant
// keeps that working memory in a fixed array inside the library image instead, so a
// caller with nothing but its own input and output buffers can still sort routes.
//
// Rules that follow from the fixed array:
//   * it is sized for at most kNoAllocMaxTokens tokens; larger calls are refused;
//   * every GPU that loads the library carries the array until the process exits;
//   * all calls on one device share it, and it keeps whatever the last call left:
//     two calls whose kernels overlap on the GPU (different streams, no dependency)
//     race on it.  Nothing in it has to start at zero: each call first writes every
//     word it later reads;
//   * the first call on each device looks the array's device address up and caches
//     it.  With lazy module loading that call may also be the one at which the driver
//     places the library's device code and this array in device memory, so make it at
//     start-up: before the host's arena takes what memory is left, and outside any
//     stream capture.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/gevva_moe.h"
#include "gv_common.cuh"
#include "gv_launchers.h"

namespace {

constexpr int kNoAllocMaxTokens = 16384;
constexpr int kNoAllocMaxRoutes = kNoAllocMaxTokens * gv::kTopK;          // 131072
constexpr int kNoAllocChunks = (kNoAllocMaxRoutes + 1023) / 1024;         // 128
constexpr int kNoAllocTileCapacity = kNoAllocMaxRoutes / gv::kTileM + gv::kExperts + 1;
// Layout in ints: [chunk histograms][tile -> expert][tile count]
constexpr int kHistInts = kNoAllocChunks * gv::kExperts;
constexpr int kNoAllocInts = kHistInts + kNoAllocTileCapacity + 1;        // about 69 KiB

// In host code this name is only a handle for cudaGetSymbolAddress, never an address
// a kernel may be given.
static __device__ __align__(256) int g_route_sort_scratch[kNoAllocInts];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
int* g_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device; resolved once per device.
cudaError_t scratch_for_current_device(int** out) {
  int device = -1;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return error;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    int* address = nullptr;
    error = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_route_sort_scratch);
    if (error != cudaSuccess) return error;
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int gevva_moe_route_sort_noalloc(const int* expert_ids, int tokens, int* sorted_experts,
                                            int* sorted_routes, int* inverse_routes,
                                            int* expert_offsets, int* scale_row_offsets,
                                            int* status, gevva_stream_t stream) {
  if (!expert_ids || !sorted_experts || !sorted_routes || !inverse_routes || !expert_offsets ||
      !scale_row_offsets || !status || tokens < 1)
    return GEVVA_MOE_BAD_ARGUMENT;
  if (tokens > kNoAllocMaxTokens) return GEVVA_MOE_TOO_LARGE;
  int* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != cudaSuccess) return GEVVA_MOE_CUDA_ERROR;
  gv::RoutePlan plan{};
  plan.sorted_experts = sorted_experts;
  plan.sorted_routes = sorted_routes;
  plan.inverse_routes = inverse_routes;
  plan.expert_offsets = expert_offsets;
  plan.scale_row_offsets = scale_row_offsets;
  plan.chunk_hist = scratch;
  plan.tile_expert = scratch + kHistInts;
  plan.num_m_tiles = scratch + kHistInts + kNoAllocTileCapacity;
  plan.status = status;
  gv::launch_route_sort(expert_ids, tokens * gv::kTopK, plan, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}
