// Router, route sort, NVFP4 quantisers, weighted reduce and the synthetic weight
// packer: the HBM-bound stages around the two grouped GEMMs.
//
// Arithmetic that decides a code or a scale byte is written with explicit
// round-to-nearest intrinsics so that it equals the IEEE statement of the
// reference kernels (src/nvfp4_cutlass.cu:290-327, :552-601) bit for bit.
#include "gv_common.cuh"
#include "gv_launchers.h"
#include "gv_plan.cuh"
#include "gv_quantize.cuh"
#include "gv_route.cuh"

namespace gv {

// ---------------------------------------------------------------------------
// Router: top-8 of 128 logits + softmax over the eight + per-expert scale.
// Reference: route_128_top8_kernel, src/cuda/kernels/routing_sampling.cuh:396-431
// (a 128-thread CTA and a full CUB radix sort per token).  Here four lanes own one
// token (gv_route.cuh): 32 tokens per CTA of 128 threads.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
route_128_top8_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                      const __nv_bfloat16* __restrict__ expert_scale, float* __restrict__ weights,
                      int* __restrict__ ids, int rows, const float* __restrict__ activation_scales,
                      const float* __restrict__ projection_weight_scale) {
  const int row = blockIdx.x * 32 + (threadIdx.x >> 2);
  const int part = threadIdx.x & 3;
  const bool valid = row < rows;
  const int safe_row = valid ? row : 0;
  const uint16_t* src = reinterpret_cast<const uint16_t*>(logits) + static_cast<size_t>(safe_row) * ld + 32 * part;
  uint32_t packed[16];
  if ((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && (ld & 7) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + i);
      packed[4 * i] = v.x;
      packed[4 * i + 1] = v.y;
      packed[4 * i + 2] = v.z;
      packed[4 * i + 3] = v.w;
    }
  } else {  // a view whose rows are not 16-byte aligned
#pragma unroll
    for (int i = 0; i < 16; ++i)
      packed[i] = static_cast<uint32_t>(src[2 * i]) | (static_cast<uint32_t>(src[2 * i + 1]) << 16);
  }
  float rescale = 1.0f;
  if (activation_scales) rescale = __fmul_rn(activation_scales[safe_row], projection_weight_scale[0]);
  route_top8_quad(packed, part, activation_scales != nullptr, rescale, valid, expert_scale,
                  weights + static_cast<size_t>(safe_row) * kTopK, ids + static_cast<size_t>(safe_row) * kTopK);
}

void launch_route(const void* logits_bf16, int ld, const void* expert_scale_bf16, float* weights,
                  int* ids, int tokens, const float* activation_scales,
                  const float* projection_weight_scale, cudaStream_t stream) {
  route_128_top8_kernel<<<(tokens + 31) / 32, 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(logits_bf16), ld,
      static_cast<const __nv_bfloat16*>(expert_scale_bf16), weights, ids, tokens, activation_scales,
      projection_weight_scale);
}

// ---------------------------------------------------------------------------
// Route sort: stable counting sort of R = 8*T routes by expert, plus the group
// geometry every later stage reads.  Reference: four variants at
// src/nvfp4_cutlass.cu:329-550 (one CTA, or cub::DeviceRadixSort above 2560
// routes).  Here: chunks of 1024 routes; per chunk, per-warp match_any counts give
// each route its stable rank; chunks are chained by a 128-thread prefix kernel.
// ---------------------------------------------------------------------------
constexpr int kSortChunk = 1024;

// Per-warp population of each expert inside a 1024-route chunk.  `warp_counts`
// must be zero on entry.  Returns the lanes of this warp that share this lane's expert.
__device__ __forceinline__ uint32_t count_chunk(int expert, int* warp_counts) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t peers = __match_any_sync(0xffffffffu, expert);
  if (expert < kExperts && (peers & (0u - peers)) == (1u << lane))
    warp_counts[warp * kExperts + expert] = __popc(peers);
  return peers;
}

__global__ void __launch_bounds__(kSortChunk)
route_sort_single_kernel(const int* __restrict__ expert_ids, int routes, RoutePlan plan) {
  grid_launch_dependents();
  __shared__ int warp_counts[32 * kExperts];
  __shared__ int begins[kExperts];
  __shared__ int scan_scratch[16];
  const int tid = threadIdx.x;
  for (int i = tid; i < 32 * kExperts; i += kSortChunk) warp_counts[i] = 0;
  __syncthreads();
  int expert = kExperts;
  if (tid < routes) {
    expert = expert_ids[tid];
    if (expert < 0 || expert >= kExperts) {
      atomicExch(plan.status, static_cast<int>(kBadExpertId));
      expert = kExperts;
    } else if (plan.remap) {
      expert = plan.remap[expert];
    }
  }
  const uint32_t peers = count_chunk(expert, warp_counts);
  __syncthreads();
  if (tid < kExperts) {
    int running = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = warp_counts[w * kExperts + tid];
      warp_counts[w * kExperts + tid] = running;
      running += c;
    }
    begins[tid] = publish_groups(running, routes, plan, scan_scratch);
  }
  __syncthreads();
  if (expert < kExperts) {
    const int lane = tid & 31, warp = tid >> 5;
    const int dst = begins[expert] + warp_counts[warp * kExperts + expert] +
                    __popc(peers & ((1u << lane) - 1u));
    plan.sorted_experts[dst] = expert;
    plan.sorted_routes[dst] = tid;
    plan.inverse_routes[tid] = dst;
  }
}

__global__ void __launch_bounds__(kSortChunk)
route_histogram_kernel(const int* __restrict__ expert_ids, int routes, RoutePlan plan) {
  __shared__ int warp_counts[32 * kExperts];
  const int tid = threadIdx.x;
  for (int i = tid; i < 32 * kExperts; i += kSortChunk) warp_counts[i] = 0;
  __syncthreads();
  const int route = blockIdx.x * kSortChunk + tid;
  int expert = kExperts;
  if (route < routes) {
    expert = expert_ids[route];
    if (expert < 0 || expert >= kExperts) {
      atomicExch(plan.status, static_cast<int>(kBadExpertId));
      expert = kExperts;
    } else if (plan.remap) {
      expert = plan.remap[expert];
    }
  }
  count_chunk(expert, warp_counts);
  __syncthreads();
  if (tid < kExperts) {
    int total = 0;
    for (int w = 0; w < 32; ++w) total += warp_counts[w * kExperts + tid];
    plan.chunk_hist[blockIdx.x * kExperts + tid] = total;
  }
}

__global__ void __launch_bounds__(kExperts)
route_prefix_kernel(int chunks, int routes, RoutePlan plan) {
  __shared__ int scan_scratch[16];
  const int expert = threadIdx.x;
  int running = 0;
  for (int c = 0; c < chunks; ++c) {
    const int v = plan.chunk_hist[c * kExperts + expert];
    plan.chunk_hist[c * kExperts + expert] = running;
    running += v;
  }
  publish_groups(running, routes, plan, scan_scratch);
}

__global__ void __launch_bounds__(kSortChunk)
route_scatter_kernel(const int* __restrict__ expert_ids, int routes, RoutePlan plan) {
  grid_launch_dependents();
  __shared__ int warp_counts[32 * kExperts];
  const int tid = threadIdx.x;
  for (int i = tid; i < 32 * kExperts; i += kSortChunk) warp_counts[i] = 0;
  __syncthreads();
  const int route = blockIdx.x * kSortChunk + tid;
  int expert = kExperts;
  if (route < routes) {
    expert = expert_ids[route];
    if (expert < 0 || expert >= kExperts) expert = kExperts;
    else if (plan.remap) expert = plan.remap[expert];
  }
  const uint32_t peers = count_chunk(expert, warp_counts);
  __syncthreads();
  if (tid < kExperts) {
    int running = plan.expert_offsets[tid] + plan.chunk_hist[blockIdx.x * kExperts + tid];
    for (int w = 0; w < 32; ++w) {
      const int c = warp_counts[w * kExperts + tid];
      warp_counts[w * kExperts + tid] = running;
      running += c;
    }
  }
  __syncthreads();
  if (expert < kExperts) {
    const int lane = tid & 31, warp = tid >> 5;
    const int dst = warp_counts[warp * kExperts + expert] + __popc(peers & ((1u << lane) - 1u));
    plan.sorted_experts[dst] = expert;
    plan.sorted_routes[dst] = route;
    plan.inverse_routes[route] = dst;
  }
}

// Barrier over the CTAs of one cooperative launch.  sync[0] counts arrivals, sync[1]
// departures; the last CTA to leave zeroes both for the next launch.  The wait is bounded:
// on expiry the status word gets kWaitTimeout and every thread of the CTA sees false.
__device__ __forceinline__ bool grid_barrier(int* sync, int ctas, int* status) {
  __shared__ int passed;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&sync[0], 1);
    const long long start = clock64();
    int ok = 1;
    while (*reinterpret_cast<volatile int*>(&sync[0]) < ctas) {
      if (clock64() - start > 4000000000ll) {
        atomicExch(status, static_cast<int>(kWaitTimeout));
        ok = 0;
        break;
      }
    }
    __threadfence();
    if (atomicAdd(&sync[1], 1) == ctas - 1) {
      sync[0] = 0;
      sync[1] = 0;
    }
    passed = ok;
  }
  __syncthreads();
  return passed != 0;
}

// The three phases above in one cooperative launch (chunks <= number of SMs): every CTA
// counts its chunk, all meet at a grid barrier, every CTA scans the chunk histograms for
// its own base (the group geometry is written by all of them with identical values) and
// scatters its routes.
__global__ void __launch_bounds__(kSortChunk)
route_sort_fused_kernel(const int* __restrict__ expert_ids, int routes, int chunks, RoutePlan plan) {
  grid_launch_dependents();
  __shared__ int warp_counts[32 * kExperts];
  __shared__ int scan_scratch[16];
  const int tid = threadIdx.x;
  for (int i = tid; i < 32 * kExperts; i += kSortChunk) warp_counts[i] = 0;
  __syncthreads();
  grid_dependency_wait();  // the ids are written, and the plan's last readers are done
  const int route = blockIdx.x * kSortChunk + tid;
  int expert = kExperts;
  if (route < routes) {
    expert = expert_ids[route];
    if (expert < 0 || expert >= kExperts) {
      atomicExch(plan.status, static_cast<int>(kBadExpertId));
      expert = kExperts;
    } else if (plan.remap) {
      expert = plan.remap[expert];
    }
  }
  const uint32_t peers = count_chunk(expert, warp_counts);
  __syncthreads();
  if (tid < kExperts) {
    int total = 0;
    for (int w = 0; w < 32; ++w) total += warp_counts[w * kExperts + tid];
    plan.chunk_hist[blockIdx.x * kExperts + tid] = total;
  }
  if (!grid_barrier(plan.sync, chunks, plan.status)) return;
  // All chunk histograms, 32 chunks at a time: the whole CTA fetches them in one round of loads
  // (128 threads walking them chunk by chunk is a chain of trips to L2), then expert `tid` adds
  // its column from shared memory.
  __shared__ int fetched[32 * kExperts];
  int before = 0, total = 0;
  for (int first = 0; first < chunks; first += 32) {
    const int count = chunks - first < 32 ? chunks - first : 32;
    for (int i = tid; i < count * kExperts; i += kSortChunk) fetched[i] = __ldcg(&plan.chunk_hist[first * kExperts + i]);
    __syncthreads();
    if (tid < kExperts) {
      for (int c = 0; c < count; ++c) {
        const int v = fetched[c * kExperts + tid];
        if (first + c < static_cast<int>(blockIdx.x)) before += v;
        total += v;
      }
    }
    __syncthreads();
  }
  if (tid < kExperts) {
    int running = publish_groups(total, routes, plan, scan_scratch) + before;
    for (int w = 0; w < 32; ++w) {
      const int c = warp_counts[w * kExperts + tid];
      warp_counts[w * kExperts + tid] = running;
      running += c;
    }
  }
  __syncthreads();
  if (expert < kExperts) {
    const int lane = tid & 31, warp = tid >> 5;
    const int dst = warp_counts[warp * kExperts + expert] + __popc(peers & ((1u << lane) - 1u));
    plan.sorted_experts[dst] = expert;
    plan.sorted_routes[dst] = route;
    plan.inverse_routes[route] = dst;
  }
}

namespace {
// SM count of the current device, cached per device ordinal.
int current_sm_count() {
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess) cached[device] = count;
  }
  return cached[device];
}
}  // namespace

void launch_route_sort(const int* expert_ids, int routes, const RoutePlan& plan,
                       cudaStream_t stream) {
  if (routes <= kSortChunk) {
    route_sort_single_kernel<<<1, kSortChunk, 0, stream>>>(expert_ids, routes, plan);
    return;
  }
  int chunks = (routes + kSortChunk - 1) / kSortChunk;
  // While a stream is being captured into a graph the three plain launches are used: they
  // need no co-residency guarantee and are certain to be capturable.
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) capture = cudaStreamCaptureStatusActive;
  if (plan.sync != nullptr && chunks <= current_sm_count() && capture == cudaStreamCaptureStatusNone) {
    // A cooperative launch (its CTAs meet at a grid barrier) that may also begin while the previous
    // kernel of the stream is still running: the kernel clears its shared memory, then waits for
    // that kernel at grid_dependency_wait before it reads the ids or writes the plan.
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(chunks);
    config.blockDim = dim3(kSortChunk);
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    const cudaError_t e = cudaLaunchKernelEx(&config, route_sort_fused_kernel, expert_ids, routes, chunks, plan);
    if (e == cudaSuccess) return;
    (void)cudaGetLastError();  // not launchable as one grid here: fall through to the three launches
  }
  route_histogram_kernel<<<chunks, kSortChunk, 0, stream>>>(expert_ids, routes, plan);
  route_prefix_kernel<<<1, kExperts, 0, stream>>>(chunks, routes, plan);
  route_scatter_kernel<<<chunks, kSortChunk, 0, stream>>>(expert_ids, routes, plan);
}

// ---------------------------------------------------------------------------
// Input quantiser.  Reference: quantize_bf16_sorted_moe, src/nvfp4_cutlass.cu:
// 290-327 (one CTA per sorted route, 16 scalar loads per thread, byte stores, the
// token row fetched eight times).  Here a token row is read once; a thread owns 32
// consecutive columns (two 16-value blocks) and, for each of the token's eight routes,
// quantises them with that expert's static scale, storing 16 code bytes and the two scale
// bytes (adjacent in the swizzled layout) of the route's sorted row.  Nothing is computed
// twice: no lane shares a block with another, and routes with equal static scales share one
// quantisation.  At 4096 tokens the kernel moves 75 MB, 52 MB of them written, in 21 us; a
// form with 64 columns per thread (whole 4-byte scale words, half as many threads) took 30 us.
// ---------------------------------------------------------------------------
template <int kTokensPerBlock, int kBlocks>
__global__ void __launch_bounds__(kHidden / (16 * kBlocks) * kTokensPerBlock)
quantize_input_kernel(const __nv_bfloat16* __restrict__ input, const int* __restrict__ expert_ids,
                      const float* __restrict__ in_scale_q, RoutePlan plan, int tokens,
                      uint8_t* __restrict__ packed, uint8_t* __restrict__ scales) {
  constexpr int groups = kHidden / 16;
  __shared__ float route_multiplier[kTokensPerBlock][kTopK];
  __shared__ int route_row[kTokensPerBlock][kTopK];  // sorted row, or -1 for a rejected expert id
  __shared__ unsigned long long route_scale_base[kTokensPerBlock][kTopK];
  grid_launch_dependents();
  grid_dependency_wait();  // the route sort's plan, and the previous user of the output buffers
  if (threadIdx.x < kTokensPerBlock * kTopK) {
    const int slot = threadIdx.x / kTopK;
    const int k = threadIdx.x % kTopK;
    const int token = blockIdx.x * kTokensPerBlock + slot;
    int dst = -1;
    if (token < tokens) {
      const int route = token * kTopK + k;
      const int expert = expert_ids[route];
      if (expert >= 0 && expert < kExperts) {  // others are flagged by the route sort
        dst = plan.inverse_routes[route];
        const int row = dst - plan.expert_offsets[expert];
        route_multiplier[slot][k] = in_scale_q[expert];
        route_scale_base[slot][k] =
            static_cast<unsigned long long>(plan.scale_row_offsets[expert]) * groups + sf_offset(row, 0, groups);
      }
    }
    route_row[slot][k] = dst;
  }
  constexpr int threads_per_token = kHidden / (16 * kBlocks);
  const int slot = threadIdx.x / threads_per_token;
  const int part = threadIdx.x - slot * threads_per_token;  // columns [16*kBlocks*part, +16*kBlocks)
  const int token = blockIdx.x * kTokensPerBlock + slot;
  float values[16 * kBlocks];
  float maximum[kBlocks];
  if (token < tokens) load_token_columns<kBlocks>(input, token, part, values, maximum);
  __syncthreads();
  if (token >= tokens) return;
  quantize_routes_of_token<kBlocks>(values, maximum, part, route_row[slot], route_multiplier[slot],
                                    route_scale_base[slot], packed, scales);
}

// Route sort and input quantiser in one launch, for batches of at most 1024 routes (decode
// sizes, where the layer is a chain of short kernels and every launch costs as much as the
// work).  One CTA per token: it counts all routes per expert in shared memory, ranks its own
// eight routes among those with the same expert and a lower route index (the stable counting
// sort of route_sort_single_kernel, computed redundantly per token), scans the 128 counts,
// and quantises its token.  CTA 0 also writes the group geometry.
__global__ void __launch_bounds__(kQuantizeThreadsPerToken)
route_sort_quantize_small_kernel(const __nv_bfloat16* __restrict__ input, const int* __restrict__ expert_ids,
                                 const float* __restrict__ in_scale_q, RoutePlan plan, int tokens,
                                 uint8_t* __restrict__ packed, uint8_t* __restrict__ scales) {
  constexpr int groups = kHidden / 16;
  __shared__ int histogram[kExperts];
  __shared__ int row_begin[kExperts];
  __shared__ int scale_row_begin[kExperts];
  __shared__ int own_expert[kTopK];
  __shared__ int own_rank[kTopK];
  __shared__ float route_multiplier[kTopK];
  __shared__ int route_row[kTopK];
  __shared__ unsigned long long route_scale_base[kTopK];
  grid_launch_dependents();
  grid_dependency_wait();
  const int tid = threadIdx.x;
  const int token = blockIdx.x;
  const int routes = tokens * kTopK;
  for (int i = tid; i < kExperts; i += kQuantizeThreadsPerToken) histogram[i] = 0;
  if (tid < kTopK) {
    int expert = expert_ids[token * kTopK + tid];
    if (expert < 0 || expert >= kExperts) expert = kExperts;
    else if (plan.remap) expert = plan.remap[expert];
    own_expert[tid] = expert;
    own_rank[tid] = 0;
  }
  __syncthreads();
  for (int route = tid; route < routes; route += kQuantizeThreadsPerToken) {
    int expert = expert_ids[route];
    if (expert < 0 || expert >= kExperts) {
      if (token == 0) atomicExch(plan.status, static_cast<int>(kBadExpertId));
      continue;
    }
    if (plan.remap) expert = plan.remap[expert];
    atomicAdd(&histogram[expert], 1);
#pragma unroll
    for (int k = 0; k < kTopK; ++k)
      if (expert == own_expert[k] && route < token * kTopK + k) atomicAdd(&own_rank[k], 1);
  }
  __syncthreads();
  if (tid < 32) {
    // lane l scans experts 4l..4l+3: rows and 128-row tiles
    int counts[4], rows = 0, tiles = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      counts[i] = histogram[4 * tid + i];
      rows += counts[i];
      tiles += (counts[i] + kTileM - 1) / kTileM;
    }
    int rows_inclusive = rows, tiles_inclusive = tiles;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, rows_inclusive, offset);
      const int t = __shfl_up_sync(0xffffffffu, tiles_inclusive, offset);
      if (tid >= offset) {
        rows_inclusive += r;
        tiles_inclusive += t;
      }
    }
    int row = rows_inclusive - rows, tile = tiles_inclusive - tiles;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int expert = 4 * tid + i;
      row_begin[expert] = row;
      scale_row_begin[expert] = tile * kTileM;
      if (token == 0) {
        plan.expert_offsets[expert] = row;
        plan.scale_row_offsets[expert] = tile * kTileM;
        const int expert_tiles = (counts[i] + kTileM - 1) / kTileM;
        for (int j = 0; j < expert_tiles; ++j) {
          plan.tile_expert[tile + j] = expert;
          if (plan.tile_ready) plan.tile_ready[tile + j] = 0;
        }
      }
      row += counts[i];
      tile += (counts[i] + kTileM - 1) / kTileM;
    }
    if (token == 0 && tid == 31) {
      plan.expert_offsets[kExperts] = row;
      plan.scale_row_offsets[kExperts] = tile * kTileM;
      plan.num_m_tiles[0] = tile;
    }
  }
  __syncthreads();
  if (tid < kTopK) {
    const int route = token * kTopK + tid;
    const int expert = own_expert[tid];
    int dst = -1;
    if (expert < kExperts) {
      dst = row_begin[expert] + own_rank[tid];
      plan.sorted_experts[dst] = expert;
      plan.sorted_routes[dst] = route;
      plan.inverse_routes[route] = dst;
      // the static scale belongs to the expert id as the caller numbers it
      route_multiplier[tid] = in_scale_q[expert_ids[route]];
      route_scale_base[tid] = static_cast<unsigned long long>(scale_row_begin[expert]) * groups +
                              sf_offset(own_rank[tid], 0, groups);
    }
    route_row[tid] = dst;
  }
  float values[32];
  float maximum[2];
  load_token_columns<2>(input, token, tid, values, maximum);
  __syncthreads();
  quantize_routes_of_token<2>(values, maximum, tid, route_row, route_multiplier, route_scale_base, packed, scales);
}

void launch_route_sort_quantize_small(const void* input_bf16, const int* expert_ids, const float* in_scale_q,
                                      const RoutePlan& plan, int tokens, uint8_t* packed, uint8_t* scales,
                                      cudaStream_t stream) {
  launch_chained(route_sort_quantize_small_kernel, dim3(tokens), dim3(kQuantizeThreadsPerToken), 0, stream,
                 static_cast<const __nv_bfloat16*>(input_bf16), expert_ids, in_scale_q, plan, tokens, packed,
                 scales);
}

void launch_quantize_input(const void* input_bf16, const int* expert_ids, const float* in_scale_q,
                           const RoutePlan& plan, int tokens, uint8_t* packed, uint8_t* scales,
                           cudaStream_t stream) {
  const __nv_bfloat16* input = static_cast<const __nv_bfloat16*>(input_bf16);
  // One token per CTA at every size: small CTAs keep more of them resident, which is what hides the
  // latency of this short kernel (4096 tokens: 3 us less per layer than four tokens per CTA).
  launch_chained(quantize_input_kernel<1, 2>, dim3(tokens), dim3(kQuantizeThreadsPerToken), 0, stream, input,
                 expert_ids, in_scale_q, plan, tokens, packed, scales);
}

// ---------------------------------------------------------------------------
// GeGLU + requantise of the w13 output.  Reference: geglu_quantize_sorted_moe,
// src/nvfp4_cutlass.cu:552-601: v = gelu_erf(gate) * up from the bf16 GEMM output,
// columns [0,704) = up and [704,1408) = gate.
// ---------------------------------------------------------------------------
constexpr int kQuadsInter = kInter / 64;    // 11
constexpr int kGegluRowsPerBlock = 32;

__global__ void __launch_bounds__(kGegluRowsPerBlock * kQuadsInter)
geglu_quantize_kernel(const __nv_bfloat16* __restrict__ fused, const float* __restrict__ in_scale_q,
                      RoutePlan plan, int routes, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ scales) {
  __shared__ __align__(16) float erf_table[GV_ERF_TABLE_FLOATS];
  load_erf_table(erf_table);
  __syncthreads();
  const int route = blockIdx.x * kGegluRowsPerBlock + threadIdx.x / kQuadsInter;
  const int quad = threadIdx.x % kQuadsInter;
  if (route >= routes) return;
  const int expert = plan.sorted_experts[route];
  const int row = route - plan.expert_offsets[expert];
  const float multiplier = in_scale_q[expert];
  const uint4* up = reinterpret_cast<const uint4*>(fused + static_cast<size_t>(route) * kW13Out + quad * 64);
  const uint4* gate = reinterpret_cast<const uint4*>(fused + static_cast<size_t>(route) * kW13Out + kInter + quad * 64);
  uint32_t codes[8];
  uint32_t scale_word = 0;
#pragma unroll
  for (int block = 0; block < 4; ++block) {
    float u[16], g[16], values[16];
    unpack_bf16x8(__ldg(up + 2 * block), u);
    unpack_bf16x8(__ldg(up + 2 * block + 1), u + 8);
    unpack_bf16x8(__ldg(gate + 2 * block), g);
    unpack_bf16x8(__ldg(gate + 2 * block + 1), g + 8);
#pragma unroll
    for (int i = 0; i < 16; ++i) values[i] = __fmul_rn(gv_gelu_erf(g[i], erf_table), u[i]);
    scale_word |= quantize_block16(values, multiplier, codes[2 * block], codes[2 * block + 1])
                  << (8 * block);
  }
  uint4* out = reinterpret_cast<uint4*>(packed + static_cast<size_t>(route) * (kInter / 2) + quad * 32);
  out[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
  out[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
  constexpr int groups = kInter / 16;
  *reinterpret_cast<uint32_t*>(scales + static_cast<size_t>(plan.scale_row_offsets[expert]) * groups +
                               sf_offset(row, 4 * quad, groups)) = scale_word;
}

void launch_geglu_quantize(const void* fused_bf16, const float* in_scale_q, const RoutePlan& plan,
                           int routes, uint8_t* packed, uint8_t* scales, cudaStream_t stream) {
  geglu_quantize_kernel<<<(routes + kGegluRowsPerBlock - 1) / kGegluRowsPerBlock,
                          kGegluRowsPerBlock * kQuadsInter, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(fused_bf16), in_scale_q, plan, routes, packed, scales);
}

// ---------------------------------------------------------------------------
// Weighted un-permute/reduce.  Reference: reduce_expert_routes,
// src/nvfp4_cutlass.cu:229-247: fp32 fmaf over the eight routes in route order,
// one bf16 rounding.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kHidden / 8)
reduce_routes_kernel(const __nv_bfloat16* __restrict__ routed, const float* __restrict__ route_weights,
                     const int* __restrict__ inverse_routes, __nv_bfloat16* __restrict__ output) {
  const int token = blockIdx.x;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  unsigned long long read_once;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(read_once));
  grid_launch_dependents();
  grid_dependency_wait();  // the down GEMM's rows
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    const int index = token * kTopK + k;
    const int source = inverse_routes[index];
    const float weight = route_weights[index];
    float v[8];
    // read once and dead afterwards: the rows must not push the rows that other CTAs have not yet read out of L2
    uint4 raw;
    asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                 : "l"(reinterpret_cast<const uint4*>(routed + static_cast<size_t>(source) * kHidden) + threadIdx.x),
                   "l"(read_once));
    unpack_bf16x8(raw, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fmaf_rn(v[i], weight, acc[i]);
  }
  uint32_t packed[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
  }
  reinterpret_cast<uint4*>(output + static_cast<size_t>(token) * kHidden)[threadIdx.x] =
      make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

void launch_reduce_routes(const void* routed_bf16, const float* route_weights,
                          const int* inverse_routes, int tokens, void* output_bf16,
                          cudaStream_t stream) {
  launch_chained(reduce_routes_kernel, dim3(tokens), dim3(kHidden / 8), 0, stream,
                 static_cast<const __nv_bfloat16*>(routed_bf16), route_weights, inverse_routes,
                 static_cast<__nv_bfloat16*>(output_bf16));
}

// ---------------------------------------------------------------------------
// Synthetic expert packer: fp32 weights -> the sidecar's NVFP4 layout
// (tensor shapes: src/runtime.cpp:233-252; scale interleave per expert:
// tools/pack_trtllm_experts.py:59-64).  global = amax/(6*448) per expert matrix.
// ---------------------------------------------------------------------------
__global__ void expert_amax_kernel(const float* __restrict__ weights, size_t per_expert,
                                   unsigned int* __restrict__ amax_bits) {
  const int expert = blockIdx.y;
  const float* w = weights + static_cast<size_t>(expert) * per_expert;
  float maximum = 0.0f;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < per_expert;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    maximum = fmaxf(maximum, fabsf(w[i]));
  for (int offset = 16; offset; offset >>= 1)
    maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + expert, __float_as_uint(maximum));
}

__global__ void pack_weights_kernel(const float* __restrict__ weights, int n_out, int k_in,
                                    const unsigned int* __restrict__ amax_bits,
                                    uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                    float* __restrict__ global_scales) {
  const int expert = blockIdx.y;
  const int groups = k_in / 16;
  const int block_index = blockIdx.x * blockDim.x + threadIdx.x;
  const float global = __fdiv_rn(__uint_as_float(amax_bits[expert]), __fmul_rn(6.0f, 448.0f));
  if (block_index == 0) global_scales[expert] = global;
  if (block_index >= n_out * groups) return;
  const int n = block_index / groups, g = block_index % groups;
  const float multiplier = global == 0.0f ? 0.0f : __fdiv_rn(1.0f, global);
  const float4* src = reinterpret_cast<const float4*>(
      weights + (static_cast<size_t>(expert) * n_out + n) * k_in + g * 16);
  float values[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = __ldg(src + i);
    values[4 * i] = v.x;
    values[4 * i + 1] = v.y;
    values[4 * i + 2] = v.z;
    values[4 * i + 3] = v.w;
  }
  uint32_t lo, hi;
  const uint32_t scale = quantize_block16(values, multiplier, lo, hi);
  *reinterpret_cast<uint2*>(codes + (static_cast<size_t>(expert) * n_out + n) * (k_in / 2) + g * 8) =
      make_uint2(lo, hi);
  scales[static_cast<size_t>(expert) * n_out * groups + sf_offset(n, g, groups)] =
      static_cast<uint8_t>(scale);
}

void launch_pack_weights(const float* weights, int experts, int n_out, int k_in, uint8_t* codes,
                         uint8_t* scales, float* global_scales, cudaStream_t stream) {
  // Not on the hot path: a stream-ordered temporary holds the per-expert amax bit patterns
  // (the bits of a non-negative float order like an unsigned integer).
  unsigned int* accumulator = nullptr;
  cudaMallocAsync(reinterpret_cast<void**>(&accumulator), sizeof(unsigned int) * experts, stream);
  cudaMemsetAsync(accumulator, 0, sizeof(unsigned int) * experts, stream);
  const size_t per_expert = static_cast<size_t>(n_out) * k_in;
  expert_amax_kernel<<<dim3(64, experts), 256, 0, stream>>>(weights, per_expert, accumulator);
  const int blocks = n_out * (k_in / 16);
  pack_weights_kernel<<<dim3((blocks + 255) / 256, experts), 256, 0, stream>>>(
      weights, n_out, k_in, accumulator, codes, scales, global_scales);
  cudaFreeAsync(accumulator, stream);
}

}  // namespace gv
