// Expert-parallel form of the MoE layer: experts sharded over the GPUs of one
// node, tokens data-parallel, rows exchanged by stores into peer memory over NVLink.
// The reference is single-GPU and has no counterpart.
//
// Placement.  By default expert e lives on rank e % world as local expert e / world; a
// caller's table may place experts otherwise (e.g. by observed load).  Either way the
// "virtual" id v = owner * EL + local index (EL = 128 / world) orders experts by owning
// rank, so a sender's sorted routes are contiguous per destination.
//
// One step, on every rank (the caller places a cross-rank barrier where marked):
//   1. route_sort   sort local routes by v; store this rank's 128 counts into
//                   every peer's count matrix                       -- barrier --
//   2. dispatch     from the full count matrix compute, for every v, where this
//                   rank's rows land in the owner's receive buffer; quantise each
//                   route with its expert's static scale and store codes and scale
//                   rows straight into the owner's receive buffers
//                   (1584 B per route instead of 5632 B of bf16); then, from the same
//                   matrix, the group geometry of the local experts and the address
//                   of every result row                              -- barrier --
//   3. compute      received scale rows into the MMA layout; w13 (+GeGLU+requantise)
//                   and w2 grouped GEMMs; the w2
//                   epilogue stores every result row straight into its source
//                   rank's combine buffer at the source's own sorted position
//                                                                    -- barrier --
//   4. reduce       the source's usual weighted reduce over its eight routes.
// Receive order is fixed by (local expert, source rank, source order), so results do
// not depend on timing.  All peer traffic is plain global stores through mapped
// peer pointers; nothing here waits on a peer inside a kernel (the barriers are the
// caller's collectives), and no TMA load touches peer memory: the GEMMs read only
// this GPU's own receive buffers.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <new>

#include "../../include/gevva_moe.h"
#include "gv_common.cuh"
#include "gv_ep_protocol.h"
#include "gv_launchers.h"
#include "gv_plan.cuh"

namespace gv {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxComputeChunks = 4;  // parts the compute phase may be cut into (see gevva_moe_ep_compute)

struct EpDevice {            // device-visible description, passed to kernels by value
  int rank, world, local_experts;
  uint8_t* peer_codes[kMaxWorld];   // each rank's w13 operand codes [capacity, 1408]
  uint8_t* peer_scales[kMaxWorld];  // each rank's scale staging, row-major [capacity, 176]
  __nv_bfloat16* peer_combine[kMaxWorld];  // each rank's combine buffer [8*T_local, 2816]
  int* peer_counts[kMaxWorld];      // each rank's count matrix [world][128]
  int* peer_flags[kMaxWorld];       // each rank's barrier flags [world]
  int* counts;                      // == peer_counts[rank]
  int* send_row_base;               // [128] by v
  int* send_src_prefix;             // [128] by v
  int* send_scale_rows;             // [128] by v
  int* source_offsets;              // [world][EL]: sorted position of (source, local expert) on the source
  const int* remap;                 // [128] e -> v
};

// ---- barrier across ranks -----------------------------------------------------------
// Rank r stores `epoch` into flag r of every peer, then waits until all of its own flags
// have reached `epoch`.  The stores of earlier kernels of this stream are complete when this
// kernel starts; the fence orders the flag behind them at system scope.  The wait is bounded:
// on expiry the status word gets kWaitTimeout and the kernel returns.
// Device side of gv_ep_protocol.h: flags in peer-mapped global memory, system-scope release /
// acquire, the SM cycle counter as the clock (about two seconds).
struct DeviceFlagPort {
  const EpDevice& ep;
  long long start;
  __device__ void publish(int peer, int slot, int value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ep.peer_flags[peer] + slot), "r"(value) : "memory");
  }
  __device__ int observe(int slot) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(ep.peer_flags[ep.rank] + slot) : "memory");
    return seen;
  }
  __device__ void start_clock() { start = clock64(); }
  __device__ bool expired() { return clock64() - start > 4000000000ll; }
  __device__ void pause() { __nanosleep(64); }
};

__global__ void __launch_bounds__(32) ep_barrier_kernel(EpDevice ep, int epoch, int* status) {
  grid_launch_dependents();
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible
  const int lane = threadIdx.x;
  if (lane < ep.world) {
    DeviceFlagPort port{ep, 0};
    ep_barrier_announce(port, ep.rank, lane, epoch);
    if (!ep_barrier_await(port, lane, epoch)) atomicExch(status, static_cast<int>(kWaitTimeout));
  }
}

// ---- 1: the count exchange and everything that depends on the counts only ------------
// One CTA of 128 threads, launched behind the route sort:
//   - thread v stores this rank's count of sort key v into every peer's count matrix;
//   - a flag barrier (the protocol of ep_barrier_kernel, same flags and epoch sequence): when it
//     ends every rank's counts of this step are in this rank's matrix, and every rank has
//     finished reading its receive buffers of the step before;
//   - the matrix is read once, coalesced, into shared memory (the prefix loops below would
//     otherwise be chains of dependent trips to L2);
//   - send side: where this rank's rows land on their owners;
//   - receive side: the group geometry of the local experts, the sorted position on each source
//     of the first row it sends to each local expert, and the parts of the compute phase.
// These were four launches (publish, barrier, send bases, receive plan: 19 us of kernels at one
// rank, plus their gaps); as one kernel 14 us in the same serialised, cold-cache view, and the
// step is 22 us shorter at two ranks.
__global__ void __launch_bounds__(kExperts)
ep_exchange_kernel(EpDevice ep, RoutePlan send_plan, RoutePlan plan, int* split, int chunks, int first_share,
                   int epoch, int* status) {
  __shared__ int counts[kMaxWorld][kExperts];
  __shared__ int prefix[kMaxWorld + 2][kExperts];   // exclusive sums over the sort keys
  __shared__ int warp_sums[4][kMaxWorld + 2];
  __shared__ int scan_scratch[16];
  __shared__ int first_tile[kExperts + 1];
  __shared__ int cuts[kMaxComputeChunks];
  grid_launch_dependents();
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible
  const int v = threadIdx.x;
  const int le = threadIdx.x;
  const int el = ep.local_experts;
  {
    const int count = send_plan.expert_offsets[v + 1] - send_plan.expert_offsets[v];
    for (int d = 0; d < ep.world; ++d) ep.peer_counts[d][ep.rank * kExperts + v] = count;
  }
  __threadfence_system();
  __syncthreads();
  if (v < ep.world) {
    DeviceFlagPort port{ep, 0};
    ep_barrier_announce(port, ep.rank, v, epoch);
    if (!ep_barrier_await(port, v, epoch)) atomicExch(status, static_cast<int>(kWaitTimeout));
  }
  __syncthreads();
  int total = 0;
  int values[kMaxWorld + 2];
#pragma unroll
  for (int s = 0; s < kMaxWorld; ++s) {
    const int c = s < ep.world ? ep.counts[s * kExperts + v] : 0;
    counts[s][v] = c;
    values[s] = c;
    total += c;
  }
  values[kMaxWorld] = total;
  values[kMaxWorld + 1] = (total + kTileM - 1) / kTileM * kTileM;
  // Exclusive prefix sums over the 128 sort keys of all ten series at once (each source's counts,
  // the totals, the totals padded to whole tiles): warp scans, then the warps' sums.
  {
    const int lane = v & 31, warp = v >> 5;
    int inclusive[kMaxWorld + 2];
#pragma unroll
    for (int i = 0; i < kMaxWorld + 2; ++i) {
      int x = values[i];
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, offset);
        if (lane >= offset) x += y;
      }
      inclusive[i] = x;
      if (lane == 31) warp_sums[warp][i] = x;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kMaxWorld + 2; ++i) {
      int base = 0;
      for (int w = 0; w < warp; ++w) base += warp_sums[w][i];
      prefix[i][v] = base + inclusive[i] - values[i];
    }
  }
  __syncthreads();
  // send side: rows of the owner's earlier experts, then rows of earlier sources for this expert
  {
    const int owner_first = (v / el) * el;
    int src_prefix = 0;
    for (int s = 0; s < ep.rank; ++s) src_prefix += counts[s][v];
    ep.send_row_base[v] = prefix[kMaxWorld][v] - prefix[kMaxWorld][owner_first] + src_prefix;
    ep.send_src_prefix[v] = src_prefix;
    ep.send_scale_rows[v] = prefix[kMaxWorld + 1][v] - prefix[kMaxWorld + 1][owner_first];
  }
  // receive side
  int local_count = 0;
  if (le < el)
    for (int s = 0; s < ep.world; ++s) local_count += counts[s][ep.rank * el + le];
  publish_groups(local_count, 0, plan, scan_scratch);
  // sorted position, on source rank s, of the first row it sent to local expert le
  for (int index = threadIdx.x; index < ep.world * el; index += kExperts) {
    const int s = index / el, e = index % el;
    ep.source_offsets[index] = prefix[s][ep.rank * el + e];
  }
  // `chunks` parts of the tile list, cut at expert boundaries near equal shares: part p ends at
  // the first expert (after the first) whose first tile t satisfies chunks * t >= (p + 1) * tiles,
  // or at the end.  First tiles are non-decreasing, so the expert that is the cut of a part knows
  // it from its own value and its predecessor's.
  __syncthreads();
  first_tile[le] = plan.scale_row_offsets[le] / kTileM;
  if (le == 0) first_tile[kExperts] = plan.scale_row_offsets[kExperts] / kTileM;
  if (le < kMaxComputeChunks) cuts[le] = -1;
  __syncthreads();
  const int all_tiles = first_tile[kExperts];
  if (le >= 1 && le < el) {
    for (int part = 0; part + 1 < chunks; ++part) {
      // with two parts the first takes `first_share` percent of the tiles (see gevva_moe_ep_create)
      const int numerator = chunks == 2 ? first_share : 100 * (part + 1);
      const int denominator = chunks == 2 ? 100 : 100 * chunks;
      const bool here = denominator * first_tile[le] >= numerator * all_tiles;
      const bool before = le >= 2 && denominator * first_tile[le - 1] >= numerator * all_tiles;
      if (here && !before) cuts[part] = first_tile[le];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int first = 0;
    for (int part = 0; part < chunks; ++part) {
      const int cut = part + 1 < chunks && cuts[part] >= 0 ? cuts[part] : all_tiles;
      split[2 * part] = first;
      split[2 * part + 1] = cut - first;
      first = cut;
    }
  }
}

// ---- 2b: quantise and store into the owners' operand buffers -----------------------
// Same arithmetic and thread mapping as quantize_input_kernel (a token row is read once, a
// thread owns 32 consecutive columns = two 16-value blocks, four tokens per CTA); only the
// destination differs.
constexpr int kDispatchThreadsPerToken = kHidden / 32;  // 88
constexpr int kDispatchTokensPerBlock = 4;
constexpr int kDispatchThreads = kDispatchThreadsPerToken * kDispatchTokensPerBlock;

__global__ void __launch_bounds__(kDispatchThreads)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ input, const int* __restrict__ expert_ids,
                   const float* __restrict__ in_scale_q_global, EpDevice ep, RoutePlan plan, int tokens) {
  constexpr int groups = kHidden / 16;
  __shared__ float route_multiplier[kDispatchTokensPerBlock][kTopK];
  __shared__ uint8_t* route_codes[kDispatchTokensPerBlock][kTopK];
  __shared__ uint8_t* route_scales[kDispatchTokensPerBlock][kTopK];
  // one 176-byte scale row per route
  __shared__ __align__(16) uint16_t scale_rows[kDispatchTokensPerBlock][kTopK][groups / 2];
  grid_launch_dependents();
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible
  if (threadIdx.x < kDispatchTokensPerBlock * kTopK) {
    const int slot = threadIdx.x / kTopK;
    const int k = threadIdx.x % kTopK;
    const int token = blockIdx.x * kDispatchTokensPerBlock + slot;
    uint8_t* codes_row = nullptr;
    if (token < tokens) {
      const int route = token * kTopK + k;
      const int expert = expert_ids[route];
      if (expert >= 0 && expert < kExperts) {
        const int v = ep.remap[expert];
        const int owner = v / ep.local_experts;
        const int j = plan.inverse_routes[route] - plan.expert_offsets[v];
        const int row = ep.send_row_base[v] + j;
        route_multiplier[slot][k] = in_scale_q_global[expert];
        codes_row = ep.peer_codes[owner] + static_cast<size_t>(row) * (kHidden / 2);
        route_scales[slot][k] = ep.peer_scales[owner] + static_cast<size_t>(row) * groups;
      }
    }
    route_codes[slot][k] = codes_row;
  }
  const int slot = threadIdx.x / kDispatchThreadsPerToken;
  const int part = threadIdx.x - slot * kDispatchThreadsPerToken;  // columns [32*part, 32*part+32)
  const int token = blockIdx.x * kDispatchTokensPerBlock + slot;
  float values[32];
  float maximum[2] = {0.0f, 0.0f};
  if (token < tokens) {
    const uint4* source = reinterpret_cast<const uint4*>(input + static_cast<size_t>(token) * kHidden) + 4 * part;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 raw = __ldg(source + i);
      values[8 * i + 0] = __uint_as_float(raw.x << 16);
      values[8 * i + 1] = __uint_as_float(raw.x & 0xffff0000u);
      values[8 * i + 2] = __uint_as_float(raw.y << 16);
      values[8 * i + 3] = __uint_as_float(raw.y & 0xffff0000u);
      values[8 * i + 4] = __uint_as_float(raw.z << 16);
      values[8 * i + 5] = __uint_as_float(raw.z & 0xffff0000u);
      values[8 * i + 6] = __uint_as_float(raw.w << 16);
      values[8 * i + 7] = __uint_as_float(raw.w & 0xffff0000u);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      maximum[0] = fmaxf(maximum[0], fabsf(values[i]));
      maximum[1] = fmaxf(maximum[1], fabsf(values[16 + i]));
    }
  }
  __syncthreads();
  if (token < tokens) {
#pragma unroll 2
    for (int k = 0; k < kTopK; ++k) {
      uint8_t* codes_row = route_codes[slot][k];
      if (!codes_row) continue;
      const float multiplier = route_multiplier[slot][k];
      uint32_t codes[4];
      uint32_t scale_pair = 0;
#pragma unroll
      for (int block = 0; block < 2; ++block) {
        const float unrounded = __fdiv_rn(__fmul_rn(multiplier, maximum[block]), 6.0f);
        const uint32_t scale = encode_e4m3(unrounded);
        const float rounded = decode_e4m3(scale);
        const float inverse = rounded == 0.0f ? 0.0f : __fdiv_rn(multiplier, rounded);
        scale_pair |= scale << (8 * block);
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
      reinterpret_cast<uint4*>(codes_row)[part] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      scale_rows[slot][k][part] = static_cast<uint16_t>(scale_pair);
    }
  }
  // Scale bytes cross NVLink as one contiguous 176-byte row per route (eleven 16-byte
  // stores); the owner puts them into the MMA's interleaved layout itself.
  __syncthreads();
  for (int index = threadIdx.x; index < kDispatchTokensPerBlock * kTopK * (groups / 16); index += kDispatchThreads) {
    const int piece = index % (groups / 16);
    const int k = (index / (groups / 16)) % kTopK;
    const int s = index / (groups / 16) / kTopK;
    if (route_codes[s][k])
      reinterpret_cast<uint4*>(route_scales[s][k])[piece] = reinterpret_cast<const uint4*>(scale_rows[s][k])[piece];
  }
}

// ---- 3a': received scale rows -> the interleaved layout of the w13 operand -------------
// One CTA per 128-row tile of the receive plan (grid-stride): the tile's rows are contiguous in
// the staging buffer (176 bytes each), so they are read as one run of 4-byte words into shared
// memory, and written as the tile's 44 atoms of 512 bytes, 16 bytes (rows q, q+32, q+64, q+96
// of one 4-group word) per thread.  Rows past the expert's end get scale zero.
__global__ void __launch_bounds__(256)
ep_swizzle_scales_kernel(const uint8_t* staged, EpDevice ep, RoutePlan plan, uint8_t* scales, int await_epoch,
                         int* status) {
  constexpr int groups = kHidden / 16;
  constexpr int words = groups / 4;  // 44 per row
  __shared__ uint32_t tile[kTileM][words + 1];
  grid_launch_dependents();
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible
  if (await_epoch) {
    // The barrier between dispatch and compute: every rank announced, behind its dispatch kernel
    // (ep_row_destinations_kernel), that its rows are in their owners' buffers.  `staged` is written
    // by peers until this wait ends, so it is read with ordinary loads, after the wait.
    if (threadIdx.x < ep.world) {
      DeviceFlagPort port{ep, 0};
      if (!ep_barrier_await(port, threadIdx.x, await_epoch)) atomicExch(status, static_cast<int>(kWaitTimeout));
    }
    __syncthreads();
  }
  const int tiles = plan.num_m_tiles[0];
  for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int expert = plan.tile_expert[t];
    const int row0 = plan.expert_offsets[expert] + (t * kTileM - plan.scale_row_offsets[expert]);
    const int left = plan.expert_offsets[expert + 1] - row0;
    const int valid = left < kTileM ? left : kTileM;
    // all of a thread's loads are issued before the first is used: six 16-byte pieces at most
    const uint4* source = reinterpret_cast<const uint4*>(staged + static_cast<size_t>(row0) * groups);
    constexpr int kPieces = (kTileM * (groups / 16) + 255) / 256;
    uint4 piece[kPieces];
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
      const int i = threadIdx.x + j * 256;
      piece[j] = i < valid * (groups / 16) ? source[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < valid * (groups / 16)) {
        const int row = i / (groups / 16), first = 4 * (i % (groups / 16));
        tile[row][first] = piece[j].x;
        tile[row][first + 1] = piece[j].y;
        tile[row][first + 2] = piece[j].z;
        tile[row][first + 3] = piece[j].w;
      }
    }
    __syncthreads();
    uint4* out = reinterpret_cast<uint4*>(scales + static_cast<size_t>(t) * kTileM * groups);
#pragma unroll 2
    for (int i = threadIdx.x; i < words * 32; i += 256) {
      const int word = i >> 5, q = i & 31;
      uint4 v;
      v.x = q < valid ? tile[q][word] : 0u;
      v.y = q + 32 < valid ? tile[q + 32][word] : 0u;
      v.z = q + 64 < valid ? tile[q + 64][word] : 0u;
      v.w = q + 96 < valid ? tile[q + 96][word] : 0u;
      out[word * 32 + q] = v;
    }
    __syncthreads();
  }
}

// ---- 3b: where every received row's result goes ------------------------------------
// One 64-bit address per receive row: the row of the source rank's combine buffer at the
// source's own sorted position.  The w2 GEMM epilogue stores through these addresses, so
// results cross NVLink while the GEMM is still running and never touch local memory.
__global__ void __launch_bounds__(256)
ep_row_destinations_kernel(EpDevice ep, RoutePlan plan, unsigned long long* __restrict__ row_dest,
                           int announce_epoch) {
  grid_launch_dependents();
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible
  if (announce_epoch && blockIdx.x == 0 && threadIdx.x < ep.world) {
    // This launch follows the dispatch kernel in its stream, so this rank's rows are in their
    // owners' buffers: say so to every rank (first half of the barrier before compute; the
    // scale re-tiling kernel of the compute phase waits for all ranks' announcements).
    DeviceFlagPort port{ep, 0};
    ep_barrier_announce(port, ep.rank, threadIdx.x, announce_epoch);
  }
  // (The small tables a row consults stay in global memory: after the first touch they are L1
  // hits, and staging them in shared memory first made this launch 2 us longer.)
  const int el = ep.local_experts;
  const int total = plan.expert_offsets[kExperts];
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < total; row += gridDim.x * blockDim.x) {
    // local expert of this row: the last le with expert_offsets[le] <= row
    int lo = 0, hi = el - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (plan.expert_offsets[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int le = lo;
    int within = row - plan.expert_offsets[le];
    const int v = ep.rank * el + le;
    int s = 0;
    for (; s < ep.world - 1; ++s) {
      const int c = ep.counts[s * kExperts + v];
      if (within < c) break;
      within -= c;
    }
    const int dst_row = ep.source_offsets[s * el + le] + within;
    row_dest[row] = reinterpret_cast<unsigned long long>(ep.peer_combine[s] +
                                                         static_cast<size_t>(dst_row) * kHidden);
  }
}

// Measurement aid: the same table with every destination inside this rank's own combine buffer
// (rows wrap around its 8 * max_tokens rows), so the compute phase can be timed with no byte
// crossing NVLink.
__global__ void __launch_bounds__(256)
ep_row_destinations_local_kernel(EpDevice ep, RoutePlan plan, unsigned long long* __restrict__ row_dest,
                                 int combine_rows) {
  const int total = plan.expert_offsets[kExperts];
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < total; row += gridDim.x * blockDim.x)
    row_dest[row] = reinterpret_cast<unsigned long long>(ep.peer_combine[ep.rank] +
                                                         static_cast<size_t>(row % combine_rows) * kHidden);
}

}  // namespace

}  // namespace gv

// ------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------
namespace {

using namespace gv;

inline bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, int box_rows) {
  return gv::make_operand_tensor_map(map, base, rows, row_bytes, box_rows);
}

}  // namespace

struct gevva_moe_ep {
  gv::EpDevice dev{};
  gv::RoutePlan send_plan{};     // this rank's own routes, sorted by v
  gv::RoutePlan receive_plan{};  // rows received for the local experts
  gv::GemmOperands w13{}, w2{};
  const float* in_scale_q1_global = nullptr;
  int max_tokens = 0;
  size_t capacity_rows = 0;
  int sm_count = 0;
  int epoch = 0;
  int dispatch_epoch = 0;  // epoch announced by the last gevva_moe_ep_dispatch, awaited by gevva_moe_ep_compute
  // owned device memory
  int* ints = nullptr;
  uint8_t* input_sf = nullptr;
  uint8_t* inter_codes = nullptr;
  uint8_t* inter_sf = nullptr;
  unsigned long long* row_dest = nullptr;
  unsigned long long* row_dest_local = nullptr;  // measurement aid, allocated on first use
  uint8_t* w13_sf_tiled = nullptr;
  // the compute phase runs the local experts in two halves so that the NVLink-bound w2 of the
  // first half overlaps the w13 of the second: a side stream and two events order them
  int* split = nullptr;  // device [2 * chunks]: first tile and tile count of each part
  int chunks = 2;        // parts of the compute phase
  int first_share = 50;  // percent of the row tiles in the first of two parts
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};

extern "C" {

void gevva_moe_ep_destroy(gevva_moe_ep* ep) {
  if (!ep) return;
  cudaFree(ep->ints);
  cudaFree(ep->input_sf);
  cudaFree(ep->inter_codes);
  cudaFree(ep->inter_sf);
  cudaFree(ep->row_dest);
  cudaFree(ep->row_dest_local);
  cudaFree(ep->w13_sf_tiled);
  if (ep->side) cudaStreamDestroy(ep->side);
  if (ep->fork) cudaEventDestroy(ep->fork);
  if (ep->join) cudaEventDestroy(ep->join);
  delete ep;
}

int gevva_moe_ep_create(gevva_moe_ep** out, const gevva_moe_weights* local_weights,
                        const float* in_scale_q1_global, const gevva_moe_ep_config* config) {
  if (!out || !local_weights || !in_scale_q1_global || !config) return GEVVA_MOE_BAD_ARGUMENT;
  const int world = config->world, rank = config->rank;
  if (world < 1 || world > gv::kMaxWorld || kExperts % world != 0 || rank < 0 || rank >= world ||
      config->max_tokens < 1)
    return GEVVA_MOE_BAD_ARGUMENT;
  // Nothing on the device bounds a receive row against the capacity, so the capacity must cover
  // the case in which every route of every rank lands on this one.
  if (config->recv_capacity_rows < static_cast<size_t>(world) * kTopK * static_cast<size_t>(config->max_tokens))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (!config->peer_recv_codes || !config->peer_recv_sf || !config->peer_combine || !config->peer_counts ||
      !config->peer_flags)
    return GEVVA_MOE_BAD_ARGUMENT;
  for (int d = 0; d < world; ++d)
    if (!config->peer_recv_codes[d] || !config->peer_recv_sf[d] || !config->peer_combine[d] ||
        !config->peer_counts[d] || !config->peer_flags[d])
      return GEVVA_MOE_BAD_ARGUMENT;
  if (gv::prepare_grouped_gemm() != 0) return GEVVA_MOE_CUDA_ERROR;
  cudaDeviceProp prop;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess)
    return GEVVA_MOE_CUDA_ERROR;
  if (prop.major != 10) return GEVVA_MOE_NO_DEVICE;
  gevva_moe_ep* ep = new (std::nothrow) gevva_moe_ep;
  if (!ep) return GEVVA_MOE_CUDA_ERROR;
  const int el = kExperts / world;
  ep->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->join, cudaEventDisableTiming) != cudaSuccess) {
    gevva_moe_ep_destroy(ep);
    return GEVVA_MOE_CUDA_ERROR;
  }
  ep->max_tokens = config->max_tokens;
  // two parts measured best at 2, 4 and 8 GPUs (four parts: 268 against 234 us of compute at
  // 2 GPUs, 383 against 332 us at 8)
  ep->chunks = 2;
  // The first part's w13 runs with NVLink idle; afterwards the first part's result rows cross
  // NVLink (W us for all rows) while the second part's w13 has 84 of 148 SMs.  Both end together
  // when the first part is 176 / (W + 176) of the rows: W grows with the share of rows that
  // leave the GPU, about 150, 220 and 260 us at 2, 4 and 8 ranks.
  ep->first_share = world >= 8 ? 40 : world >= 4 ? 44 : world >= 2 ? 54 : 50;
  if (const char* share = getenv("GEVVA_EP_FIRST_SHARE")) ep->first_share = atoi(share);
  ep->capacity_rows = config->recv_capacity_rows;
  ep->in_scale_q1_global = in_scale_q1_global;
  ep->dev.rank = rank;
  ep->dev.world = world;
  ep->dev.local_experts = el;
  for (int d = 0; d < world; ++d) {
    ep->dev.peer_codes[d] = static_cast<uint8_t*>(config->peer_recv_codes[d]);
    ep->dev.peer_scales[d] = static_cast<uint8_t*>(config->peer_recv_sf[d]);
    ep->dev.peer_combine[d] = static_cast<__nv_bfloat16*>(config->peer_combine[d]);
    ep->dev.peer_counts[d] = config->peer_counts[d];
    ep->dev.peer_flags[d] = config->peer_flags[d];
  }
  ep->dev.counts = ep->dev.peer_counts[rank];

  const size_t local_routes = static_cast<size_t>(config->max_tokens) * kTopK;
  const size_t cap = ep->capacity_rows;
  const size_t send_tiles = local_routes / kTileM + kExperts + 1;
  const size_t recv_tiles = cap / kTileM + kExperts + 1;
  const size_t chunks = (local_routes + 1023) / 1024;
  const size_t int_count = 3 * local_routes + 2 * (kExperts + 1) + send_tiles + 1 + chunks * kExperts + 1 +
                           2 * (kExperts + 1) + 2 * (recv_tiles + 1) + 1 +   // receive plan
                           4 * kExperts + kExperts + 64;                // tables + remap
  const size_t padded = cap + static_cast<size_t>(kExperts) * 127;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ep->ints), int_count * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ep->ints, 0, int_count * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ep->input_sf), padded * (kHidden / 16));
  if (e == cudaSuccess) e = cudaMemset(ep->input_sf, 0, padded * (kHidden / 16));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ep->inter_codes), cap * (kInter / 2));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ep->inter_sf), padded * (kInter / 16));
  if (e == cudaSuccess) e = cudaMemset(ep->inter_sf, 0, padded * (kInter / 16));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ep->row_dest), cap * sizeof(unsigned long long));
  if (e == cudaSuccess)
    e = cudaMalloc(reinterpret_cast<void**>(&ep->w13_sf_tiled), gv::retiled_w13_scale_bytes(el));
  if (e != cudaSuccess) {
    gevva_moe_ep_destroy(ep);
    return GEVVA_MOE_CUDA_ERROR;
  }
  int* cursor = ep->ints;
  auto carve = [&](size_t n) { int* p = cursor; cursor += n; return p; };
  gv::RoutePlan& sp = ep->send_plan;
  sp.sorted_experts = carve(local_routes);
  sp.sorted_routes = carve(local_routes);
  sp.inverse_routes = carve(local_routes);
  sp.expert_offsets = carve(kExperts + 1);
  sp.scale_row_offsets = carve(kExperts + 1);
  sp.tile_expert = carve(send_tiles);
  sp.num_m_tiles = carve(1);
  sp.chunk_hist = carve(chunks * kExperts);
  sp.status = carve(1);
  sp.sync = carve(2);  // from the 64 spare ints
  ep->split = carve(2 * gv::kMaxComputeChunks);
  gv::RoutePlan& rp = ep->receive_plan;
  rp.expert_offsets = carve(kExperts + 1);
  rp.scale_row_offsets = carve(kExperts + 1);
  rp.tile_expert = carve(recv_tiles);
  rp.num_m_tiles = carve(1);
  rp.pair_tile = carve(recv_tiles);
  rp.num_pairs = carve(1);
  rp.status = sp.status;
  ep->dev.send_row_base = carve(kExperts);
  ep->dev.send_src_prefix = carve(kExperts);
  ep->dev.send_scale_rows = carve(kExperts);
  ep->dev.source_offsets = carve(kExperts);
  int* remap = carve(kExperts);
  int host_remap[kExperts];
  for (int x = 0; x < kExperts; ++x) host_remap[x] = (x % world) * el + x / world;
  if (config->placement) {
    bool taken[kExperts] = {};
    for (int x = 0; x < kExperts; ++x) {
      const int v = config->placement[x];
      if (v < 0 || v >= kExperts || taken[v]) {  // not a permutation
        gevva_moe_ep_destroy(ep);
        return GEVVA_MOE_BAD_ARGUMENT;
      }
      taken[v] = true;
      host_remap[x] = v;
    }
  }
  e = cudaMemcpy(remap, host_remap, sizeof(host_remap), cudaMemcpyHostToDevice);
  ep->dev.remap = remap;
  sp.remap = remap;

  gv::launch_retile_w13_scales(static_cast<const uint8_t*>(local_weights->w13_sf), ep->w13_sf_tiled, el,
                               nullptr);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
  bool ok = e == cudaSuccess;
  ok = ok && make_map(&ep->w13.map_a, ep->dev.peer_codes[rank], cap, kHidden / 2, kTileM);
  ok = ok && make_map(&ep->w13.map_a32, ep->dev.peer_codes[rank], cap, kHidden / 2, 32);
  ok = ok && make_map(&ep->w2.map_a32, ep->inter_codes, cap, kInter / 2, 32);
  ok = ok && make_map(&ep->w13.map_b, local_weights->w13, static_cast<uint64_t>(el) * kW13Out,
                      kHidden / 2, kTileM);
  ok = ok && make_map(&ep->w13.map_b64, local_weights->w13, static_cast<uint64_t>(el) * kW13Out,
                      kHidden / 2, 64);
  ok = ok && make_map(&ep->w2.map_a, ep->inter_codes, cap, kInter / 2, kTileM);
  ok = ok && make_map(&ep->w2.map_b, local_weights->w2, static_cast<uint64_t>(el) * kHidden, kInter / 2,
                      kTileM);
  if (!ok) {
    gevva_moe_ep_destroy(ep);
    return GEVVA_MOE_CUDA_ERROR;
  }
  ep->w13.a_scales = ep->input_sf;
  ep->w13.b_scales = ep->w13_sf_tiled;
  ep->w13.alpha = local_weights->alpha1;
  ep->w13.out = nullptr;
  ep->w13.n_out = kW13Out;
  ep->w13.k_in = kHidden;
  ep->w13.fused_geglu = true;
  ep->w13.next_codes = ep->inter_codes;
  ep->w13.next_scales = ep->inter_sf;
  ep->w13.next_scale_q = local_weights->in_scale_q2;
  ep->w2.a_scales = ep->inter_sf;
  ep->w2.b_scales = static_cast<const uint8_t*>(local_weights->w2_sf);
  ep->w2.alpha = local_weights->alpha2;
  ep->w2.out = nullptr;
  ep->w2.row_dest = ep->row_dest;
  ep->w2.n_out = kHidden;
  ep->w2.k_in = kInter;
  ep->w2.fused_geglu = false;
  *out = ep;
  return GEVVA_MOE_OK;
}

int gevva_moe_ep_barrier(gevva_moe_ep* ep, gevva_stream_t stream) {
  if (!ep) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_chained(gv::ep_barrier_kernel, dim3(1), dim3(32), 0, stream, ep->dev, ++ep->epoch, ep->send_plan.status);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

int gevva_moe_ep_route_sort(gevva_moe_ep* ep, const int* ids, int tokens, gevva_stream_t stream) {
  if (!ep || !ids || tokens < 1 || tokens > ep->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_route_sort(ids, tokens * kTopK, ep->send_plan, stream);
  gv::launch_chained(gv::ep_exchange_kernel, dim3(1), dim3(kExperts), 0, stream, ep->dev, ep->send_plan, ep->receive_plan, ep->split,
                                                      ep->chunks, ep->first_share, ++ep->epoch, ep->send_plan.status);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

int gevva_moe_ep_dispatch(gevva_moe_ep* ep, const void* in, const int* ids, int tokens,
                          gevva_stream_t stream) {
  if (!ep || !in || !ids || tokens < 1 || tokens > ep->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_chained(gv::ep_dispatch_kernel, dim3((tokens + gv::kDispatchTokensPerBlock - 1) / gv::kDispatchTokensPerBlock),
                     dim3(gv::kDispatchThreads), 0, stream, static_cast<const __nv_bfloat16*>(in), ids, ep->in_scale_q1_global, ep->dev, ep->send_plan, tokens);
  // The combine address table depends on the count matrix only, so it is computed here, while
  // other ranks' rows are still arriving, rather than after the barrier that precedes
  // gevva_moe_ep_compute.
  ep->dispatch_epoch = ++ep->epoch;
  gv::launch_chained(gv::ep_row_destinations_kernel, dim3(ep->sm_count * 2), dim3(256), 0, stream, ep->dev, ep->receive_plan, ep->row_dest,
                                                                        ep->dispatch_epoch);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

namespace {
int run_compute(gevva_moe_ep* ep, const unsigned long long* row_dest, cudaStream_t stream, int await_epoch);
}

int gevva_moe_ep_compute(gevva_moe_ep* ep, gevva_stream_t stream) {
  if (!ep) return GEVVA_MOE_BAD_ARGUMENT;
  return run_compute(ep, ep->row_dest, stream, ep->dispatch_epoch);
}

int gevva_moe_ep_compute_local(gevva_moe_ep* ep, gevva_stream_t stream) {
  if (!ep) return GEVVA_MOE_BAD_ARGUMENT;
  if (!ep->row_dest_local &&
      cudaMalloc(reinterpret_cast<void**>(&ep->row_dest_local), ep->capacity_rows * sizeof(unsigned long long)) !=
          cudaSuccess)
    return GEVVA_MOE_CUDA_ERROR;
  gv::ep_row_destinations_local_kernel<<<ep->sm_count * 2, 256, 0, stream>>>(
      ep->dev, ep->receive_plan, ep->row_dest_local, ep->max_tokens * kTopK);
  return run_compute(ep, ep->row_dest_local, stream, 0);
}

int gevva_moe_ep_dispatch_local(gevva_moe_ep* ep, const void* in, const int* ids, int tokens,
                                gevva_stream_t stream) {
  if (!ep || !in || !ids || tokens < 1 || tokens > ep->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  gv::EpDevice local = ep->dev;
  for (int d = 0; d < local.world; ++d) {
    local.peer_codes[d] = ep->dev.peer_codes[ep->dev.rank];
    local.peer_scales[d] = ep->dev.peer_scales[ep->dev.rank];
  }
  gv::launch_chained(gv::ep_dispatch_kernel, dim3((tokens + gv::kDispatchTokensPerBlock - 1) / gv::kDispatchTokensPerBlock),
                     dim3(gv::kDispatchThreads), 0, stream, static_cast<const __nv_bfloat16*>(in), ids, ep->in_scale_q1_global, local, ep->send_plan, tokens);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

}  // extern "C"

namespace {
int run_compute(gevva_moe_ep* ep, const unsigned long long* row_dest, cudaStream_t stream, int await_epoch) {
  gv::GemmOperands w2 = ep->w2;
  w2.row_dest = row_dest;
  gv::launch_chained(gv::ep_swizzle_scales_kernel, dim3(ep->sm_count * 4), dim3(256), 0, stream,
                     ep->dev.peer_scales[ep->dev.rank], ep->dev, ep->receive_plan, ep->input_sf, await_epoch,
      ep->send_plan.status);
  // The local experts are processed in `chunks` parts of about equal rows.  A part's w2
  // is bound by the NVLink stores of its epilogue, not by the tensor pipe, so it runs on 64 SMs
  // of a side stream while the next part's w13 takes the other SMs; the first w13 and the
  // last w2 have the whole GPU.
  const int side_sms = ep->sm_count >= 128 ? 64 : ep->sm_count / 2;
  for (int part = 0; part < ep->chunks; ++part) {
    gv::RoutePlan plan = ep->receive_plan;
    plan.tile_first = ep->split + 2 * part;
    plan.num_m_tiles = ep->split + 2 * part + 1;
    const bool last = part + 1 == ep->chunks;
    gv::launch_grouped_gemm(ep->w13, plan, part == 0 ? ep->sm_count : ep->sm_count - side_sms, stream);
    if (!last) {
      cudaEventRecord(ep->fork, stream);
      cudaStreamWaitEvent(ep->side, ep->fork, 0);
      gv::launch_grouped_gemm(w2, plan, side_sms, ep->side);
    } else {
      // launched the ordinary way: its CTAs must not take SMs (and wait there) before this
      // part's w13 has ended, or the previous part's w2 would be left without room
      gv::GemmOperands serial = w2;
      serial.serial_launch = true;
      gv::launch_grouped_gemm(serial, plan, ep->sm_count, stream);
    }
  }
  cudaEventRecord(ep->join, ep->side);
  cudaStreamWaitEvent(stream, ep->join, 0);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}
}  // namespace

extern "C" {

int gevva_moe_ep_reduce(gevva_moe_ep* ep, const float* route_weights, void* out, int tokens,
                        gevva_stream_t stream) {
  if (!ep || !route_weights || !out || tokens < 1 || tokens > ep->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_reduce_routes(ep->dev.peer_combine[ep->dev.rank], route_weights,
                           ep->send_plan.inverse_routes, tokens, out, stream);
  return cudaGetLastError() == cudaSuccess ? GEVVA_MOE_OK : GEVVA_MOE_CUDA_ERROR;
}

int gevva_moe_ep_status(gevva_moe_ep* ep, int* received_rows) {
  if (!ep) return GEVVA_MOE_BAD_ARGUMENT;
  int status = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return GEVVA_MOE_CUDA_ERROR;
  if (cudaMemcpy(&status, ep->send_plan.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return GEVVA_MOE_CUDA_ERROR;
  if (status) cudaMemset(ep->send_plan.status, 0, sizeof(int));
  if (received_rows)
    cudaMemcpy(received_rows, ep->receive_plan.expert_offsets + kExperts, sizeof(int),
               cudaMemcpyDeviceToHost);
  return -status;
}

}  // extern "C"
