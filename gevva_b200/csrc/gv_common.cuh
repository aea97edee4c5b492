// Shared constants, status codes and sm_100a PTX wrappers for the MoE path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gv_transcendentals.h"

namespace gv {

constexpr int kExperts = 128;
constexpr int kTopK = 8;
constexpr int kHidden = 2816;        // H
constexpr int kInter = 704;          // I
constexpr int kW13Out = 2 * kInter;  // rows of the fused [up;gate] weight

// Values of the device status word and of the C ABI's return codes (negated).
enum Status : int {
  kOk = 0,
  kBadExpertId = 1,     // an expert id outside [0,128) reached the route sort
  kWaitTimeout = 2,     // a bounded mbarrier wait ran out inside a GEMM kernel
  kBadArgument = 3,
  kCudaError = 4,
  kNoDevice = 5,
  kTooLarge = 6,
};

// Tile geometry of the grouped GEMM (tokens on MMA-M, weight rows on MMA-N).
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kTileKBytes = 128;               // 256 FP4 elements = one 128B swizzle row
constexpr int kTileK = 2 * kTileKBytes;
constexpr int kSfAtomBytes = 512;              // 128 rows x 4 scale bytes (K = 64)
constexpr int kSfStageBytes = 4 * kSfAtomBytes;

// erf coefficient table; kernels copy it to shared memory once (load_erf_table) because
// lanes read different rows of it.
static __constant__ float g_erf_table[8][8] = GV_ERF_TABLE_INIT;

__device__ __forceinline__ void load_erf_table(float* shared_table) {
  if (threadIdx.x < GV_ERF_TABLE_FLOATS) shared_table[threadIdx.x] = g_erf_table[threadIdx.x >> 3][threadIdx.x & 7];
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// E4M3 decode by bit arithmetic (exact; NaN codes do not occur for scales made by
// the saturating encoder).
__device__ __forceinline__ float decode_e4m3(uint32_t code) {
  const uint32_t exponent = (code >> 3) & 15u;
  const uint32_t mant = code & 7u;
  const float mag = exponent == 0 ? __uint2float_rn(mant) * 0.001953125f
                                  : __uint_as_float(((exponent + 120u) << 23) | (mant << 20));
  return (code & 0x80u) ? -mag : mag;
}

__device__ __forceinline__ uint32_t encode_e4m3(float value) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3));
}

// Two floats -> one byte, low nibble = first (cvt.rn.satfinite.e2m1x2.f32).
__device__ __forceinline__ uint32_t encode_e2m1x2(float first, float second) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp4x2(float2{first, second}, __NV_E2M1, cudaRoundNearest));
}

// NVFP4 block quantiser for 16 values held in registers
// (reference: src/nvfp4_cutlass.cu:304-320).  Returns the E4M3 scale byte and the
// eight code bytes packed into two 32-bit words.
__device__ __forceinline__ uint32_t quantize_block16(const float (&values)[16], float multiplier,
                                                     uint32_t& codes_lo, uint32_t& codes_hi) {
  float maximum = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) maximum = fmaxf(maximum, fabsf(values[i]));
  const float unrounded = __fdiv_rn(__fmul_rn(multiplier, maximum), 6.0f);
  const uint32_t scale = encode_e4m3(unrounded);
  const float rounded = decode_e4m3(scale);
  const float inverse = rounded == 0.0f ? 0.0f : __fdiv_rn(multiplier, rounded);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    lo |= encode_e2m1x2(__fmul_rn(values[2 * pair], inverse),
                        __fmul_rn(values[2 * pair + 1], inverse)) << (8 * pair);
    hi |= encode_e2m1x2(__fmul_rn(values[8 + 2 * pair], inverse),
                        __fmul_rn(values[9 + 2 * pair], inverse)) << (8 * pair);
  }
  codes_lo = lo;
  codes_hi = hi;
  return scale;
}

// Byte offset of scale (row, group) inside one operand region; 128-row blocks
// major, four-group atoms next (reference: src/nvfp4_cutlass.cu:321-323).
__host__ __device__ __forceinline__ size_t sf_offset(int row, int group, int groups) {
  return static_cast<size_t>(row >> 7) * (128u * static_cast<size_t>(groups)) +
         static_cast<size_t>(group >> 2) * 512u + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (group & 3);
}

// ----------------------------------------------------------------------------
// PTX wrappers (sm_100a)
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

// True in exactly one lane of a fully active warp (the same lane every time).
__device__ __forceinline__ bool elect_one() {
  uint32_t elected;
  asm volatile(
      "{\n\t"
      ".reg .b32 leader;\n\t"
      ".reg .pred p;\n\t"
      "elect.sync leader|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(elected));
  return elected != 0;
}

// Programmatic dependent launch.  A kernel launched with launch_chained() below may begin
// while its predecessor in the stream is still running; it must call grid_dependency_wait()
// before it touches anything the predecessor (or any earlier kernel) reads or writes.  The
// wait returns once the predecessor has completed and its writes are visible; in a kernel
// launched the ordinary way it returns at once.  grid_launch_dependents() lets the successor
// start its own preamble early.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Host side: launches `kernel` so that it may start before the previous kernel of `stream`
// has finished (see grid_dependency_wait above).  Every kernel launched this way waits at its
// top, so results are those of ordinary stream order.
template <class... Params, class... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes,
                                  cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

// Non-blocking phase test.  The pollers below spin on this rather than on
// mbarrier.try_wait: try_wait may suspend the thread for a hardware-defined time, which
// measured here as roughly 300 extra cycles per wait in the MMA-issuing thread even for
// phases that had completed long before.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait: gives up after `limit_cycles` SM clock cycles and reports false.  The
// caller records the failure in the status word and unwinds; nothing spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0 && clock64() - start > limit_cycles) return false;
  }
}

// Bounded wait on an mbarrier.  The time limit is kept with the SM's cycle counter (a
// cheap register read); it is consulted only every 1024 failed polls so that a short
// stall costs nothing but the polls themselves.
constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s at 2 GHz

// kBackoff: sleep between polls.  Warps that wait with slack (producers, epilogue) must not
// spin, because a spinning warp takes issue slots from the MMA warp on the same scheduler and
// every instruction of the main loop then costs several times its latency.
template <bool kBackoff, class Smem>
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Smem* smem,
                                              int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (kBackoff) __nanosleep(spin < 8 ? 32 : 128);
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & (kBackoff ? 63u : 1023u)) == 0) {
      if (smem->abort) return false;
      if (clock64() - start > kWaitLimitCycles) {
        smem->abort = 1;
        if (status) atomicExch(status, static_cast<int>(kWaitTimeout));
        return false;
      }
    }
  }
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// TMA tiled 2-D load, global -> shared, completion on an mbarrier.  x is the
// innermost (byte) coordinate and must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tensor_map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Untiled bulk copy, global -> shared; both addresses 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_tensor_map(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---- thread-block clusters ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// Barrier over every thread of the cluster; writes to (distributed) shared memory made before
// the arrive are visible to every thread after its wait.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address, in the cluster's shared window, of the byte that `local_address` names in the CTA of
// rank `cta_rank`.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local_address, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(cta_rank));
  return remote;
}

// Posted store into the shared memory of a CTA of the cluster; visible to that CTA after the next
// cluster barrier.
__device__ __forceinline__ void cluster_store_uint4(uint32_t cluster_address, uint4 v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_address), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float4 cluster_load_float4(uint32_t cluster_address) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_address)
               : "memory");
  return v;
}

// ---- tensor memory ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives on the mbarrier once every tcgen05 operation issued so far by this
// thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Shared -> tensor memory copy of one 32-row x 16-byte scale-factor atom,
// replicated into all four 32-lane quarters.
__device__ __forceinline__ void tc_copy_sf(uint32_t tmem_address, uint64_t smem_descriptor) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address),
               "l"(smem_descriptor)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T with per-16-element UE4M3 scales read from
// tensor memory; E2M1 operands; M = 128, K = 64.
__device__ __forceinline__ void tc_mma_nvfp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t instr_desc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(instr_desc), "r"(accumulate), "r"(tmem_sfa),
        "r"(tmem_sfb)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread.
__device__ __forceinline__ void tmem_load_32x32(uint32_t tmem_address, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(tmem_address)
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread.
__device__ __forceinline__ void tmem_load_32x16(uint32_t tmem_address, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(tmem_address)
      : "memory");
}

// Barrier among `threads` threads (a multiple of 32) that all name the same id (1..15).
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version 1).
//   layout: 0 = no swizzle, 2 = 128-byte swizzle
//   stride_bytes: distance between 8-row groups
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_address, uint32_t stride_bytes,
                                                   uint32_t layout) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);   // start address, bits [0,14)
  desc |= static_cast<uint64_t>(stride_bytes >> 4) << 32;          // stride byte offset, [32,46)
  desc |= 1ull << 46;                                              // descriptor version
  desc |= static_cast<uint64_t>(layout) << 61;                     // swizzle mode, [61,64)
  return desc;
}

}  // namespace gv
