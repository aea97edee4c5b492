// Measures what the tensor pipe of an SM sustains for the K block of the expert GEMMs: four
// block-scaled NVFP4 MMAs (128 x 256 x 64, or 256 x 256 x 64 on a CTA pair) with and without
// the twelve scale-factor copies of the block, all SMs at once, operands resident in shared
// memory (no loads).  Prints SM cycles and nanoseconds per K block; the tensor-pipe time of a
// K block is 512 cycles.  Build: python -m gevva_b200.build --probes
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "../gv_common.cuh"
using namespace gv;

constexpr int kBlocks = 3000;          // K blocks per launch
constexpr int kStageBytes = 54 * 1024; // [activations 16 KiB][weights 32 KiB][scales 6 KiB]

enum Variant { kMma = 0, kMmaCopies = 1, kCopies = 2, kMmaCopiesOtherWarp = 3, kPairMma = 4, kPairMmaCopies = 5, kVariants = 6 };

__device__ __forceinline__ void fill(uint8_t* smem, int bytes) {
  for (int i = threadIdx.x; i < bytes / 4; i += blockDim.x) {
    uint32_t h = (i + blockIdx.x * 7919u) * 2654435761u;
    h ^= h >> 15;
    reinterpret_cast<uint32_t*>(smem)[i] = h & 0x77777777u;  // finite E2M1 codes and E4M3 scales
  }
}

template <bool kPair>
__device__ __forceinline__ void copy_sf(uint32_t tmem, uint64_t desc) {
  if (kPair) asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(desc) : "memory");
  else asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(desc) : "memory");
}

template <bool kPair>
__device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                    uint32_t accumulate) {
  if (kPair)
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}

template <bool kPair>
__device__ __forceinline__ void run(int variant, uint8_t* smem, long long* out) {
  __shared__ uint64_t done, done_other;
  __shared__ uint32_t tmem_slot;
  fill(smem, 4 * kStageBytes);
  if (threadIdx.x == 0) {
    mbar_init(&done, 1);
    mbar_init(&done_other, 1);
    fence_barrier_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (kPair) cluster_sync_all();
  const uint32_t tmem = tmem_slot;
  const bool leader_cta = !kPair || cluster_cta_rank() == 0;
  const uint64_t hi_ab = static_cast<uint64_t>((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
  const uint64_t hi_sf = static_cast<uint64_t>((128u >> 4) | (1u << 14)) << 32;
  const uint32_t idesc = (1u << 7) | (1u << 10) | (uint32_t(256 >> 3) << 17) | (uint32_t((kPair ? 256 : 128) >> 4) << 24);
  const bool with_mma = variant != kCopies;
  const bool copies_here = variant == kMmaCopies || variant == kCopies || variant == kPairMmaCopies;
  auto copies = [&](int stage) {
    const uint32_t sf_lo = (smem_u32(smem + stage * kStageBytes + 48 * 1024) & 0x3ffff) >> 4;
    const uint32_t ts = tmem + 256 + 48 * stage;
#pragma unroll
    for (int j = 0; j < 12; ++j) copy_sf<kPair>(ts + 4 * j, hi_sf | (sf_lo + j * 32));
  };
  const int warp = threadIdx.x >> 5;
  if (warp == 0 && leader_cta) {
    if (elect_one()) {
      const long long t0 = clock64();
      const uint64_t g0 = global_timer_ns();
      for (int it = 0; it < kBlocks; ++it) {
        const int stage = it & 3;
        if (copies_here) copies(stage);
        if (with_mma) {
          const uint32_t a_lo = (smem_u32(smem + stage * kStageBytes) & 0x3ffff) >> 4;
          const uint32_t b_lo = (smem_u32(smem + stage * kStageBytes + 16384) & 0x3ffff) >> 4;
          const uint32_t ts = tmem + 256 + 48 * stage;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mma<kPair>(tmem, hi_ab | (a_lo + j * 2), hi_ab | (b_lo + j * 2), idesc, ts + 12 * j, ts + 12 * j + 4,
                       (it | j) ? 1u : 0u);
        }
      }
      if (kPair)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&done)) : "memory");
      else
        tc_commit(&done);
      mbar_wait_bounded(&done, 0, 4000000000ll);
      out[blockIdx.x * 2] = clock64() - t0;
      out[blockIdx.x * 2 + 1] = static_cast<long long>(global_timer_ns() - g0);
    }
    __syncwarp();
  } else if (warp == 1 && variant == kMmaCopiesOtherWarp) {
    // unsynchronised with the MMA thread: only the rates matter here
    if (elect_one()) {
      for (int it = 0; it < kBlocks; ++it) copies(it & 3);
      tc_commit(&done_other);
      mbar_wait_bounded(&done_other, 0, 4000000000ll);
    }
    __syncwarp();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync_all();
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

__global__ void __launch_bounds__(128, 1) probe_single(int variant, long long* out) {
  extern __shared__ uint8_t raw[];
  run<false>(variant, reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023)), out);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) probe_pair(int variant, long long* out) {
  extern __shared__ uint8_t raw[];
  run<true>(variant, reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023)), out);
}

int main() {
  const char* names[kVariants] = {"4 MMA",
                                  "4 MMA + 12 scale copies, one thread",
                                  "12 scale copies",
                                  "4 MMA + 12 scale copies from another warp",
                                  "CTA pair: 4 MMA (M = 256)",
                                  "CTA pair: 4 MMA + 12 scale copies"};
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  sms &= ~1;
  long long* d;
  cudaMalloc(&d, sms * 16);
  cudaMemset(d, 0, sms * 16);
  cudaFuncSetAttribute(probe_single, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  cudaFuncSetAttribute(probe_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  long long* h = new long long[sms * 2];
  for (int rep = 0; rep < 2; ++rep)
    for (int v = 0; v < kVariants; ++v) {
      const bool pair = v >= kPairMma;
      cudaMemset(d, 0, sms * 16);
      if (pair) probe_pair<<<sms, 128, 220 * 1024>>>(v, d);
      else probe_single<<<sms, 128, 220 * 1024>>>(v, d);
      const cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) {
        printf("%s: %s\n", names[v], cudaGetErrorString(e));
        return 1;
      }
      cudaMemcpy(h, d, sms * 16, cudaMemcpyDeviceToHost);
      double cycles = 0, ns = 0;
      int reporting = 0;
      for (int i = 0; i < sms; ++i)
        if (h[2 * i]) {
          cycles += h[2 * i];
          ns += h[2 * i + 1];
          ++reporting;
        }
      cycles /= reporting;
      ns /= reporting;
      printf("pass %d  %-44s cycles per K block %6.1f   ns per K block %6.1f   SM clock %.2f GHz\n", rep, names[v],
             cycles / kBlocks, ns / kBlocks, cycles / ns);
    }
  return 0;
}
