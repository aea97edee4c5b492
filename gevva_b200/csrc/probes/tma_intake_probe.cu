// Measures how many bytes per second an SM takes in through bulk copies into shared memory with a
// bounded number of bytes in flight, all SMs at once: from a footprint that stays in L2 (every CTA
// re-reads its own 216 KiB), from one that streams from HBM, and with several CTAs reading the same
// bytes.  The stage sizes are those of the expert GEMMs (54 KiB per K block for one CTA per tile,
// 38 KiB for a CTA pair).  Build: python -m gevva_b200.build --probes
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "../gv_common.cuh"
using namespace gv;

__global__ void __launch_bounds__(128, 1) stream(const uint8_t* source, size_t footprint_per_cta, int chunk, int depth,
                                                 int pieces, int iterations, int sharing, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[16];
  if (threadIdx.x == 0) {
    for (int s = 0; s < 16; ++s) mbar_init(&bar[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint8_t* src = source + static_cast<size_t>(blockIdx.x / sharing) * footprint_per_cta;
    const int piece = chunk / pieces;
    size_t offset = 0;
    const long long t0 = clock64();
    const uint64_t g0 = global_timer_ns();
    for (int it = 0; it < iterations; ++it) {
      const int s = it % depth;
      if (it >= depth && !mbar_wait_bounded(&bar[s], ((it / depth) - 1) & 1, 4000000000ll)) break;
      mbar_arrive_expect_tx(&bar[s], chunk);
      for (int q = 0; q < pieces; ++q)
        bulk_load_1d(smem + s * chunk + q * piece, src + offset + q * piece, piece, &bar[s]);
      offset += chunk;
      if (offset + chunk > footprint_per_cta) offset = 0;
    }
    for (int it = iterations; it < iterations + depth; ++it)
      mbar_wait_bounded(&bar[it % depth], ((it / depth) - 1) & 1, 4000000000ll);
    out[blockIdx.x * 2] = clock64() - t0;
    out[blockIdx.x * 2 + 1] = static_cast<long long>(global_timer_ns() - g0);
  }
}

int main() {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  long long* d;
  cudaMalloc(&d, sms * 16);
  const size_t total = static_cast<size_t>(4) << 30;
  uint8_t* src;
  if (cudaMalloc(&src, total) != cudaSuccess) {
    printf("cudaMalloc of 4 GiB failed\n");
    return 1;
  }
  cudaMemset(src, 0x33, total);
  cudaFuncSetAttribute(stream, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  long long* h = new long long[sms * 2];
  struct Case { const char* name; size_t footprint; int chunk, depth, pieces, sharing; };
  const size_t hot = 216 * 1024, cold = ((total / sms) / (216 * 1024)) * (216 * 1024);
  const Case cases[] = {
      {"L2-resident, 4 x 54 KiB in flight", hot, 54 * 1024, 4, 2, 1},
      {"L2-resident, 3 x 54 KiB in flight", hot, 54 * 1024, 3, 2, 1},
      {"L2-resident, 8 x 27 KiB in flight", hot, 27 * 1024, 8, 1, 1},
      {"L2-resident, 5 x 38 KiB in flight", hot, 38 * 1024, 5, 2, 1},
      {"L2-resident, 2 CTAs read the same bytes, 4 x 54 KiB", hot, 54 * 1024, 4, 2, 2},
      {"L2-resident, 4 CTAs read the same bytes, 4 x 54 KiB", hot, 54 * 1024, 4, 2, 4},
      {"from HBM,    4 x 54 KiB in flight", cold, 54 * 1024, 4, 2, 1},
      {"from HBM,    5 x 38 KiB in flight", cold, 38 * 1024, 5, 2, 1},
      {"from HBM, 2 CTAs read the same bytes, 4 x 54 KiB", cold, 54 * 1024, 4, 2, 2},
      {"from HBM, 4 CTAs read the same bytes, 4 x 54 KiB", cold, 54 * 1024, 4, 2, 4},
  };
  for (int pass = 0; pass < 2; ++pass)
    for (const Case& c : cases) {
      const int iterations = 1500;
      stream<<<sms, 128, 220 * 1024>>>(src, c.footprint, c.chunk, c.depth, c.pieces, iterations, c.sharing, d);
      const cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) {
        printf("%s: %s\n", c.name, cudaGetErrorString(e));
        return 1;
      }
      cudaMemcpy(h, d, sms * 16, cudaMemcpyDeviceToHost);
      double ns = 0;
      for (int i = 0; i < sms; ++i) ns += h[2 * i + 1];
      ns /= sms;
      const double per_sm = static_cast<double>(c.chunk) * iterations / ns;  // GB/s
      printf("pass %d  %-50s ns per stage %7.1f   per SM %6.1f GB/s   all SMs %6.2f TB/s\n", pass, c.name,
             ns / iterations, per_sm, per_sm * sms / 1000);
    }
  return 0;
}
