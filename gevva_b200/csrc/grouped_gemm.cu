// Grouped block-scaled NVFP4 GEMM for sm_100a: tcgen05.mma kind::mxf4nvf4 with
// UE4M3 scales per 16 elements, fp32 accumulators in tensor memory, operands
// brought in by TMA into 128-byte-swizzled shared memory.
//
// Replaces the reference's CUTLASS SM120 grouped GEMM
// (src/nvfp4_cutlass.cu:81-100 traits, :755-962 plan, :913-930 run):
//   D_e[r, n] = bf16(alpha[e] * sum_k A[r,k] sfa[r,k/16] B_e[n,k] sfb_e[n,k/16])
// for the rows r of each expert e, over all 128 experts in one launch.
//
// Mapping.  Tokens (sorted routes) sit on MMA-M, weight rows on MMA-N.  A work
// item is (128-row tile of one expert) x (128 weight rows).  Row tiles are listed
// in device memory by the route sort; CTAs are persistent and take items
// round-robin.  Warp 0 is the TMA producer, warp 1 allocates tensor memory and
// issues the MMAs, warps 2..5 drain accumulators (two accumulator stages, so the
// epilogue of one item overlaps the main loop of the next).
//
// Scale factors.  Both operands keep scales in the 128-row x 4-scale atoms of
// 512 bytes (row%32)*16 + (row/32)*4 + k that the reference writes
// (src/nvfp4_cutlass.cu:321-323); one atom is exactly what one MMA (K = 64)
// consumes and what tcgen05.cp 32x128b.warpx4 moves, so a K block of 256 needs a
// contiguous 2 KiB per operand, fetched with one untiled bulk copy.
//
// Every wait is bounded: on expiry the kernel records kWaitTimeout in the status
// word, all roles leave their loops, tensor memory is released and the CTA exits.
#include "gv_common.cuh"
#include "gv_launchers.h"

namespace gv {

namespace {

constexpr int kStages = 5;
constexpr int kAccStages = 2;
constexpr int kGemmThreads = 192;
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kSfaColumn = kAccStages * kTileN;  // 256
constexpr uint32_t kSfbColumn = kSfaColumn + 16;      // 272
constexpr int kOperandStageBytes = kTileM * kTileKBytes;  // 16 KiB, same for A and B

struct alignas(1024) GemmSmem {
  uint8_t a[kStages][kOperandStageBytes];
  uint8_t b[kStages][kOperandStageBytes];
  uint8_t sfa[kStages][kSfStageBytes];
  uint8_t sfb[kStages][kSfStageBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint32_t tmem_base;
  volatile int abort;
};

constexpr size_t kGemmSmemBytes = sizeof(GemmSmem) + 1024;  // slack for manual alignment

// Instruction descriptor: E2M1 x E2M1 (format 1 in the mxf4 kinds), both K-major,
// UE4M3 scales (bit 23 clear), N at [17,23) in units of 8, M at [24,29) in units of 16,
// K = 64 (bit 31 clear), scale ids 0.
constexpr uint32_t kInstrDesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
                                (static_cast<uint32_t>(kTileM >> 4) << 24);

struct GemmParams {
  const uint8_t* a_scales;
  const uint8_t* b_scales;
  const float* alpha;
  __nv_bfloat16* out;
  const int* tile_expert;
  const int* expert_offsets;
  const int* scale_row_offsets;
  const int* num_m_tiles;
  int* status;
  int n_out;
  int n_tiles;      // n_out / 128
  int groups;       // k_in / 16
  int k_blocks;     // ceil(k_in / 256)
  int last_mmas;    // MMAs (K = 64 each) in the last K block, 1..4
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, GemmSmem* smem,
                                              int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      if (smem->abort) return false;
      if (global_timer_ns() - start > 1000000000ull) {
        smem->abort = 1;
        atomicExch(status, static_cast<int>(kWaitTimeout));
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmem* smem = reinterpret_cast<GemmSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&smem->full[s], 1);
      mbar_init(&smem->empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&smem->acc_full[s], 1);
      mbar_init(&smem->acc_empty[s], 128);
    }
    smem->abort = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = smem->tmem_base;

  const int total_items = p.num_m_tiles[0] * p.n_tiles;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int m_tile = item / p.n_tiles;
        const int n_tile = item - m_tile * p.n_tiles;
        const int expert = p.tile_expert[m_tile];
        const int row0 = p.expert_offsets[expert] + (m_tile * kTileM - p.scale_row_offsets[expert]);
        const int b_row = expert * p.n_out + n_tile * kTileN;
        const uint8_t* sfa_src = p.a_scales + static_cast<size_t>(m_tile) * kTileM * p.groups;
        const uint8_t* sfb_src = p.b_scales + static_cast<size_t>(b_row) * p.groups;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_or_abort(&smem->empty[stage], phase ^ 1u, smem, p.status)) {
            ok = false;
            break;
          }
          const uint32_t sf_bytes =
              (kb == p.k_blocks - 1 ? p.last_mmas : 4) * static_cast<uint32_t>(kSfAtomBytes);
          mbar_arrive_expect_tx(&smem->full[stage], 2u * kOperandStageBytes + 2u * sf_bytes);
          tma_load_2d(smem->a[stage], &map_a, &smem->full[stage], kb * kTileKBytes, row0);
          tma_load_2d(smem->b[stage], &map_b, &smem->full[stage], kb * kTileKBytes, b_row);
          bulk_load_1d(smem->sfa[stage], sfa_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes,
                       &smem->full[stage]);
          bulk_load_1d(smem->sfb[stage], sfb_src + static_cast<size_t>(kb) * kSfStageBytes, sf_bytes,
                       &smem->full[stage]);
          ++issued;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Unwinding: let the copies already issued land before shared memory is given up.
        const int pending = issued < kStages ? issued : kStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = kStages - 1;
            ph ^= 1u;
          }
          mbar_wait_bounded(&smem->full[s], ph, 20000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc_stage = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        if (!wait_or_abort(&smem->acc_empty[acc_stage], acc_phase ^ 1u, smem, p.status)) break;
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc_stage * kTileN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_or_abort(&smem->full[stage], phase, smem, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const int mmas = kb == p.k_blocks - 1 ? p.last_mmas : 4;
          const uint32_t sfa_addr = smem_u32(smem->sfa[stage]);
          const uint32_t sfb_addr = smem_u32(smem->sfb[stage]);
          for (int j = 0; j < mmas; ++j) {
            tc_copy_sf(tmem_base + kSfaColumn + 4u * j,
                       make_smem_desc(sfa_addr + j * kSfAtomBytes, 128, 0));
            tc_copy_sf(tmem_base + kSfbColumn + 4u * j,
                       make_smem_desc(sfb_addr + j * kSfAtomBytes, 128, 0));
          }
          const uint64_t desc_a = make_smem_desc(smem_u32(smem->a[stage]), 1024, 2);
          const uint64_t desc_b = make_smem_desc(smem_u32(smem->b[stage]), 1024, 2);
          for (int j = 0; j < mmas; ++j) {
            // 64 FP4 elements = 32 bytes along K inside the swizzle row: +2 in 16-byte units
            tc_mma_nvfp4(tmem_acc, desc_a + 2u * j, desc_b + 2u * j, kInstrDesc,
                         tmem_base + kSfaColumn + 4u * j, tmem_base + kSfbColumn + 4u * j,
                         (kb | j) != 0 ? 1u : 0u);
          }
          tc_commit(&smem->empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(&smem->acc_full[acc_stage]);
        if (++acc_stage == kAccStages) {
          acc_stage = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, one 32-lane quarter each ----------------
    const int quarter = warp & 3;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const int m_tile = item / p.n_tiles;
      const int n_tile = item - m_tile * p.n_tiles;
      const int expert = p.tile_expert[m_tile];
      const int local0 = m_tile * kTileM - p.scale_row_offsets[expert];
      const int row0 = p.expert_offsets[expert] + local0;
      const int rows_valid = p.expert_offsets[expert + 1] - row0;  // may exceed 128
      const float alpha = p.alpha[expert];
      if (!wait_or_abort(&smem->acc_full[acc_stage], acc_phase, smem, p.status)) break;
      tc_fence_after_sync();
      const int row_local = quarter * 32 + lane;
      const bool valid = row_local < rows_valid;
      __nv_bfloat16* dst = p.out + static_cast<size_t>(row0 + row_local) * p.n_out + n_tile * kTileN;
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                static_cast<uint32_t>(acc_stage * kTileN);
#pragma unroll 1
      for (int chunk = 0; chunk < kTileN / 32; ++chunk) {
        uint32_t r[32];
        tmem_load_32x32(tmem_row + chunk * 32, r);
        tmem_load_wait();
        if (valid) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const __nv_bfloat162 pair =
                __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(r[2 * i])),
                                      __fmul_rn(alpha, __uint_as_float(r[2 * i + 1])));
            packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
          }
          uint4* out16 = reinterpret_cast<uint4*>(dst + chunk * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            out16[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&smem->acc_empty[acc_stage]);
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

}  // namespace

int prepare_grouped_gemm() {
  return static_cast<int>(cudaFuncSetAttribute(grouped_nvfp4_gemm_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kGemmSmemBytes)));
}

void launch_grouped_gemm(const GemmOperands& op, const RoutePlan& plan, int sm_count,
                         cudaStream_t stream) {
  GemmParams p;
  p.a_scales = op.a_scales;
  p.b_scales = op.b_scales;
  p.alpha = op.alpha;
  p.out = static_cast<__nv_bfloat16*>(op.out);
  p.tile_expert = plan.tile_expert;
  p.expert_offsets = plan.expert_offsets;
  p.scale_row_offsets = plan.scale_row_offsets;
  p.num_m_tiles = plan.num_m_tiles;
  p.status = plan.status;
  p.n_out = op.n_out;
  p.n_tiles = op.n_out / kTileN;
  p.groups = op.k_in / 16;
  p.k_blocks = (op.k_in + kTileK - 1) / kTileK;
  p.last_mmas = (op.k_in - (p.k_blocks - 1) * kTileK) / 64;
  grouped_nvfp4_gemm_kernel<<<sm_count, kGemmThreads, kGemmSmemBytes, stream>>>(op.map_a, op.map_b, p);
}

}  // namespace gv
