// Router projection fused with top-8 routing, for sm_100a.
//
// The reference computes the router logits with a library GEMM and then routes
// (src/cuda/runtime/prefill.cuh:414-422, :1203-1210: cublasGemmEx / cuBLASLt FP8
// [tokens,2816] x [128,2816]^T -> bf16 [tokens,128], followed by
// route_128_top8_kernel<<<tokens,128>>>).  Here both are one kernel and the logits never
// reach HBM: tokens sit on MMA-M (128 per tile), the 128 experts on MMA-N, K = 2816.
//
// A tile's K range is split over a cluster of four CTAs (two, or one, for batches whose tiles
// would otherwise not fit one wave of SMs; eight for batches of at most 512 tokens), so a
// 4096-token batch runs on 128 SMs and a decode-sized batch streams the router matrix through
// eight SMs instead of one.  Each
// CTA accumulates its K slice in tensor memory (tcgen05.mma kind::f16 for bf16 operands,
// kind::f8f6f4 for E4M3).  Tile row r belongs to CTA r % split of the cluster: every CTA stores
// its 128 x 128 fp32 partial sums row by row straight into the owners' shared memory (posted
// st.shared::cluster stores), and after one cluster barrier each owner sums the partials of its
// 128 / split rows in rank order (a fixed order: results do not depend on timing), adds the optional
// per-expert bias, rounds to bf16 as the GEMM would have stored it, and routes its rows with four
// lanes per token (gv_route.cuh).
//
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer and owner of tensor memory, warps
// 2..5 epilogue (thread = accumulator row).  Every mbarrier wait is bounded (status word
// kWaitTimeout); the cluster barrier is reached by every thread whatever happened before.
#include "gv_common.cuh"
#include "gv_launchers.h"
#include "gv_route.cuh"

namespace gv {

namespace {

// CTAs per cluster = K slices per token tile: 8 for small batches, else 4, 2 or 1, the largest that
// keeps the launch within one wave of SMs (a tile's pass is a chain of latencies, so waves cost more
// than depth)
constexpr int kRpStages = 5;
constexpr int kRpThreads = 192;
constexpr int kRpTileBytes = kTileM * kTileKBytes;  // 16 KiB: 128 rows of one 128-byte K block

struct alignas(1024) RouterSmem {
  uint8_t a[kRpStages][kRpTileBytes];
  uint8_t b[kRpStages][kRpTileBytes];
  // Partial sums of this CTA's 32 rows as received from the four CTAs of the cluster (its own
  // included): [source][local row][128 floats]; the 16-byte chunks of a row are permuted
  // (received_chunk_position) so that neither the row-wise stores nor the reduce's reads, where
  // four lanes share a row, meet in a bank.
  float received[kTileM * kExperts];   // [kSplit][128 / kSplit rows][128 floats]
  uint64_t full[kRpStages];
  uint64_t empty[kRpStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  volatile int abort;
};

// Position of 16-byte chunk `chunk` (0..31) inside local row `row`: the chunk's low three bits are
// XORed with (row + 2 * (chunk / 8)) % 8.  For a fixed chunk, eight consecutive rows fall into eight
// different bank groups (the stores); for a fixed chunk % 8, two consecutive rows times the four
// column quarters do too (the loads of a quarter-warp).
__device__ __forceinline__ int received_chunk_position(int chunk, int row) {
  return chunk ^ ((row + 2 * (chunk >> 3)) & 7);
}

constexpr size_t kRpSmemBytes = sizeof(RouterSmem) + 1024;
static_assert(kRpSmemBytes <= 232448, "shared memory budget of one sm_100 CTA");

struct RouterParams {
  const float* bias;                   // optional f32 [128], added before the bf16 rounding
  const __nv_bfloat16* expert_scale;   // bf16 [128]
  float* weights;                      // f32 [tokens, 8]
  int* ids;                            // i32 [tokens, 8]
  __nv_bfloat16* logits_out;           // optional bf16 [tokens, 128]
  const float* activation_scales;      // E4M3 form: f32 [tokens]
  const float* weight_scale;           // E4M3 form: f32 [1]
  int* status;                         // optional device status word
  int tokens;
  int k_blocks;                        // 128-byte K blocks per row
};

// Instruction descriptors: fp32 accumulate (bit 4), both operands K-major, N at [17,23) in units
// of 8, M at [24,29) in units of 16; operand formats at [7,10) and [10,13): BF16 = 1 in
// kind::f16, E4M3 = 0 in kind::f8f6f4.
constexpr uint32_t kIdescBase = (1u << 4) | (static_cast<uint32_t>(kExperts >> 3) << 17) |
                                (static_cast<uint32_t>(kTileM >> 4) << 24);
constexpr uint32_t kIdescBf16 = kIdescBase | (1u << 7) | (1u << 10);
constexpr uint32_t kIdescE4m3 = kIdescBase;

// The four MMAs of one 128-byte K block (K = 16 bf16 or 32 E4M3 values each, 32 bytes apart).
template <bool kFp8>
__device__ __forceinline__ void issue_router_k_block(uint32_t tmem_acc, uint32_t a_lo, uint32_t b_lo,
                                                     uint32_t accumulate) {
  constexpr uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8 rows x 128 B groups, 128B swizzle
#define GV_RP_MMA(kind, j, pred)                                     \
  "add.u32 lo, %1, " #j "*2;\n\t"                                    \
  "mov.b64 d0, {lo, %3};\n\t"                                        \
  "add.u32 lo, %2, " #j "*2;\n\t"                                    \
  "mov.b64 d1, {lo, %3};\n\t"                                        \
  "tcgen05.mma.cta_group::1.kind::" kind " [%0], d0, d1, %4, " pred ";\n\t"
#define GV_RP_BLOCK(kind)                                                                            \
  asm volatile("{\n\t.reg .pred p, pt;\n\t.reg .b32 lo;\n\t.reg .b64 d0, d1;\n\t"                     \
               "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"                                   \
               GV_RP_MMA(kind, 0, "p") GV_RP_MMA(kind, 1, "pt") GV_RP_MMA(kind, 2, "pt")              \
               GV_RP_MMA(kind, 3, "pt") "}"                                                           \
               ::"r"(tmem_acc), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(kFp8 ? kIdescE4m3 : kIdescBf16),    \
                 "r"(accumulate)                                                                      \
               : "memory")
  if constexpr (kFp8) {
    GV_RP_BLOCK("f8f6f4");
  } else {
    GV_RP_BLOCK("f16");
  }
#undef GV_RP_BLOCK
#undef GV_RP_MMA
}

template <bool kFp8, int kSplit>
__global__ void __launch_bounds__(kRpThreads, 1)
route_project_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const RouterParams p) {
  extern __shared__ uint8_t smem_raw[];
  RouterSmem* smem = reinterpret_cast<RouterSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  constexpr int kOwnRows = kTileM / kSplit;   // tile rows this CTA reduces and routes
  const int m_tile = static_cast<int>(blockIdx.x) / kSplit;
  const int kb_begin = static_cast<int>(rank) * p.k_blocks / kSplit;
  const int kb_end = (static_cast<int>(rank) + 1) * p.k_blocks / kSplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRpStages; ++s) {
      mbar_init(&smem->full[s], 1);
      mbar_init(&smem->empty[s], 1);
    }
    mbar_init(&smem->acc_full, 1);
    smem->abort = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_x);
    prefetch_tensor_map(&map_w);
  }
  if (warp == 1) {
    tmem_alloc(&smem->tmem_base, kExperts);
    tmem_relinquish();
  }
  // The next kernel of the stream (launched with programmatic serialization) may take its place on
  // the SMs now; it waits at its own top for this grid to complete.
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = smem->tmem_base;
  grid_dependency_wait();  // the previous kernel of the stream has completed and its writes are visible

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      ok = __all_sync(0xffffffffu, wait_or_abort<true>(&smem->empty[stage], phase ^ 1u, smem, p.status));
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&smem->full[stage], 2u * kRpTileBytes);
        tma_load_2d(smem->a[stage], &map_x, &smem->full[stage], kb * kTileKBytes, m_tile * kTileM);
        tma_load_2d(smem->b[stage], &map_w, &smem->full[stage], kb * kTileKBytes, 0);
      }
      __syncwarp();
      ++issued;
      if (++stage == kRpStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (!ok && lane == 0) {
      // let the copies already issued land before shared memory is given up
      const int pending = issued < kRpStages ? issued : kRpStages;
      int s = stage;
      uint32_t ph = phase;
      for (int i = 0; i < pending; ++i) {
        if (--s < 0) {
          s = kRpStages - 1;
          ph ^= 1u;
        }
        mbar_wait_bounded(&smem->full[s], ph, 40000000ll);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t a_lo0 = (smem_u32(smem->a[0]) & 0x3ffffu) >> 4;
    const uint32_t b_lo0 = (smem_u32(smem->b[0]) & 0x3ffffu) >> 4;
    const bool leader = elect_one();
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      if (!wait_or_abort<false>(&smem->full[stage], phase, smem, p.status)) break;
      if (leader) {
        issue_router_k_block<kFp8>(tmem_base, a_lo0 + static_cast<uint32_t>(stage) * (kRpTileBytes >> 4),
                                   b_lo0 + static_cast<uint32_t>(stage) * (kRpTileBytes >> 4),
                                   kb != kb_begin ? 1u : 0u);
        tc_commit(&smem->empty[stage]);
        if (kb + 1 == kb_end) tc_commit(&smem->acc_full);
      }
      if (++stage == kRpStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue, part 1: partial sums to the rows' owners ----------------
    const int quarter = warp & 3;  // the tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    const int owner = row % kSplit;
    const int owner_row = row / kSplit;
    // rows past the end of the batch (most rows of a decode-sized batch) are not sent; the
    // tensor-memory loads are warp-wide, so a warp takes part if any of its 32 rows exists
    const bool row_exists = m_tile * kTileM + row < p.tokens;
    const bool warp_has_rows = m_tile * kTileM + quarter * 32 < p.tokens;
    if (wait_or_abort<true>(&smem->acc_full, 0, smem, p.status) && warp_has_rows) {
      tc_fence_after_sync();
      const uint32_t remote_row =
          cluster_map_shared(smem_u32(smem->received + (rank * kOwnRows + owner_row) * kExperts),
                             static_cast<uint32_t>(owner));
#pragma unroll 1
      for (int part = 0; part < 4; ++part) {
        uint32_t r[32];
        tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + part * 32, r);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int chunk = part * 8 + i;
          if (row_exists)
            cluster_store_uint4(remote_row + (static_cast<uint32_t>(received_chunk_position(chunk, owner_row)) << 4),
                              make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]));
        }
      }
      tc_fence_before_sync();
    }
  }

  // Every thread of every CTA of the cluster arrives here, also after a failed wait.  The barrier
  // orders the posted stores above before the owners' reads below; after it no CTA touches another
  // CTA's shared memory, so a CTA may finish while its peers still work.
  cluster_sync_all();

  if (warp >= 2 && !smem->abort) {
    // ---------------- epilogue, part 2: reduce this CTA's rows and route them, 32 at a time ----------------
    const int t = threadIdx.x - 64;
    const int part = t & 3;         // columns [32 * part, 32 * part + 32)
#pragma unroll 1
    for (int pass = 0; pass < (kOwnRows + 31) / 32; ++pass) {
      if (m_tile * kTileM + pass * 32 * kSplit >= p.tokens) break;   // no row of this pass exists
      // tile row kSplit * row_local + rank; with eight owners a CTA has 16 rows and half of the
      // threads only keep their quads company (they read row 15 again and store nothing)
      const bool row_owned = pass * 32 + (t >> 2) < kOwnRows;
      const int row_local = row_owned ? pass * 32 + (t >> 2) : kOwnRows - 1;
      const int token = m_tile * kTileM + row_local * kSplit + static_cast<int>(rank);
      const bool valid = row_owned && token < p.tokens;
      float4 acc[8];
#pragma unroll
      for (int source = 0; source < kSplit; ++source) {
        const float4* source_row =
            reinterpret_cast<const float4*>(smem->received + (source * kOwnRows + row_local) * kExperts);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 v = source_row[received_chunk_position(part * 8 + i, row_local)];
          if (source == 0) {
            acc[i] = v;
          } else {
            acc[i].x = __fadd_rn(acc[i].x, v.x);
            acc[i].y = __fadd_rn(acc[i].y, v.y);
            acc[i].z = __fadd_rn(acc[i].z, v.z);
            acc[i].w = __fadd_rn(acc[i].w, v.w);
          }
        }
      }
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v = acc[i];
        if (p.bias) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias) + part * 8 + i);
          v.x = __fadd_rn(v.x, b.x);
          v.y = __fadd_rn(v.y, b.y);
          v.z = __fadd_rn(v.z, b.z);
          v.w = __fadd_rn(v.w, b.w);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
        packed[2 * i] = *reinterpret_cast<const uint32_t*>(&lo);
        packed[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
      const size_t safe_token = valid ? static_cast<size_t>(token) : 0;
      if (p.logits_out && valid) {
        uint4* out = reinterpret_cast<uint4*>(p.logits_out + safe_token * kExperts + 32 * part);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          out[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
      // the reference's rescale of an unscaled FP8 GEMM output (routing_sampling.cuh:405-411)
      const float rescale = kFp8 ? __fmul_rn(p.activation_scales[safe_token], p.weight_scale[0]) : 1.0f;
      route_top8_quad(packed, part, kFp8, rescale, valid, p.expert_scale, p.weights + safe_token * kTopK,
                      p.ids + safe_token * kTopK);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, kExperts);
  }
}

template <bool kFp8, int kSplit>
cudaError_t launch_variant(const CUtensorMap& map_x, const CUtensorMap& map_w, const RouterParams& p,
                           cudaStream_t stream) {
  static bool prepared[64] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device >= 0 && device < 64 && !prepared[device]) {
    e = cudaFuncSetAttribute(route_project_kernel<kFp8, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kRpSmemBytes));
    if (e != cudaSuccess) return e;
    prepared[device] = true;
  }
  const int m_tiles = (p.tokens + kTileM - 1) / kTileM;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(m_tiles * kSplit));
  config.blockDim = dim3(kRpThreads);
  config.dynamicSmemBytes = kRpSmemBytes;
  config.stream = stream;
  // Clusters of kSplit CTAs; and the launch may begin while the previous kernel of the stream is
  // still running (the kernel waits at grid_dependency_wait before it reads or writes global memory),
  // so that its set-up hides behind a predecessor that lets its dependents go early.
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = kSplit;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 2;
  return cudaLaunchKernelEx(&config, route_project_kernel<kFp8, kSplit>, map_x, map_w, p);
}

template <bool kFp8>
cudaError_t launch_split(const CUtensorMap& map_x, const CUtensorMap& map_w, const RouterParams& p,
                         cudaStream_t stream) {
  const int m_tiles = (p.tokens + kTileM - 1) / kTileM;
  if (m_tiles <= 4) return launch_variant<kFp8, 8>(map_x, map_w, p, stream);
  if (m_tiles * 4 <= 160) return launch_variant<kFp8, 4>(map_x, map_w, p, stream);
  if (m_tiles * 2 <= 160) return launch_variant<kFp8, 2>(map_x, map_w, p, stream);
  return launch_variant<kFp8, 1>(map_x, map_w, p, stream);
}

}  // namespace

int launch_route_project(const void* x, const void* router_w, bool fp8, const float* bias,
                         const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                         const float* activation_scales, const float* weight_scale, int tokens, int* status,
                         cudaStream_t stream) {
  const uint64_t row_bytes = fp8 ? kHidden : 2 * kHidden;
  CUtensorMap map_x, map_w;
  if (!make_operand_tensor_map(&map_x, x, static_cast<uint64_t>(tokens), row_bytes, kTileM) ||
      !make_operand_tensor_map(&map_w, router_w, kExperts, row_bytes, kTileM))
    return static_cast<int>(cudaErrorInvalidValue);
  RouterParams p{};
  p.bias = bias;
  p.expert_scale = static_cast<const __nv_bfloat16*>(expert_scale_bf16);
  p.weights = weights;
  p.ids = ids;
  p.logits_out = static_cast<__nv_bfloat16*>(logits_out);
  p.activation_scales = activation_scales;
  p.weight_scale = weight_scale;
  p.status = status;
  p.tokens = tokens;
  p.k_blocks = static_cast<int>(row_bytes / kTileKBytes);
  const cudaError_t e = fp8 ? launch_split<true>(map_x, map_w, p, stream) : launch_split<false>(map_x, map_w, p, stream);
  return static_cast<int>(e);
}

}  // namespace gv
