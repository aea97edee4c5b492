// Host side of the C ABI declared in include/gevva_moe.h: owns scratch, builds
// the TMA tensor maps once, and enqueues the stages of one MoE layer in the order
// of the reference's Impl::launch (src/nvfp4_cutlass.cu:1827-1886).  No
// allocation, synchronisation or host-dependent branch on device data happens on
// the launch path, so a launch can be captured into a CUDA graph like the
// reference's (src/cuda/runtime/verifier.cuh:1058-1078).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "../../include/gevva_moe.h"
#include <nvtx3/nvToolsExt.h>

#include "gv_common.cuh"
#include "gv_launchers.h"
#include "gv_scratch.h"

namespace {

using namespace gv;

constexpr int kMaxTokens = 131072;

// The CUDA face of the allocator that gv_scratch.h takes as a parameter.
struct CudaScratchRuntime {
  static inline cudaError_t last_error = cudaSuccess;
  static bool allocate(void** pointer, size_t bytes) {
    last_error = cudaMalloc(pointer, bytes);
    return last_error == cudaSuccess;
  }
  static bool zero(void* pointer, size_t bytes) {
    last_error = cudaMemset(pointer, 0, bytes);
    return last_error == cudaSuccess;
  }
  static void release(void* pointer) noexcept { cudaFree(pointer); }
};

struct Scratch {
  int references = 1;
  int max_tokens = 0;
  int routes = 0;
  uint8_t* input_codes = nullptr;
  uint8_t* input_sf = nullptr;
  void* w13_out = nullptr;
  uint8_t* inter_codes = nullptr;
  uint8_t* inter_sf = nullptr;
  void* w2_out = nullptr;
  int* ints = nullptr;  // one allocation carved into the RoutePlan arrays
  gv::ScratchMemory<CudaScratchRuntime> memory;
  RoutePlan plan{};
  size_t input_sf_bytes = 0, inter_sf_bytes = 0, tile_capacity = 0;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Byte matrix [rows, row_bytes] viewed through a 128-row x 128-byte box with the
// 128-byte swizzle the MMA descriptors expect.  Out-of-range bytes read as zero.
bool make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                      int box_rows = kTileM) {
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
            element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_scale_map(CUtensorMap* map, const void* base, uint64_t bytes, int box_atoms) {
  const cuuint64_t dims[2] = {128, bytes / 512};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_atoms)};
  const cuuint32_t element_strides[2] = {1, 1};
  EncodeTiledFn fn = encode_tiled();
  if (!fn || dims[1] == 0) return false;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
            element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// w13 codes [experts, 2 halves (up, gate), 704 rows, 1408 bytes] through a box of both halves x
// 64 rows x 128 bytes (128-byte swizzle): one copy brings a unit's up rows and gate rows.
bool make_w13_unit_map(CUtensorMap* map, const void* base, uint64_t experts) {
  const cuuint64_t dims[3] = {kHidden / 2, kInter, experts * 2};
  const cuuint64_t strides[2] = {kHidden / 2, static_cast<cuuint64_t>(kInter) * (kHidden / 2)};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(kTileKBytes), 64, 2};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
            element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Scale bytes of an activation operand as [128-row blocks, atoms per block, 128 x u32] through a
// box of two blocks x four atoms: the scales of one K block for up to 256 rows in one copy.
bool make_block_scale_map(CUtensorMap* map, const void* base, uint64_t bytes, int atoms_per_block) {
  const uint64_t block_bytes = static_cast<uint64_t>(atoms_per_block) * 512;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(atoms_per_block), bytes / block_bytes};
  const cuuint64_t strides[2] = {512, block_bytes};
  const cuuint32_t box[3] = {128, 4, 2};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  EncodeTiledFn fn = encode_tiled();
  if (!fn || dims[2] == 0) return false;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box,
            element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

thread_local char g_error_text[256] = "";

int cuda_failure(cudaError_t error, const char* what) {
  std::snprintf(g_error_text, sizeof(g_error_text), "%s: %s", what, cudaGetErrorString(error));
  return GEVVA_MOE_CUDA_ERROR;
}

#define GV_CUDA(call, what)                                  \
  do {                                                       \
    const cudaError_t gv_error_ = (call);                    \
    if (gv_error_ != cudaSuccess) return cuda_failure(gv_error_, what); \
  } while (0)

void free_scratch(Scratch* s) {
  if (!s) return;
  s->memory.release();
  delete s;
}

int make_scratch(int tokens, Scratch** out) {
  Scratch* s = new (std::nothrow) Scratch;
  if (!s) return GEVVA_MOE_CUDA_ERROR;
  const gv::ScratchSizes sizes = gv::scratch_sizes(tokens);
  s->max_tokens = tokens;
  s->routes = static_cast<int>(sizes.routes);
  s->input_sf_bytes = sizes.bytes[1];
  s->inter_sf_bytes = sizes.bytes[4];
  s->tile_capacity = sizes.tile_capacity;
  const size_t routes = sizes.routes;
  const size_t chunks = sizes.chunks;
  if (!s->memory.acquire(sizes)) {
    delete s;
    return cuda_failure(CudaScratchRuntime::last_error, "scratch allocation");
  }
  s->input_codes = static_cast<uint8_t*>(s->memory.buffers[0]);
  s->input_sf = static_cast<uint8_t*>(s->memory.buffers[1]);
  s->w13_out = s->memory.buffers[2];
  s->inter_codes = static_cast<uint8_t*>(s->memory.buffers[3]);
  s->inter_sf = static_cast<uint8_t*>(s->memory.buffers[4]);
  s->w2_out = s->memory.buffers[5];
  s->ints = static_cast<int*>(s->memory.buffers[6]);
  int* cursor = s->ints;
  auto carve = [&](size_t count) {
    int* p = cursor;
    cursor += count;
    return p;
  };
  s->plan.sorted_experts = carve(routes);
  s->plan.sorted_routes = carve(routes);
  s->plan.inverse_routes = carve(routes);
  s->plan.expert_offsets = carve(kExperts + 1);
  s->plan.scale_row_offsets = carve(kExperts + 1);
  s->plan.tile_expert = carve(s->tile_capacity);
  s->plan.num_m_tiles = carve(1);
  s->plan.pair_tile = carve(s->tile_capacity);
  s->plan.num_pairs = carve(1);
  s->plan.tile_ready = carve(s->tile_capacity + 1);
  s->plan.chunk_hist = carve(chunks * kExperts);
  s->plan.status = carve(1);
  s->plan.sync = carve(2);  // taken from the 64 spare ints; zero like everything else here
  s->plan.front_sync = carve(2);  // likewise
  *out = s;
  return GEVVA_MOE_OK;
}

}  // namespace

namespace gv {
bool make_operand_tensor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                             int box_rows) {
  return make_operand_map(map, base, rows, row_bytes, box_rows);
}
bool make_scale_tensor_map(CUtensorMap* map, const void* base, uint64_t bytes, int box_atoms) {
  return make_scale_map(map, base, bytes, box_atoms);
}
}  // namespace gv

namespace {
// The bounded-wait primitive of the GEMM kernels, exercised on its own: one thread waits on
// a local mbarrier that nothing will ever complete, gives up after `limit_cycles`, records
// kWaitTimeout in the status word and returns normally.
__global__ void bounded_wait_probe_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t barrier;
  if (threadIdx.x == 0) {
    gv::mbar_init(&barrier, 1);
    gv::fence_barrier_init();
    if (!gv::mbar_wait_bounded(&barrier, 0, limit_cycles))
      atomicExch(status, static_cast<int>(gv::kWaitTimeout));
  }
}
}  // namespace

struct gevva_moe {
  Scratch* scratch = nullptr;
  gevva_moe_weights weights{};
  gv::GemmOperands w13{};        // bf16 output (stage access, debugging)
  gv::GemmOperands w13_fused{};  // GeGLU + requantise in the epilogue (the production path)
  gv::GemmOperands w2{};
  uint8_t* w13_sf_tiled = nullptr;  // runner-owned re-tiling of weights.w13_sf
  gv::W13PairOperands w13_pairs{};  // the CTA-pair form of the fused w13 stage
  uint8_t* w13_sf_units = nullptr;  // runner-owned re-tiling of weights.w13_sf for it
  bool w13_pair_form = false;       // GEVVA_MOE_OPTION_W13_PAIRS, or GEVVA_MOE_W13_PAIRS=1 for a whole process
  int sm_count = 0;
  bool pairs = false;               // GEVVA_MOE_OPTION_PAIRS: prefill-sized launches run the expert GEMMs as CTA pairs
  bool decode_front = true;         // ... and the route sort and the input quantiser in the same launch (GEVVA_MOE_DECODE_FRONT=0: a launch of their own)
  bool merged_decode = true;        // batches of at most 128 tokens: w13 and w2 in one launch (GEVVA_MOE_DECODE_MERGED=0: two)
  bool nvtx = false;                // GEVVA_MOE_OPTION_NVTX: one range per stage around its launches
};

namespace {
// A named NVTX range around the launches of one stage, when the runner was created with the
// option (the ranges cost nothing unless a tool is attached, but are off by default).
struct StageRange {
  bool on;
  StageRange(bool enabled, const char* name) : on(enabled) {
    if (on) nvtxRangePushA(name);
  }
  ~StageRange() {
    if (on) nvtxRangePop();
  }
};
}  // namespace

extern "C" {

const char* gevva_moe_strerror(int status) {
  switch (status) {
    case GEVVA_MOE_OK: return "ok";
    case GEVVA_MOE_BAD_EXPERT_ID: return "expert id outside [0,128)";
    case GEVVA_MOE_WAIT_TIMEOUT: return "bounded device wait expired";
    case GEVVA_MOE_BAD_ARGUMENT: return "bad argument";
    case GEVVA_MOE_CUDA_ERROR: return g_error_text[0] ? g_error_text : "CUDA error";
    case GEVVA_MOE_NO_DEVICE: return "no sm_100 device or driver entry point";
    case GEVVA_MOE_TOO_LARGE: return "size beyond the supported maximum";
    default: return "unknown status";
  }
}

int gevva_moe_create(gevva_moe** out, const gevva_moe_weights* weights, int max_tokens,
                     gevva_moe* share_scratch_with, const gevva_moe_options* options) {
  if (options && (options->flags & ~static_cast<uint32_t>(GEVVA_MOE_OPTION_NVTX | GEVVA_MOE_OPTION_PAIRS | GEVVA_MOE_OPTION_W13_PAIRS)))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (!out || !weights || !weights->w13 || !weights->w13_sf || !weights->w2 || !weights->w2_sf ||
      !weights->alpha1 || !weights->alpha2 || !weights->in_scale_q1 || !weights->in_scale_q2)
    return GEVVA_MOE_BAD_ARGUMENT;
  if (max_tokens < 1) return GEVVA_MOE_BAD_ARGUMENT;
  if (max_tokens > kMaxTokens) return GEVVA_MOE_TOO_LARGE;
  if (share_scratch_with && share_scratch_with->scratch->max_tokens != max_tokens)
    return GEVVA_MOE_BAD_ARGUMENT;  // "shared expert capacity mismatch", src/nvfp4_cutlass.cu:1788
  int device = 0;
  GV_CUDA(cudaGetDevice(&device), "cudaGetDevice");
  cudaDeviceProp prop;
  GV_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
  if (prop.major != 10 || !encode_tiled()) return GEVVA_MOE_NO_DEVICE;
  GV_CUDA(static_cast<cudaError_t>(gv::prepare_grouped_gemm()), "cudaFuncSetAttribute");

  gevva_moe* m = new (std::nothrow) gevva_moe;
  if (!m) return GEVVA_MOE_CUDA_ERROR;
  m->weights = *weights;
  m->nvtx = options && (options->flags & GEVVA_MOE_OPTION_NVTX);
  // The CTA-pair form (tcgen05 cta_group::2) is bit-identical but measured slower than one CTA per
  // tile on this part (175 against 102 us for w13 at 4096 tokens), so it is opt-in: by option, or
  // for a whole process by GEVVA_MOE_PAIRS=1.
  const char* merged_env = std::getenv("GEVVA_MOE_DECODE_MERGED");
  m->merged_decode = !(merged_env && merged_env[0] == '0');
  const char* front_env = getenv("GEVVA_MOE_DECODE_FRONT");
  m->decode_front = !(front_env && front_env[0] == '0');
  const char* pairs_env = std::getenv("GEVVA_MOE_PAIRS");
  m->pairs = (options && (options->flags & GEVVA_MOE_OPTION_PAIRS)) || (pairs_env && pairs_env[0] == '1');
  m->sm_count = prop.multiProcessorCount;
  if (share_scratch_with) {
    m->scratch = share_scratch_with->scratch;
    ++m->scratch->references;
  } else {
    const int status = make_scratch(max_tokens, &m->scratch);
    if (status != GEVVA_MOE_OK) {
      delete m;
      return status;
    }
  }
  Scratch* s = m->scratch;
  const uint64_t rows = static_cast<uint64_t>(s->routes);
  bool ok = true;
  ok = ok && make_operand_map(&m->w13.map_a, s->input_codes, rows, kHidden / 2);
  ok = ok && make_operand_map(&m->w13.map_a32, s->input_codes, rows, kHidden / 2, 32);
  ok = ok && make_operand_map(&m->w2.map_a32, s->inter_codes, rows, kInter / 2, 32);
  ok = ok && make_operand_map(&m->w13.map_b, weights->w13, static_cast<uint64_t>(kExperts) * kW13Out,
                              kHidden / 2);
  ok = ok && make_operand_map(&m->w2.map_a, s->inter_codes, rows, kInter / 2);
  ok = ok && make_operand_map(&m->w2.map_b, weights->w2, static_cast<uint64_t>(kExperts) * kHidden,
                              kInter / 2);
  ok = ok && make_operand_map(&m->w13.map_b64, weights->w13, static_cast<uint64_t>(kExperts) * kW13Out,
                              kHidden / 2, 64);
  if (!ok) {
    gevva_moe_destroy(m);
    std::snprintf(g_error_text, sizeof(g_error_text), "cuTensorMapEncodeTiled failed");
    return GEVVA_MOE_CUDA_ERROR;
  }
  // The fused w13 epilogue pairs up rows with gate rows inside one MMA tile; its weight
  // scales are a one-off re-tiling of the caller's tensor (the caller's memory is not touched).
  cudaError_t tiled_error =
      cudaMalloc(reinterpret_cast<void**>(&m->w13_sf_tiled), gv::retiled_w13_scale_bytes(kExperts));
  if (tiled_error == cudaSuccess) {
    gv::launch_retile_w13_scales(static_cast<const uint8_t*>(weights->w13_sf), m->w13_sf_tiled, kExperts,
                                 nullptr);
    tiled_error = cudaGetLastError();
  }
  if (tiled_error == cudaSuccess) tiled_error = cudaStreamSynchronize(nullptr);
  if (tiled_error != cudaSuccess) {
    gevva_moe_destroy(m);
    return cuda_failure(tiled_error, "w13 scale re-tiling");
  }
  ok = make_scale_map(&m->w13.map_a_sf, s->input_sf, s->input_sf_bytes, 4) &&
       make_scale_map(&m->w13.map_b_sf, m->w13_sf_tiled, gv::retiled_w13_scale_bytes(kExperts), 8) &&
       make_scale_map(&m->w2.map_a_sf, s->inter_sf, s->inter_sf_bytes, 4) &&
       make_scale_map(&m->w2.map_b_sf, weights->w2_sf, static_cast<uint64_t>(kExperts) * kHidden * (kInter / 16), 4);
  if (!ok) {
    gevva_moe_destroy(m);
    std::snprintf(g_error_text, sizeof(g_error_text), "cuTensorMapEncodeTiled failed (scale maps)");
    return GEVVA_MOE_CUDA_ERROR;
  }
  const char* w13_pairs_env = std::getenv("GEVVA_MOE_W13_PAIRS");
  m->w13_pair_form = (options && (options->flags & GEVVA_MOE_OPTION_W13_PAIRS)) || (w13_pairs_env && w13_pairs_env[0] == '1');
  if (m->w13_pair_form) {
    // opt-in (measured slower than the one-CTA kernel on this part): its 35 MB re-tiled scale copy
    // and its tensor maps exist only when asked for
    cudaError_t e = static_cast<cudaError_t>(gv::prepare_w13_pairs());
    if (e == cudaSuccess)
      e = cudaMalloc(reinterpret_cast<void**>(&m->w13_sf_units), gv::w13_unit_scale_bytes(kExperts));
    if (e == cudaSuccess) {
      gv::launch_retile_w13_unit_scales(static_cast<const uint8_t*>(weights->w13_sf), m->w13_sf_units, kExperts,
                                        nullptr);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
    if (e != cudaSuccess) {
      gevva_moe_destroy(m);
      return cuda_failure(e, "w13 unit scale re-tiling");
    }
    gv::W13PairOperands& wp = m->w13_pairs;
    ok = true;
    for (int i = 0; i < 16; ++i)
      ok = ok && make_operand_map(&wp.map_x[i], s->input_codes, rows, kHidden / 2, 8 * (i + 1));
    ok = ok && make_w13_unit_map(&wp.map_w, weights->w13, kExperts) &&
         make_block_scale_map(&wp.map_x_sf, s->input_sf, s->input_sf_bytes, kHidden / 64) &&
         make_scale_map(&wp.map_w_sf, m->w13_sf_units, gv::w13_unit_scale_bytes(kExperts), 4);
    if (!ok) {
      gevva_moe_destroy(m);
      std::snprintf(g_error_text, sizeof(g_error_text), "cuTensorMapEncodeTiled failed (w13 pair maps)");
      return GEVVA_MOE_CUDA_ERROR;
    }
    wp.alpha = weights->alpha1;
    wp.next_codes = s->inter_codes;
    wp.next_scales = s->inter_sf;
    wp.next_scale_q = weights->in_scale_q2;
    wp.serial_launch = false;
  }
  m->w13.a_scales = s->input_sf;
  m->w13.b_scales = static_cast<const uint8_t*>(weights->w13_sf);
  m->w13.alpha = weights->alpha1;
  m->w13.out = s->w13_out;
  m->w13.n_out = kW13Out;
  m->w13.k_in = kHidden;
  m->w13_fused = m->w13;
  m->w13_fused.b_scales = m->w13_sf_tiled;
  m->w13_fused.out = nullptr;
  m->w13_fused.fused_geglu = true;
  m->w13_fused.next_codes = s->inter_codes;
  m->w13_fused.next_scales = s->inter_sf;
  m->w13_fused.next_scale_q = weights->in_scale_q2;
  m->w2.a_scales = s->inter_sf;
  m->w2.b_scales = static_cast<const uint8_t*>(weights->w2_sf);
  m->w2.alpha = weights->alpha2;
  m->w2.out = s->w2_out;
  m->w2.n_out = kHidden;
  m->w2.k_in = kInter;
  *out = m;
  return GEVVA_MOE_OK;
}

void gevva_moe_destroy(gevva_moe* runner) {
  if (!runner) return;
  if (runner->scratch && --runner->scratch->references == 0) free_scratch(runner->scratch);
  cudaFree(runner->w13_sf_tiled);
  cudaFree(runner->w13_sf_units);
  delete runner;
}

int gevva_moe_route(const void* logits_bf16, int ld, const void* expert_scale_bf16, float* weights,
                    int* ids, int tokens, const float* act_scales, const float* w_scale,
                    gevva_stream_t stream) {
  if (!logits_bf16 || !expert_scale_bf16 || !weights || !ids || ld < kExperts || tokens < 0 ||
      (act_scales != nullptr) != (w_scale != nullptr))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (tokens == 0) return GEVVA_MOE_OK;
  gv::launch_route(logits_bf16, ld, expert_scale_bf16, weights, ids, tokens, act_scales, w_scale,
                   stream);
  GV_CUDA(cudaGetLastError(), "route_128_top8");
  return GEVVA_MOE_OK;
}

int gevva_moe_route_project(const void* router_input_bf16, const void* router_weight_bf16, const float* bias,
                            const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                            int tokens, int* device_status, gevva_stream_t stream) {
  if (!router_input_bf16 || !router_weight_bf16 || !expert_scale_bf16 || !weights || !ids || tokens < 0 ||
      (reinterpret_cast<uintptr_t>(router_input_bf16) & 15) || (reinterpret_cast<uintptr_t>(router_weight_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(bias) & 15))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (tokens == 0) return GEVVA_MOE_OK;
  if (!encode_tiled()) return GEVVA_MOE_NO_DEVICE;
  GV_CUDA(static_cast<cudaError_t>(gv::launch_route_project(router_input_bf16, router_weight_bf16, false, bias,
                                                            expert_scale_bf16, weights, ids, logits_out, nullptr,
                                                            nullptr, tokens, device_status, stream)),
          "route_project");
  return GEVVA_MOE_OK;
}

int gevva_moe_route_project_fp8(const void* router_input_e4m3, const float* activation_scales,
                                const void* router_weight_e4m3, const float* weight_scale,
                                const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                                int tokens, int* device_status, gevva_stream_t stream) {
  if (!router_input_e4m3 || !activation_scales || !router_weight_e4m3 || !weight_scale || !expert_scale_bf16 ||
      !weights || !ids || tokens < 0 || (reinterpret_cast<uintptr_t>(router_input_e4m3) & 15) ||
      (reinterpret_cast<uintptr_t>(router_weight_e4m3) & 15))
    return GEVVA_MOE_BAD_ARGUMENT;
  if (tokens == 0) return GEVVA_MOE_OK;
  if (!encode_tiled()) return GEVVA_MOE_NO_DEVICE;
  GV_CUDA(static_cast<cudaError_t>(gv::launch_route_project(router_input_e4m3, router_weight_e4m3, true, nullptr,
                                                            expert_scale_bf16, weights, ids, logits_out,
                                                            activation_scales, weight_scale, tokens, device_status,
                                                            stream)),
          "route_project_fp8");
  return GEVVA_MOE_OK;
}

int* gevva_moe_status_word(gevva_moe* runner) { return runner ? runner->scratch->plan.status : nullptr; }

int gevva_moe_launch_stages(gevva_moe* runner, const void* in, const int* ids,
                            const float* route_weights, void* out, int tokens, unsigned stages,
                            gevva_stream_t stream) {
  if (!runner) return GEVVA_MOE_BAD_ARGUMENT;
  Scratch* s = runner->scratch;
  // "expert runner token count exceeds its plan", src/nvfp4_cutlass.cu:1830-1832
  if (tokens < 1 || tokens > s->max_tokens) return GEVVA_MOE_BAD_ARGUMENT;
  if ((stages & (GEVVA_MOE_STAGE_SORT | GEVVA_MOE_STAGE_QUANTIZE)) && !ids) return GEVVA_MOE_BAD_ARGUMENT;
  if ((stages & GEVVA_MOE_STAGE_QUANTIZE) && !in) return GEVVA_MOE_BAD_ARGUMENT;
  if ((stages & GEVVA_MOE_STAGE_REDUCE) && (!out || !route_weights)) return GEVVA_MOE_BAD_ARGUMENT;
  const int routes = tokens * kTopK;
  // Decode-sized batches (at most a few rows per expert) stream weights and gain nothing from
  // pairing two row tiles of an expert; they keep the one-CTA-per-tile kernel.
  const bool use_pairs = runner->pairs && tokens > gv::kFusedSortQuantizeMaxTokens;
  const unsigned front = GEVVA_MOE_STAGE_SORT | GEVVA_MOE_STAGE_QUANTIZE;
  const unsigned layer_body = front | GEVVA_MOE_STAGE_W13 | GEVVA_MOE_STAGE_GEGLU | GEVVA_MOE_STAGE_W2;
  if ((stages & layer_body) == layer_body && !(stages & GEVVA_MOE_STAGE_UNFUSED) && runner->merged_decode &&
      runner->decode_front && tokens <= gv::kFusedSortQuantizeMaxTokens && tokens <= runner->sm_count) {
    // decode-sized batch: sort, quantiser and both GEMMs in one persistent launch; the weights start
    // streaming while the input is still being quantised
    StageRange range(runner->nvtx, "gevva_moe.sort+quantize+w13+geglu+w2");
    gv::launch_decode_layer(in, ids, runner->weights.in_scale_q1, tokens, s->input_codes, s->input_sf,
                            runner->w13_fused, runner->w2, s->plan, runner->sm_count, stream);
    stages &= ~layer_body;
  }
  if ((stages & front) == front && tokens <= gv::kFusedSortQuantizeMaxTokens) {
    // decode-sized batch: one launch does both
    StageRange range(runner->nvtx, "gevva_moe.sort+quantize");
    gv::launch_route_sort_quantize_small(in, ids, runner->weights.in_scale_q1, s->plan, tokens, s->input_codes,
                                         s->input_sf, stream);
  } else {
    if (stages & GEVVA_MOE_STAGE_SORT) {
      StageRange range(runner->nvtx, "gevva_moe.sort");
      gv::launch_route_sort(ids, routes, s->plan, stream);
    }
    StageRange range(runner->nvtx && (stages & GEVVA_MOE_STAGE_QUANTIZE), "gevva_moe.quantize");
    if (stages & GEVVA_MOE_STAGE_QUANTIZE)
      gv::launch_quantize_input(in, ids, runner->weights.in_scale_q1, s->plan, tokens, s->input_codes,
                                s->input_sf, stream);
  }
  const unsigned both = GEVVA_MOE_STAGE_W13 | GEVVA_MOE_STAGE_GEGLU;
  const unsigned gemms = both | GEVVA_MOE_STAGE_W2;
  if ((stages & gemms) == gemms && !(stages & GEVVA_MOE_STAGE_UNFUSED) && runner->merged_decode &&
      tokens <= gv::kFusedSortQuantizeMaxTokens && (stages & front) == front) {
    // decode-sized batch: both GEMMs in one persistent launch, weights streaming across the boundary
    // (the readiness counters it needs are zeroed by the fused sort + quantise launch above)
    StageRange range(runner->nvtx, "gevva_moe.w13+geglu+w2");
    gv::launch_decode_experts(runner->w13_fused, runner->w2, s->plan, runner->sm_count, stream);
    stages &= ~gemms;
  }
  if ((stages & both) == both && !(stages & GEVVA_MOE_STAGE_UNFUSED)) {
    // production path: GeGLU + requantise inside the w13 epilogue, no bf16 w13 output
    StageRange range(runner->nvtx, "gevva_moe.w13+geglu");
    if (runner->w13_pair_form && tokens > gv::kFusedSortQuantizeMaxTokens && s->plan.pair_tile &&
        runner->sm_count >= 2) {
      gv::launch_w13_pairs(runner->w13_pairs, s->plan, runner->sm_count, stream);
    } else {
      gv::GemmOperands w13 = runner->w13_fused;
      w13.use_pairs = use_pairs;
      gv::launch_grouped_gemm(w13, s->plan, runner->sm_count, stream);
    }
  } else {
    if (stages & GEVVA_MOE_STAGE_W13)
      gv::launch_grouped_gemm(runner->w13, s->plan, runner->sm_count, stream);
    if (stages & GEVVA_MOE_STAGE_GEGLU)
      gv::launch_geglu_quantize(s->w13_out, runner->weights.in_scale_q2, s->plan, routes,
                                s->inter_codes, s->inter_sf, stream);
  }
  if (stages & GEVVA_MOE_STAGE_W2) {
    StageRange range(runner->nvtx, "gevva_moe.w2");
    gv::GemmOperands w2 = runner->w2;
    w2.use_pairs = use_pairs;
    gv::launch_grouped_gemm(w2, s->plan, runner->sm_count, stream);
  }
  StageRange reduce_range(runner->nvtx && (stages & GEVVA_MOE_STAGE_REDUCE), "gevva_moe.reduce");
  if (stages & GEVVA_MOE_STAGE_REDUCE)
    gv::launch_reduce_routes(s->w2_out, route_weights, s->plan.inverse_routes, tokens, out, stream);
  GV_CUDA(cudaGetLastError(), "moe launch");
  return GEVVA_MOE_OK;
}

int gevva_moe_launch(gevva_moe* runner, const void* in, const int* ids, const float* route_weights,
                     void* out, int tokens, gevva_stream_t stream) {
  if (!in || !ids) return GEVVA_MOE_BAD_ARGUMENT;
  unsigned stages = GEVVA_MOE_STAGE_ALL;
  if (!out) stages &= ~static_cast<unsigned>(GEVVA_MOE_STAGE_REDUCE);
  return gevva_moe_launch_stages(runner, in, ids, route_weights, out, tokens, stages, stream);
}

const void* gevva_moe_routed_output(const gevva_moe* runner) {
  return runner ? runner->scratch->w2_out : nullptr;
}

const int* gevva_moe_inverse_routes(const gevva_moe* runner) {
  return runner ? runner->scratch->plan.inverse_routes : nullptr;
}

int gevva_moe_last_status(gevva_moe* runner) {
  if (!runner) return GEVVA_MOE_BAD_ARGUMENT;
  int status = 0;
  GV_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  GV_CUDA(cudaMemcpy(&status, runner->scratch->plan.status, sizeof(int), cudaMemcpyDeviceToHost),
          "status read");
  if (status != 0) GV_CUDA(cudaMemset(runner->scratch->plan.status, 0, sizeof(int)), "status clear");
  return -status;
}

int gevva_moe_probe_bounded_wait(gevva_moe* runner, long long limit_cycles, gevva_stream_t stream) {
  if (!runner || limit_cycles < 1 || limit_cycles > 2000000000ll) return GEVVA_MOE_BAD_ARGUMENT;
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(runner->scratch->plan.status, limit_cycles);
  GV_CUDA(cudaGetLastError(), "bounded wait probe");
  return GEVVA_MOE_OK;
}

int gevva_moe_buffer(const gevva_moe* runner, int buffer_id, void** device_ptr, size_t* bytes) {
  if (!runner || !device_ptr || !bytes) return GEVVA_MOE_BAD_ARGUMENT;
  const Scratch* s = runner->scratch;
  const size_t routes = static_cast<size_t>(s->routes);
  switch (buffer_id) {
    case GEVVA_MOE_BUF_INPUT_CODES: *device_ptr = s->input_codes; *bytes = routes * (kHidden / 2); break;
    case GEVVA_MOE_BUF_INPUT_SF: *device_ptr = s->input_sf; *bytes = s->input_sf_bytes; break;
    case GEVVA_MOE_BUF_W13_OUT: *device_ptr = s->w13_out; *bytes = routes * kW13Out * 2; break;
    case GEVVA_MOE_BUF_INTER_CODES: *device_ptr = s->inter_codes; *bytes = routes * (kInter / 2); break;
    case GEVVA_MOE_BUF_INTER_SF: *device_ptr = s->inter_sf; *bytes = s->inter_sf_bytes; break;
    case GEVVA_MOE_BUF_W2_OUT: *device_ptr = s->w2_out; *bytes = routes * kHidden * 2; break;
    case GEVVA_MOE_BUF_SORTED_EXPERTS: *device_ptr = s->plan.sorted_experts; *bytes = routes * 4; break;
    case GEVVA_MOE_BUF_SORTED_ROUTES: *device_ptr = s->plan.sorted_routes; *bytes = routes * 4; break;
    case GEVVA_MOE_BUF_INVERSE_ROUTES: *device_ptr = s->plan.inverse_routes; *bytes = routes * 4; break;
    case GEVVA_MOE_BUF_EXPERT_OFFSETS: *device_ptr = s->plan.expert_offsets; *bytes = (kExperts + 1) * 4; break;
    case GEVVA_MOE_BUF_SCALE_ROW_OFFSETS: *device_ptr = s->plan.scale_row_offsets; *bytes = (kExperts + 1) * 4; break;
    case GEVVA_MOE_BUF_TILE_EXPERT: *device_ptr = s->plan.tile_expert; *bytes = s->tile_capacity * 4; break;
    case GEVVA_MOE_BUF_NUM_TILES: *device_ptr = s->plan.num_m_tiles; *bytes = 4; break;
    default: return GEVVA_MOE_BAD_ARGUMENT;
  }
  return GEVVA_MOE_OK;
}

int gevva_moe_pack_experts(const float* weights, int experts, int n_out, int k_in, void* codes,
                           void* scales, float* global_scales, gevva_stream_t stream) {
  if (!weights || !codes || !scales || !global_scales || experts < 1 || n_out < 128 ||
      n_out % 128 != 0 || k_in < 64 || k_in % 64 != 0)
    return GEVVA_MOE_BAD_ARGUMENT;
  gv::launch_pack_weights(weights, experts, n_out, k_in, static_cast<uint8_t*>(codes),
                          static_cast<uint8_t*>(scales), global_scales, stream);
  GV_CUDA(cudaGetLastError(), "pack experts");
  return GEVVA_MOE_OK;
}

}  // extern "C"
