/* C ABI of the B200 (sm_100a) Gemma-4 26B-A4B NVFP4 mixture-of-experts path.
 *
 * The reference exposes this path as a C++ pimpl class that throws
 * (gevva::Nvfp4ExpertRunner, include/gevva/gpu.hpp:217-247, implementation
 * src/nvfp4_cutlass.cu:1680-1938) plus one router kernel launched inline
 * (route_128_top8_kernel, src/cuda/kernels/routing_sampling.cuh:396-431).  This
 * header is the plain-C boundary underneath a header-only C++ class of the same
 * name and methods (include/gevva/nvfp4_expert_runner.hpp), so the reference's
 * call sites (src/cuda/runtime/prefill.cuh:463-476, :1232-1245,
 * src/cuda/runtime/verifier.cuh:1020-1034, src/decisions.cpp:139-143) compile
 * against it unchanged.
 *
 * Conventions: every pointer is a DEVICE pointer unless it is an out-parameter
 * of the call itself; every launch only enqueues work on `stream`; functions
 * return 0 or a negative gevva_moe_status and never throw.  A runner is used
 * from one host thread; runners that share scratch must be launched on one
 * stream (include/gevva/gpu.hpp:222).
 */
#ifndef GEVVA_MOE_H_
#define GEVVA_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gevva_moe gevva_moe;          /* opaque runner */
typedef struct CUstream_st* gevva_stream_t;  /* == cudaStream_t */

enum gevva_moe_status {
  GEVVA_MOE_OK = 0,
  GEVVA_MOE_BAD_EXPERT_ID = -1, /* device: an id outside [0,128) reached the route sort */
  GEVVA_MOE_WAIT_TIMEOUT = -2,  /* device: a bounded wait inside a GEMM kernel expired */
  GEVVA_MOE_BAD_ARGUMENT = -3,
  GEVVA_MOE_CUDA_ERROR = -4,
  GEVVA_MOE_NO_DEVICE = -5,     /* no sm_100 device / driver entry point missing */
  GEVVA_MOE_TOO_LARGE = -6
};

/* The eight sidecar tensors of one layer that the reference's constructor resolves
 * by name (src/nvfp4_cutlass.cu:1792-1802; shapes src/runtime.cpp:233-252):
 *   w13     u8  [128,1408,1408]  E2M1 pairs, rows 0..703 = up, 704..1407 = gate
 *   w13_sf  u8  [128,1408,176]   E4M3 block scales, 128x4 interleave per expert
 *   w2      u8  [128,2816,352]
 *   w2_sf   u8  [128,2816,44]
 *   alpha1, alpha2            f32 [128]   g1.alpha, g2.alpha
 *   in_scale_q1, in_scale_q2  f32 [128]   g1/g2.input_scale_quant
 * They must stay valid for the life of the runner (pointers are cached). */
typedef struct {
  const void* w13;
  const void* w13_sf;
  const void* w2;
  const void* w2_sf;
  const float* alpha1;
  const float* alpha2;
  const float* in_scale_q1;
  const float* in_scale_q2;
} gevva_moe_weights;

/* flags of gevva_moe_options */
#define GEVVA_MOE_OPTION_NVTX 1u /* one NVTX range per stage around its launches (the reference wraps its
                                    phases in NVTX ranges too, e.g. src/gpu/weight_arena.cpp:53,
                                    src/cuda/diagnostics/assistant_prefill_layers.cuh:67-77) */
#define GEVVA_MOE_OPTION_PAIRS 2u /* batches of more than 128 tokens run the two expert GEMMs as CTA pairs
                                     (tcgen05 cta_group::2, two row tiles of an expert against shared weight
                                     rows); same bits, measured slower than the default on B200 */
#define GEVVA_MOE_OPTION_W13_PAIRS 4u /* batches of more than 128 tokens run the fused w13 stage as CTA pairs with the
                                         weight rows on the MMA's M side and up to 256 rows of an expert (any
                                         multiple of 16) on its N side; same bits, measured slower than the default
                                         on B200; holds a second re-tiled copy of the w13 scales (35 MB) */
typedef struct {
  uint32_t flags; /* 0 or GEVVA_MOE_OPTION_* */
  uint32_t reserved[7];
} gevva_moe_options;

/* Replaces Nvfp4ExpertRunner::Nvfp4ExpertRunner (src/nvfp4_cutlass.cu:1888-1891,
 * Impl ctor :1764-1825, ExpertScratch :1680-1736).  Allocates scratch for
 * `max_tokens` tokens, or shares the scratch of `share_scratch_with` (which must
 * have the same capacity).  1 <= max_tokens <= 131072 (the reference stops at 4608). */
int gevva_moe_create(gevva_moe** out, const gevva_moe_weights* weights, int max_tokens,
                     gevva_moe* share_scratch_with, const gevva_moe_options* options);

void gevva_moe_destroy(gevva_moe* runner);

/* Replaces route_128_top8_kernel<<<rows,128>>> (src/cuda/kernels/routing_sampling.cuh:396-431;
 * launched at src/cuda/runtime/prefill.cuh:420-422, :1208-1210, verifier.cuh:974-976).
 * logits bf16 [tokens, ld] (ld >= 128, elements), expert_scale bf16 [128],
 * weights f32 [tokens,8], ids i32 [tokens,8]; act_scales/w_scale optional (both or none). */
int gevva_moe_route(const void* logits_bf16, int ld, const void* expert_scale_bf16, float* weights,
                    int* ids, int tokens, const float* act_scales, const float* w_scale,
                    gevva_stream_t stream);

/* Replaces the pair "router projection GEMM, then route_128_top8_kernel"
 * (src/cuda/runtime/prefill.cuh:414-422, :1203-1210: cublasGemmEx bf16 with fp32 compute, output
 * bf16 [tokens,128], src/cuda/runtime/prefill.cuh:196-200) by one kernel; the logits stay on chip.
 *   router_input bf16 [tokens,2816], router_weight bf16 [128,2816] (both 16-byte aligned),
 *   bias optional f32 [128] (added in fp32 before the bf16 rounding; the reference has none, the
 *   benchmark's skewed-load configurations use it), expert_scale bf16 [128],
 *   weights f32 [tokens,8], ids i32 [tokens,8], logits_out optional bf16 [tokens,128].
 * logit = bf16(sum_k x*w + bias) with fp32 accumulation over four K slices summed in a fixed order,
 * so results are repeatable; against an fp32 dot product in another order a logit may differ by
 * one bf16 ulp, as between any two GEMM implementations.  device_status: optional device status
 * word (e.g. gevva_moe_status_word) that receives GEVVA_MOE_WAIT_TIMEOUT if a bounded wait expires. */
int gevva_moe_route_project(const void* router_input_bf16, const void* router_weight_bf16, const float* bias,
                            const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                            int tokens, int* device_status, gevva_stream_t stream);

/* The same for the FP8 sidecar's router (Fp8LinearRunner::launch_unscaled with unit scales, then the
 * router kernel's rescale: src/cuda/runtime/fp8_linear.cuh:215-473, routing_sampling.cuh:405-411):
 * router_input e4m3 [tokens,2816] with activation_scales f32 [tokens], router_weight e4m3 [128,2816]
 * with weight_scale f32 [1]; logits_out receives the UNSCALED bf16 logits. */
int gevva_moe_route_project_fp8(const void* router_input_e4m3, const float* activation_scales,
                                const void* router_weight_e4m3, const float* weight_scale,
                                const void* expert_scale_bf16, float* weights, int* ids, void* logits_out,
                                int tokens, int* device_status, gevva_stream_t stream);

/* Device pointer of the runner's status word, for kernels launched outside the runner that should
 * report into it (read and cleared by gevva_moe_last_status). */
int* gevva_moe_status_word(gevva_moe* runner);

/* Replaces Nvfp4ExpertRunner::launch / launch_batch / launch_batch_unreduced
 * (src/nvfp4_cutlass.cu:1893-1913 -> Impl::launch :1827-1886).
 * in bf16 [tokens,2816]; ids i32 [tokens,8]; route_weights f32 [tokens,8];
 * out bf16 [tokens,2816].  out == NULL (then route_weights may be NULL) selects the
 * unreduced form: results stay in gevva_moe_routed_output(). */
int gevva_moe_launch(gevva_moe* runner, const void* in, const int* ids, const float* route_weights,
                     void* out, int tokens, gevva_stream_t stream);

/* Replaces Nvfp4ExpertRunner::routed_output (src/nvfp4_cutlass.cu:1915-1917):
 * bf16 [8*tokens,2816] in sorted-route order, valid until the next launch. */
const void* gevva_moe_routed_output(const gevva_moe* runner);

/* Replaces Nvfp4ExpertRunner::inverse_routes (src/nvfp4_cutlass.cu:1919-1921):
 * i32 [8*tokens], original route 8*t+k -> sorted row. */
const int* gevva_moe_inverse_routes(const gevva_moe* runner);

/* Reads and clears the device status word (synchronises the device).  The
 * reference has no counterpart: its kernels cannot report and its host code throws. */
int gevva_moe_last_status(gevva_moe* runner);

const char* gevva_moe_strerror(int status);

/* Failure-detection self-check (no reference counterpart): enqueues one thread that waits,
 * with the same bounded wait the GEMM kernels use, on a local barrier nothing completes; after
 * `limit_cycles` SM cycles (<= 2e9) it gives up, the status word becomes
 * GEVVA_MOE_WAIT_TIMEOUT and the kernel ends normally, leaving the context usable. */
int gevva_moe_probe_bounded_wait(gevva_moe* runner, long long limit_cycles, gevva_stream_t stream);

/* ---- stage access, for parity tests and debugging ---------------------------
 * The reference materialises every intermediate in ExpertScratch
 * (src/nvfp4_cutlass.cu:1680-1700); these two calls expose the same buffers and
 * let a test run a sub-range of Impl::launch's stages between edits. */
enum gevva_moe_stage {
  GEVVA_MOE_STAGE_SORT = 1,      /* :1851-1867 */
  GEVVA_MOE_STAGE_QUANTIZE = 2,  /* :1869-1873 */
  GEVVA_MOE_STAGE_W13 = 4,       /* :1874 */
  GEVVA_MOE_STAGE_GEGLU = 8,     /* :1875-1879 */
  GEVVA_MOE_STAGE_W2 = 16,       /* :1880 */
  GEVVA_MOE_STAGE_REDUCE = 32,   /* :1881-1885 */
  GEVVA_MOE_STAGE_ALL = 63,
  /* When W13 and GEGLU are both requested they run as one kernel (GeGLU and requantise in
   * the GEMM epilogue; the bf16 w13 output is then not materialised).  Adding this flag
   * keeps them separate, as the reference runs them. */
  GEVVA_MOE_STAGE_UNFUSED = 64
};

int gevva_moe_launch_stages(gevva_moe* runner, const void* in, const int* ids,
                            const float* route_weights, void* out, int tokens, unsigned stages,
                            gevva_stream_t stream);

enum gevva_moe_buffer_id {
  GEVVA_MOE_BUF_INPUT_CODES = 0,   /* u8 [R,1408] */
  GEVVA_MOE_BUF_INPUT_SF = 1,      /* u8 (R+128*127)*176 */
  GEVVA_MOE_BUF_W13_OUT = 2,       /* bf16 [R,1408]; written only by the unfused W13 stage */
  GEVVA_MOE_BUF_INTER_CODES = 3,   /* u8 [R,352] */
  GEVVA_MOE_BUF_INTER_SF = 4,      /* u8 (R+128*127)*44 */
  GEVVA_MOE_BUF_W2_OUT = 5,        /* bf16 [R,2816] */
  GEVVA_MOE_BUF_SORTED_EXPERTS = 6,
  GEVVA_MOE_BUF_SORTED_ROUTES = 7,
  GEVVA_MOE_BUF_INVERSE_ROUTES = 8,
  GEVVA_MOE_BUF_EXPERT_OFFSETS = 9,     /* i32 [129] */
  GEVVA_MOE_BUF_SCALE_ROW_OFFSETS = 10, /* i32 [129] */
  GEVVA_MOE_BUF_TILE_EXPERT = 11,
  GEVVA_MOE_BUF_NUM_TILES = 12
};

int gevva_moe_buffer(const gevva_moe* runner, int buffer_id, void** device_ptr, size_t* bytes);

/* Route sort for callers that cannot allocate device memory on this path: a server
 * whose arena took all device memory at start-up, a serving loop that may not stall on
 * cudaMalloc's device-wide synchronisation, a plug-in bound to its host's allocator.  It has
 * no counterpart in the reference, whose sort always works in ExpertScratch.  Same
 * results as the sort stage of gevva_moe_launch, but the working memory is a fixed
 * array inside the library (about 69 KiB per GPU, held until exit) instead of a
 * runner's scratch, and the caller supplies every output:
 *   sorted_experts, sorted_routes, inverse_routes  i32 [8*tokens]
 *   expert_offsets, scale_row_offsets               i32 [129]
 *   status   i32 [1], zeroed by the caller; set to 1 if an id is outside [0,128)
 * Limits: 1 <= tokens <= 16384, else GEVVA_MOE_TOO_LARGE.  All calls on a device share
 * the array, so calls that may overlap on the GPU race; order them on one stream.
 * The first call on each device resolves the array's address, and with lazy module
 * loading it is also the moment the driver loads the library's device code, the array
 * included, into device memory: make that call at start-up, before the host's arena
 * claims the remaining memory and before any stream capture.  After it, no call
 * allocates or calls an allocating routine. */
int gevva_moe_route_sort_noalloc(const int* expert_ids, int tokens, int* sorted_experts,
                                 int* sorted_routes, int* inverse_routes, int* expert_offsets,
                                 int* scale_row_offsets, int* status, gevva_stream_t stream);

/* ---- expert-parallel form (no counterpart in the reference, which is single-GPU) ----
 * Experts are sharded over the `world` GPUs of one node (expert e on rank e % world, local
 * index e / world); each rank routes its own tokens, stores the quantised rows straight
 * into the owning rank's operand buffers over NVLink, runs the two grouped GEMMs for its
 * experts and stores result rows back into the source rank's combine buffer.  One step is
 * four calls and one cross-rank barrier (gevva_moe_ep_barrier or any stream-ordered
 * collective):
 *   gevva_moe_ep_route_sort | gevva_moe_ep_dispatch | gevva_moe_ep_compute | barrier |
 *   gevva_moe_ep_reduce
 * The other two barriers a step needs are inside the calls (the flags and the bounded wait of
 * gevva_moe_ep_barrier): gevva_moe_ep_route_sort ends with the exchange of the per-expert route
 * counts and waits for every rank's; gevva_moe_ep_dispatch ends by announcing that this rank's
 * rows are stored and gevva_moe_ep_compute starts by waiting for every rank's announcement.
 * Every rank must make the same calls in the same order.
 * The peer-writable buffers are allocated by the caller (e.g. symmetric memory) with the
 * same sizes on every rank and passed as host arrays of `world` device pointers:
 *   peer_counts      i32 [world*128]
 *   peer_flags       i32 [world], zero-initialised
 *   peer_recv_codes  u8  [recv_capacity_rows, 1408]
 *   peer_recv_sf     u8  [recv_capacity_rows, 176]   (row-major scale bytes as received)
 *   peer_combine     bf16 [8*max_tokens, 2816]
 * recv_capacity_rows must be at least world * 8 * max_tokens (every route of every rank on one
 * owner; smaller values are refused with GEVVA_MOE_BAD_ARGUMENT because no kernel bounds a
 * receive row against the capacity).  local_weights holds
 * this rank's 128/world experts in the sidecar layout with [128/world] scale vectors;
 * in_scale_q1_global is g1.input_scale_quant of all 128 experts (the sender quantises). */
typedef struct gevva_moe_ep gevva_moe_ep;

typedef struct {
  int rank;
  int world;      /* 1, 2, 4 or 8 */
  int max_tokens; /* tokens of this rank per step */
  size_t recv_capacity_rows;
  void* const* peer_recv_codes;
  void* const* peer_recv_sf;
  void* const* peer_combine;
  int* const* peer_counts;
  int* const* peer_flags; /* i32 [world] per rank, zero-initialised: flags of gevva_moe_ep_barrier */
  /* Optional HOST array [128], the same on every rank: placement[e] = owner rank * (128/world) +
   * local index of expert e on its owner (a permutation of 0..127; local_weights then holds the
   * rank's experts in local-index order).  NULL: expert e on rank e % world at index e / world. */
  const int* placement;
} gevva_moe_ep_config;

int gevva_moe_ep_create(gevva_moe_ep** out, const gevva_moe_weights* local_weights,
                        const float* in_scale_q1_global, const gevva_moe_ep_config* config);
void gevva_moe_ep_destroy(gevva_moe_ep* ep);
/* A barrier across the ranks, enqueued on `stream`: flags in peer memory, a bounded wait
 * (expiry sets GEVVA_MOE_WAIT_TIMEOUT in the status word).  Every rank must call it the same
 * number of times.  Any other stream-ordered collective may be used instead. */
int gevva_moe_ep_barrier(gevva_moe_ep* ep, gevva_stream_t stream);
int gevva_moe_ep_route_sort(gevva_moe_ep* ep, const int* ids, int tokens, gevva_stream_t stream);
int gevva_moe_ep_dispatch(gevva_moe_ep* ep, const void* in, const int* ids, int tokens,
                          gevva_stream_t stream);
int gevva_moe_ep_compute(gevva_moe_ep* ep, gevva_stream_t stream);
int gevva_moe_ep_reduce(gevva_moe_ep* ep, const float* route_weights, void* out, int tokens,
                        gevva_stream_t stream);
/* Measurement aids: the dispatch and compute phases of the last step again with every store kept
 * on this GPU (rows go to this rank's own buffers, whose contents become meaningless).  An
 * expert-parallel step minus the same work timed this way is the step's exposed communication. */
int gevva_moe_ep_dispatch_local(gevva_moe_ep* ep, const void* in, const int* ids, int tokens,
                                gevva_stream_t stream);
int gevva_moe_ep_compute_local(gevva_moe_ep* ep, gevva_stream_t stream);
/* gevva_moe_ep_compute runs part of its work on a non-blocking side stream owned by the object
 * (forked from and joined to `stream` by events), so that one group's NVLink-bound down projection
 * overlaps the next group's up projection; a caller that captures `stream` captures it too. */
/* Synchronises; returns and clears the device status word; optionally reports how many rows
 * this rank received in the last step. */
int gevva_moe_ep_status(gevva_moe_ep* ep, int* received_rows);

/* ---- feed-forward steps around the expert path, and the dense FP8 GeGLU MLP -----------
 * (the 30-layer FFN stack).  Every tensor is bf16 unless noted; rows are 2816 wide.
 *
 * gevva_ff_prepare replaces dual_rmsnorm_router_2816_kernel
 * (src/cuda/kernels/normalization.cuh:83-123, launched at src/cuda/runtime/prefill.cuh:1200-1202):
 * one RMS statistic, three outputs (dense-MLP input, expert input, router input).
 *
 * gevva_ff_finalize replaces finalize_feedforward_routes_2816_kernel (normalization.cuh:249-377,
 * launched at prefill.cuh:1238-1245): weighted reduce of the eight routed rows (read through
 * inverse_routes from gevva_moe_routed_output), RMSNorm of the dense and expert branches, their
 * sum, a third RMSNorm, residual add and the layer scalar.  dense_activation_scales f32 [rows] and
 * dense_projection_scale f32 [1], both on the DEVICE as in the reference kernel's signature
 * (normalization.cuh:249-262), rescale an unscaled FP8 GEMM output; both NULL otherwise. */
int gevva_ff_prepare(const void* input, const void* dense_weight, const void* expert_weight,
                     const void* router_scale, void* dense_out, void* expert_out, void* router_out,
                     int rows, gevva_stream_t stream);
int gevva_ff_finalize(const void* dense, const void* dense_weight, const void* expert_routes,
                      const float* route_weights, const int* inverse_routes, const void* expert_weight,
                      const void* combined_weight, const void* residual, const void* layer_scalar,
                      void* output, int rows, const float* dense_activation_scales,
                      const float* dense_projection_scale, gevva_stream_t stream);

/* Dense GeGLU MLP of width 2112 in FP8 E4M3 with per-tensor weight scales
 * (tools/pack_fp8_dense.py:52-71) and per-row dynamic activation scales.  Replaces the
 * reference's sequence quantize_fp8_rows -> gate and up projections (cuBLASLt, unit scales)
 * -> gelu_quantize_fp8_2112 -> down projection (src/cuda/runtime/prefill.cuh:1211-1230,
 * src/cuda/kernels/fp8.cuh:2-26, :299-364).  gate_up is the gate matrix [2112,2816] followed by
 * the up matrix [2112,2816]; down is [2816,2112].  The output is the UNSCALED bf16 down
 * projection; gevva_dense_output_scales gives the per-row activation scale that, times
 * down_scale, gevva_ff_finalize applies. */
typedef struct gevva_dense gevva_dense;
typedef struct {
  const void* gate_up; /* e4m3 [4224,2816] */
  const void* down;    /* e4m3 [2816,2112] */
  float gate_scale, up_scale, down_scale;
} gevva_dense_weights;
int gevva_dense_create(gevva_dense** out, const gevva_dense_weights* weights, int max_tokens);
void gevva_dense_destroy(gevva_dense* dense);
int gevva_dense_launch(gevva_dense* dense, const void* in, void* out_unscaled, int tokens,
                       gevva_stream_t stream);
const float* gevva_dense_output_scales(const gevva_dense* dense);
/* f32 [1] on the device: weights->down_scale, in the form gevva_ff_finalize takes it */
const float* gevva_dense_projection_scale(const gevva_dense* dense);
/* stage buffers for parity tests: 0 input e4m3, 1 input scales, 2 gate|up bf16 unscaled,
 * 3 product e4m3, 4 product scales */
int gevva_dense_buffer(const gevva_dense* dense, int which, void** device_ptr, size_t* bytes);
/* Per-tensor FP8 quantiser (tools/pack_fp8_dense.py:64-70): scale = amax/448, q = e4m3(w/scale). */
int gevva_pack_fp8(const float* weights, size_t count, void* out, float* scale, gevva_stream_t stream);

/* Expert packer for synthetic or freshly quantised weights; stands where
 * tools/pack_trtllm_experts.py:51-65 stands in the reference (stack experts,
 * interleave block scales) and also performs the NVFP4 quantisation itself:
 * fp32 [experts, n_out, k_in] -> codes u8 [experts, n_out, k_in/2], scales u8
 * [experts, n_out, k_in/16] (interleaved per expert), global f32 [experts]
 * = amax/(6*448). */
int gevva_moe_pack_experts(const float* weights, int experts, int n_out, int k_in, void* codes,
                           void* scales, float* global_scales, gevva_stream_t stream);

/* Packed expert sidecar reader (host only, no CUDA call).  Replaces, for this path,
 * inspect_safetensors / MappedShard::tensor (include/gevva/safetensors.hpp:12-27, :36-53,
 * src/safetensors.cpp) and the 13-tensors-per-layer schema check of the runtime
 * (src/runtime.cpp:222-254).  The file is mapped read-only; views point into the mapping and
 * die with gevva_sidecar_close.  Validation is strict: integer shapes and offsets only, known
 * whole-byte dtypes, end-begin = numel*itemsize without overflow, tensors tile the data
 * section exactly, __metadata__ holds strings.  Failures return GEVVA_MOE_BAD_ARGUMENT and
 * leave a message for gevva_sidecar_error() (thread-local). */
typedef struct gevva_sidecar gevva_sidecar;
typedef struct {
  char dtype[16];     /* "U8", "F32", "BF16", ... */
  int rank;           /* at most 8 */
  uint64_t shape[8];
  const void* data;   /* host pointer into the mapping */
  uint64_t bytes;
} gevva_sidecar_view;
int gevva_sidecar_open(gevva_sidecar** out, const char* path);
void gevva_sidecar_close(gevva_sidecar* sidecar);
int gevva_sidecar_tensor_count(const gevva_sidecar* sidecar);
int gevva_sidecar_tensor(const gevva_sidecar* sidecar, const char* name, gevva_sidecar_view* view);
/* Names, dtypes and shapes of layers 0..layers-1 and nothing else in the file (the reference
 * checks 30 layers x 13 tensors). */
int gevva_sidecar_check_layers(const gevva_sidecar* sidecar, int layers);
/* HOST views of the eight tensors of one layer that gevva_moe_create reads; the caller copies
 * them to the device. */
int gevva_sidecar_layer_weights(const gevva_sidecar* sidecar, int layer, gevva_moe_weights* host_views);
const char* gevva_sidecar_error(void);

/* Checkpoint -> sidecar packer for one layer (host only, no CUDA call).  Replaces the per-layer
 * body of tools/pack_trtllm_experts.py:88-148: takes the checkpoint's already quantised
 * per-expert tensors (model.language_model.layers.L.experts.E.{gate,up,down}_proj.{weight,
 * weight_scale,weight_scale_2,input_scale}), stacks the experts, orders w13 rows [up; gate],
 * puts every expert's row-major E4M3 block scales into the 128-row x 4-group interleave the GEMM
 * reads (the job of flashinfer's nvfp4_block_scale_interleave there) and derives
 *   g1.alpha = gate input_scale * gate weight_scale_2,  g1.alpha_up likewise for up,
 *   g2.alpha = down input_scale * down weight_scale_2,  g*.input_scale_quant = 1 / input_scale.
 * All pointers are HOST pointers; the outputs are the thirteen tensors of the layer schema
 * (src/runtime.cpp:233-252) with the caller's sizes: hidden 2816 and intermediate 704 for
 * Gemma-4 26B-A4B.  Gate and up input scales that differ are an error, as in the script. */
typedef struct {
  const void* weight;       /* u8  [rows, k/2]   E2M1 pairs */
  const void* weight_scale; /* u8  [rows, k/16]  E4M3, row-major */
  float weight_scale_2;     /* per-tensor global scale */
  float input_scale;        /* static activation scale */
} gevva_checkpoint_projection;
typedef struct {
  gevva_checkpoint_projection gate_proj; /* rows = intermediate, k = hidden */
  gevva_checkpoint_projection up_proj;   /* rows = intermediate, k = hidden */
  gevva_checkpoint_projection down_proj; /* rows = hidden, k = intermediate */
} gevva_checkpoint_expert;
typedef struct {
  void* w13_weight;             /* u8 [E, 2*intermediate, hidden/2] */
  void* w13_weight_scale;       /* u8 [E, 2*intermediate, hidden/16], interleaved */
  void* w2_weight;              /* u8 [E, hidden, intermediate/2] */
  void* w2_weight_scale;        /* u8 [E, hidden, intermediate/16], interleaved */
  float* w13_input_scale;       /* [E] */
  float* w2_input_scale;        /* [E] */
  float* w13_weight_scale_2;    /* [E,2]: gate, up */
  float* w2_weight_scale_2;     /* [E] */
  float* g1_alpha;              /* [E] */
  float* g1_alpha_up;           /* [E] */
  float* g2_alpha;              /* [E] */
  float* g1_input_scale_quant;  /* [E] */
  float* g2_input_scale_quant;  /* [E] */
} gevva_sidecar_layer;
int gevva_moe_pack_checkpoint_layer(const gevva_checkpoint_expert* experts, int expert_count, int hidden,
                                    int intermediate, gevva_sidecar_layer* out);

#ifdef __cplusplus
}
#endif
#endif /* GEVVA_MOE_H_ */
