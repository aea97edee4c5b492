// The feed-forward steps around the expert path, and the dense FP8 GeGLU MLP that runs
// beside it (30-layer configuration):
//   ff_prepare   dual RMSNorm + router input  (reference: dual_rmsnorm_router_2816_kernel,
//                src/cuda/kernels/normalization.cuh:83-123)
//   fp8 rows     per-row dynamic E4M3 quantisation (quantize_fp8_rows_kernel,
//                src/cuda/kernels/fp8.cuh:2-26)
//   gelu+quant   tanh-GeGLU of the unscaled gate/up outputs, requantised per row
//                (gelu_quantize_fp8_2112_kernel, src/cuda/kernels/fp8.cuh:308-364)
//   ff_finalize  8-route weighted reduce + three RMSNorms + residual + layer scalar
//                (finalize_feedforward_routes_2816_kernel, normalization.cuh:249-377)
// The three projections themselves are grouped_gemm.cu's kernel in its FP8 form.
// Rows are 2816 wide: 352 threads x 8 columns, 16-byte loads and stores.  Sums of squares
// are folded in one fixed order (thread, shuffle-down tree, warps in order) and the
// reciprocal square root is IEEE, so a CPU can reproduce every bit.
#include "gv_common.cuh"
#include "gv_launchers.h"
#include "gv_plan.cuh"

namespace gv {

namespace {

constexpr int kRowThreads = kHidden / 8;  // 352
constexpr int kDense = 2112;
constexpr int kDenseThreads = 288;        // 264 active threads x 8 columns

__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
  out[0] = __uint_as_float(raw.x << 16);
  out[1] = __uint_as_float(raw.x & 0xffff0000u);
  out[2] = __uint_as_float(raw.y << 16);
  out[3] = __uint_as_float(raw.y & 0xffff0000u);
  out[4] = __uint_as_float(raw.z << 16);
  out[5] = __uint_as_float(raw.z & 0xffff0000u);
  out[6] = __uint_as_float(raw.w << 16);
  out[7] = __uint_as_float(raw.w & 0xffff0000u);
}

__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 out;
  __nv_bfloat162 p;
  p = __floats2bfloat162_rn(v[0], v[1]); out.x = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[2], v[3]); out.y = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[4], v[5]); out.z = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[6], v[7]); out.w = *reinterpret_cast<uint32_t*>(&p);
  return out;
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Block-wide sum of squares of 8 values per thread, in the fixed order described above.
// `scratch` holds blockDim/32 + 1 floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum_squares(const float* v, float* scratch) {
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = __fmaf_rn(v[i], v[i], s);
  // shuffle-down tree; lanes beyond the tree keep their own value, lane 0 ends with the sum
#pragma unroll
  for (int offset = 16; offset; offset >>= 1) {
    const float other = __shfl_down_sync(0xffffffffu, s, offset);
    if ((threadIdx.x & 31) + offset < 32) s = __fadd_rn(s, other);
  }
  const int warps = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = scratch[0];
    for (int w = 1; w < warps; ++w) total = __fadd_rn(total, scratch[w]);
    scratch[warps] = total;
  }
  __syncthreads();
  const float total = scratch[warps];
  __syncthreads();
  return total;
}

__global__ void __launch_bounds__(kRowThreads)
ff_prepare_kernel(const __nv_bfloat16* __restrict__ input, const __nv_bfloat16* __restrict__ dense_weight,
                  const __nv_bfloat16* __restrict__ expert_weight,
                  const __nv_bfloat16* __restrict__ router_scale, __nv_bfloat16* __restrict__ dense_out,
                  __nv_bfloat16* __restrict__ expert_out, __nv_bfloat16* __restrict__ router_out) {
  __shared__ float scratch[kRowThreads / 32 + 1];
  const size_t base = static_cast<size_t>(blockIdx.x) * kHidden;
  float x[8], dw[8], ew[8], rs[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(input + base) + threadIdx.x), x);
  unpack8(__ldg(reinterpret_cast<const uint4*>(dense_weight) + threadIdx.x), dw);
  unpack8(__ldg(reinterpret_cast<const uint4*>(expert_weight) + threadIdx.x), ew);
  unpack8(__ldg(reinterpret_cast<const uint4*>(router_scale) + threadIdx.x), rs);
  const float sum = block_sum_squares(x, scratch);
  const float inverse = gv_rsqrtf(__fadd_rn(__fdiv_rn(sum, static_cast<float>(kHidden)), 1e-6f));
  const float root = gv_rsqrtf(static_cast<float>(kHidden));
  float d[8], e[8], r[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float normalized = __fmul_rn(x[i], inverse);
    d[i] = __fmul_rn(normalized, dw[i]);
    e[i] = __fmul_rn(normalized, ew[i]);
    const float routed = bf16_round(__fmul_rn(bf16_round(normalized), rs[i]));
    r[i] = __fmul_rn(routed, root);
  }
  reinterpret_cast<uint4*>(dense_out + base)[threadIdx.x] = pack8(d);
  reinterpret_cast<uint4*>(expert_out + base)[threadIdx.x] = pack8(e);
  reinterpret_cast<uint4*>(router_out + base)[threadIdx.x] = pack8(r);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
  for (int offset = 16; offset; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  const int warps = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = scratch[0];
  for (int w = 1; w < warps; ++w) total = fmaxf(total, scratch[w]);
  __syncthreads();
  return total;
}

__device__ __forceinline__ uint2 encode_e4m3x8(const float* v, float inverse) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= encode_e4m3(__fmul_rn(v[i], inverse)) << (8 * i);
    hi |= encode_e4m3(__fmul_rn(v[4 + i], inverse)) << (8 * i);
  }
  return make_uint2(lo, hi);
}

__global__ void __launch_bounds__(kRowThreads)
fp8_quantize_rows_kernel(const __nv_bfloat16* __restrict__ input, uint8_t* __restrict__ out,
                         float* __restrict__ scales) {
  __shared__ float scratch[kRowThreads / 32 + 1];
  const size_t base = static_cast<size_t>(blockIdx.x) * kHidden;
  float x[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(input + base) + threadIdx.x), x);
  float maximum = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) maximum = fmaxf(maximum, fabsf(x[i]));
  maximum = block_max(maximum, scratch);
  const float scale = fmaxf(__fdiv_rn(maximum, 448.0f), 1.17549435e-38f);
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
  const float inverse = __fdiv_rn(1.0f, scale);
  reinterpret_cast<uint2*>(out + base)[threadIdx.x] = encode_e4m3x8(x, inverse);
}

__global__ void __launch_bounds__(kDenseThreads)
gelu_quantize_fp8_kernel(const __nv_bfloat16* __restrict__ gate_up,
                         const float* __restrict__ activation_scales, float gate_w_scale,
                         float up_w_scale, uint8_t* __restrict__ out, float* __restrict__ scales) {
  __shared__ float scratch[kDenseThreads / 32 + 1];
  const int row = blockIdx.x;
  const bool active = threadIdx.x < kDense / 8;
  const float gate_scale = __fmul_rn(activation_scales[row], gate_w_scale);
  const float up_scale = __fmul_rn(activation_scales[row], up_w_scale);
  float value[8];
  float maximum = 0.0f;
  if (active) {
    float g[8], u[8];
    const uint4* src = reinterpret_cast<const uint4*>(gate_up + static_cast<size_t>(row) * 2 * kDense);
    unpack8(__ldg(src + threadIdx.x), g);
    unpack8(__ldg(src + kDense / 8 + threadIdx.x), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gv = bf16_round(__fmul_rn(g[i], gate_scale));
      const float uv = bf16_round(__fmul_rn(u[i], up_scale));
      value[i] = bf16_round(__fmul_rn(gv_gelu_tanh(gv), uv));
      maximum = fmaxf(maximum, fabsf(value[i]));
    }
  }
  maximum = block_max(maximum, scratch);
  const float scale = fmaxf(__fdiv_rn(maximum, 448.0f), 1.17549435e-38f);
  if (threadIdx.x == 0) scales[row] = scale;
  const float inverse = __fdiv_rn(1.0f, scale);
  if (active)
    reinterpret_cast<uint2*>(out + static_cast<size_t>(row) * kDense)[threadIdx.x] =
        encode_e4m3x8(value, inverse);
}

__global__ void __launch_bounds__(kRowThreads)
ff_finalize_kernel(const __nv_bfloat16* __restrict__ dense, const __nv_bfloat16* __restrict__ dense_weight,
                   const __nv_bfloat16* __restrict__ expert_routes,
                   const float* __restrict__ route_weights, const int* __restrict__ inverse_routes,
                   const __nv_bfloat16* __restrict__ expert_weight,
                   const __nv_bfloat16* __restrict__ combined_weight,
                   const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ layer_scalar, __nv_bfloat16* __restrict__ output,
                   const float* __restrict__ dense_activation_scales,
                   const float* __restrict__ dense_projection_scale) {
  __shared__ float scratch[kRowThreads / 32 + 1];
  const int row = blockIdx.x;
  const size_t base = static_cast<size_t>(row) * kHidden;
  float d[8], e[8], w[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(dense + base) + threadIdx.x), d);
  if (dense_activation_scales) {
    const float scale = __fmul_rn(dense_activation_scales[row], dense_projection_scale[0]);
#pragma unroll
    for (int i = 0; i < 8; ++i) d[i] = bf16_round(__fmul_rn(d[i], scale));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = 0.0f;
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    const int index = row * kTopK + k;
    const int source = inverse_routes ? inverse_routes[index] : index;
    const float weight = route_weights[index];
    float v[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(expert_routes + static_cast<size_t>(source) * kHidden) +
                  threadIdx.x),
            v);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = __fmaf_rn(v[i], weight, e[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = bf16_round(e[i]);
  const float dense_inverse =
      gv_rsqrtf(__fadd_rn(__fdiv_rn(block_sum_squares(d, scratch), static_cast<float>(kHidden)), 1e-6f));
  const float expert_inverse =
      gv_rsqrtf(__fadd_rn(__fdiv_rn(block_sum_squares(e, scratch), static_cast<float>(kHidden)), 1e-6f));
  float combined[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(dense_weight) + threadIdx.x), w);
#pragma unroll
  for (int i = 0; i < 8; ++i) combined[i] = bf16_round(__fmul_rn(__fmul_rn(d[i], dense_inverse), w[i]));
  unpack8(__ldg(reinterpret_cast<const uint4*>(expert_weight) + threadIdx.x), w);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    combined[i] = bf16_round(__fadd_rn(combined[i], bf16_round(__fmul_rn(__fmul_rn(e[i], expert_inverse), w[i]))));
  const float combined_inverse = gv_rsqrtf(
      __fadd_rn(__fdiv_rn(block_sum_squares(combined, scratch), static_cast<float>(kHidden)), 1e-6f));
  float r[8], out[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(combined_weight) + threadIdx.x), w);
  unpack8(__ldg(reinterpret_cast<const uint4*>(residual + base) + threadIdx.x), r);
  const float scalar = __bfloat162float(*layer_scalar);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float normalized = bf16_round(__fmul_rn(__fmul_rn(combined[i], combined_inverse), w[i]));
    out[i] = __fmul_rn(bf16_round(__fadd_rn(r[i], normalized)), scalar);
  }
  reinterpret_cast<uint4*>(output + base)[threadIdx.x] = pack8(out);
}

// Plan of a dense GEMM seen as a grouped one with a single "expert" that owns every row.
__global__ void __launch_bounds__(kExperts) dense_plan_kernel(int rows, RoutePlan plan) {
  __shared__ int scan_scratch[16];
  publish_groups(threadIdx.x == 0 ? rows : 0, rows, plan, scan_scratch);
}

__global__ void fp8_amax_kernel(const float* __restrict__ w, size_t count, unsigned int* amax_bits) {
  float maximum = 0.0f;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    maximum = fmaxf(maximum, fabsf(w[i]));
  for (int offset = 16; offset; offset >>= 1)
    maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(maximum));
}

__global__ void fp8_pack_kernel(const float* __restrict__ w, size_t count, const unsigned int* amax_bits,
                                uint8_t* __restrict__ out, float* __restrict__ scale_out) {
  const float scale = fmaxf(__fdiv_rn(__uint_as_float(*amax_bits), 448.0f), 1.17549435e-38f);
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = static_cast<uint8_t>(encode_e4m3(__fdiv_rn(w[i], scale)));
}

}  // namespace

void launch_ff_prepare(const void* input, const void* dense_weight, const void* expert_weight,
                       const void* router_scale, void* dense_out, void* expert_out, void* router_out,
                       int rows, cudaStream_t stream) {
  using B = __nv_bfloat16;
  ff_prepare_kernel<<<rows, kRowThreads, 0, stream>>>(
      static_cast<const B*>(input), static_cast<const B*>(dense_weight), static_cast<const B*>(expert_weight),
      static_cast<const B*>(router_scale), static_cast<B*>(dense_out), static_cast<B*>(expert_out),
      static_cast<B*>(router_out));
}

void launch_fp8_quantize_rows(const void* input, uint8_t* out, float* scales, int rows,
                              cudaStream_t stream) {
  fp8_quantize_rows_kernel<<<rows, kRowThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(input), out,
                                                              scales);
}

void launch_gelu_quantize_fp8(const void* gate_up, const float* activation_scales, float gate_w_scale,
                              float up_w_scale, uint8_t* out, float* scales, int rows,
                              cudaStream_t stream) {
  gelu_quantize_fp8_kernel<<<rows, kDenseThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate_up), activation_scales, gate_w_scale, up_w_scale, out, scales);
}

void launch_ff_finalize(const void* dense, const void* dense_weight, const void* expert_routes,
                        const float* route_weights, const int* inverse_routes, const void* expert_weight,
                        const void* combined_weight, const void* residual, const void* layer_scalar,
                        void* output, int rows, const float* dense_activation_scales,
                        const float* dense_projection_scale, cudaStream_t stream) {
  using B = __nv_bfloat16;
  ff_finalize_kernel<<<rows, kRowThreads, 0, stream>>>(
      static_cast<const B*>(dense), static_cast<const B*>(dense_weight), static_cast<const B*>(expert_routes),
      route_weights, inverse_routes, static_cast<const B*>(expert_weight),
      static_cast<const B*>(combined_weight), static_cast<const B*>(residual),
      static_cast<const B*>(layer_scalar), static_cast<B*>(output), dense_activation_scales,
      dense_projection_scale);
}

void launch_dense_plan(int rows, const RoutePlan& plan, cudaStream_t stream) {
  dense_plan_kernel<<<1, kExperts, 0, stream>>>(rows, plan);
}

void launch_pack_fp8(const float* w, size_t count, uint8_t* out, float* scale_out, cudaStream_t stream) {
  unsigned int* accumulator = nullptr;
  cudaMallocAsync(reinterpret_cast<void**>(&accumulator), sizeof(unsigned int), stream);
  cudaMemsetAsync(accumulator, 0, sizeof(unsigned int), stream);
  fp8_amax_kernel<<<592, 256, 0, stream>>>(w, count, accumulator);
  fp8_pack_kernel<<<592, 256, 0, stream>>>(w, count, accumulator, out, scale_out);
  cudaFreeAsync(accumulator, stream);
}

}  // namespace gv
