// erf and exp evaluated as fixed fp32 fmaf chains.
//
// The reference's expert path computes gelu(x) = 0.5*x*(1+erf(x/sqrt2))
// (src/nvfp4_cutlass.cu:175-177) and its router exp(key-max)
// (src/cuda/kernels/routing_sampling.cuh:420-430) with CUDA's library functions
// under --use_fast_math, whose last bits no CPU can reproduce.  FP4 codes of the
// intermediate activation depend on those last bits, so this header pins one
// definition that compiles to the same IEEE operations with gcc
// (-ffp-contract=off) and with nvcc (every operation is an explicit fmaf or an
// __f*_rn intrinsic, so neither fast-math nor fmad contraction can touch it).
// Coefficients come from fit_transcendentals.py in this directory.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define GV_HD __host__ __device__ __forceinline__
#else
#define GV_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define GV_MUL(a, b) __fmul_rn((a), (b))
#define GV_ADD(a, b) __fadd_rn((a), (b))
#define GV_SUB(a, b) __fsub_rn((a), (b))
#define GV_DIV(a, b) __fdiv_rn((a), (b))
#define GV_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#else
#define GV_MUL(a, b) ((a) * (b))
#define GV_ADD(a, b) ((a) + (b))
#define GV_SUB(a, b) ((a) - (b))
#define GV_DIV(a, b) ((a) / (b))
#define GV_FMA(a, b, c) fmaf((a), (b), (c))
#endif

GV_HD float gv_bits_to_float(uint32_t bits) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(bits);
#else
  float value;
  memcpy(&value, &bits, 4);
  return value;
#endif
}

GV_HD uint32_t gv_float_to_bits(float value) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(value);
#else
  uint32_t bits;
  memcpy(&bits, &value, 4);
  return bits;
#endif
}

// erf as eight half-unit intervals of |x| in [0,4), each a degree-6 polynomial in
// u = |x| - centre; 1 beyond.  Branch-free apart from the NaN test, so sixteen values can
// be evaluated interleaved.  Row i of the table holds c0..c6 (and a pad) of interval i;
// max abs error 8e-8.  Coefficients from fit_transcendentals.py.
#define GV_ERF_TABLE_INIT {\
  {2.763263881e-01f, 1.060013652e+00f, -2.650032640e-01f, -3.091164231e-01f, 1.269483566e-01f, 7.830715179e-02f, -3.948784247e-02f, 0.0f},\
  {7.111556530e-01f, 6.429315209e-01f, -4.821982384e-01f, 2.672714554e-02f, 1.506790370e-01f, -5.125992000e-02f, -2.661922388e-02f, 0.0f},\
  {9.229001403e-01f, 2.365212291e-01f, -2.956515551e-01f, 1.675231010e-01f, -6.140203681e-03f, -4.677713290e-02f, 2.068483829e-02f, 0.0f},\
  {9.866716862e-01f, 5.277483538e-02f, -9.235622734e-02f, 9.017768502e-02f, -4.810455441e-02f, 5.969322287e-03f, 9.039151482e-03f, 0.0f},\
  {9.985373020e-01f, 7.142300252e-03f, -1.607019082e-02f, 2.172697149e-02f, -1.908679493e-02f, 1.058122981e-02f, -2.795148641e-03f, 0.0f},\
  {9.998993874e-01f, 5.862942780e-04f, -1.612264663e-03f, 2.758205635e-03f, -3.257828532e-03f, 2.825851319e-03f, -1.666593715e-03f, 0.0f},\
  {9.999957085e-01f, 2.919363942e-05f, -9.486651834e-05f, 1.952197636e-04f, -2.862895199e-04f, 3.326097503e-04f, -2.724775113e-04f, 0.0f},\
  {9.999998808e-01f, 8.818848301e-07f, -3.305675591e-06f, 7.911847206e-06f, -1.380229787e-05f, 2.020373722e-05f, -2.051217416e-05f, 0.0f},\
}
#define GV_ERF_TABLE_FLOATS 64

#if !defined(__CUDA_ARCH__)
static const float gv_erf_table_host[8][8] = GV_ERF_TABLE_INIT;
#endif

// `table` points at the 64 floats above: gv_erf_table_host on the CPU, a shared-memory
// copy inside kernels (lanes index it with different rows).
GV_HD float gv_erff(float x, const float* table) {
  const float a = fabsf(x);
  if (a != a) return x;  // NaN
  const float clamped = fminf(a, 3.99999976f);
  const float index = truncf(GV_MUL(clamped, 2.0f));
  const float u = GV_SUB(GV_FMA(index, -0.5f, clamped), 0.25f);
  const float* c = table + 8 * (int)index;
#if defined(__CUDA_ARCH__)
  // two 16-byte loads instead of seven 4-byte ones (the table is 16-byte aligned in kernels)
  const float4 lo = *reinterpret_cast<const float4*>(c);
  const float4 hi = *reinterpret_cast<const float4*>(c + 4);
  float p = hi.z;
  p = GV_FMA(p, u, hi.y);
  p = GV_FMA(p, u, hi.x);
  p = GV_FMA(p, u, lo.w);
  p = GV_FMA(p, u, lo.z);
  p = GV_FMA(p, u, lo.y);
  p = GV_FMA(p, u, lo.x);
#else
  float p = c[6];
  p = GV_FMA(p, u, c[5]);
  p = GV_FMA(p, u, c[4]);
  p = GV_FMA(p, u, c[3]);
  p = GV_FMA(p, u, c[2]);
  p = GV_FMA(p, u, c[1]);
  p = GV_FMA(p, u, c[0]);
#endif
  const float r = a >= 4.0f ? 1.0f : p;
  return copysignf(r, x);
}

// erf-GELU exactly as the reference writes it (src/nvfp4_cutlass.cu:175-177):
// 0.5F * value * (1.0F + erff(value * 0.7071067811865475F)), left to right.
GV_HD float gv_gelu_erf(float value, const float* table) {
  const float e = gv_erff(GV_MUL(value, 0.7071067811865475f), table);
  return GV_MUL(GV_MUL(0.5f, value), GV_ADD(1.0f, e));
}

// exp(x), relative error below 2e-7 for x in [-87, 88]; 0 below, +inf above.
GV_HD float gv_expf(float x) {
  if (x != x) return x;
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return gv_bits_to_float(0x7f800000u);
  const float n = rintf(GV_MUL(x, 1.4426950408889634f));
  float r = GV_FMA(n, -0.693145751953125f, x);       // ln2 high part (exact product)
  r = GV_FMA(n, -1.42860682030941723212e-6f, r);     // ln2 low part
  float p = 1.394110848e-03f;
  p = GV_FMA(p, r, 8.375125937e-03f);
  p = GV_FMA(p, r, 4.166635126e-02f);
  p = GV_FMA(p, r, 1.666641533e-01f);
  p = GV_FMA(p, r, 5.000000000e-01f);
  p = GV_FMA(p, r, 1.0f);
  p = GV_FMA(p, r, 1.0f);
  // p in [0.70, 1.42]; scale by 2^n in two exact steps so n = -126..128 is safe
  const int ni = (int)n;
  const int n1 = ni / 2, n2 = ni - n1;
  const float s1 = gv_bits_to_float((uint32_t)(n1 + 127) << 23);
  const float s2 = gv_bits_to_float((uint32_t)(n2 + 127) << 23);
  return GV_MUL(GV_MUL(p, s1), s2);
}

// tanh through gv_expf: 1 - 2/(exp(2y)+1).  Absolute error below 3e-7, which is what the
// GELU needs; the reference's dense-MLP GELU (src/cuda/kernels/fp8.cuh:299-306) calls tanhf.
GV_HD float gv_tanhf(float y) {
  const float e = gv_expf(GV_MUL(2.0f, y));
  return GV_SUB(1.0f, GV_DIV(2.0f, GV_ADD(e, 1.0f)));
}

// tanh-GELU times up, rounded to bf16 by the caller: 0.5*x*(1+tanh(k*(x+0.044715*x^3))),
// operations in the order the reference writes them.
GV_HD float gv_gelu_tanh(float x) {
  const float cube = GV_MUL(GV_MUL(GV_MUL(0.044715f, x), x), x);
  const float inner = GV_MUL(0.7978845608028654f, GV_ADD(x, cube));
  return GV_MUL(GV_MUL(0.5f, x), GV_ADD(1.0f, gv_tanhf(inner)));
}

// 1/sqrt(x) with IEEE square root and division (the reference calls the approximate rsqrtf).
GV_HD float gv_rsqrtf(float x) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(1.0f, __fsqrt_rn(x));
#else
  return 1.0f / sqrtf(x);
#endif
}
