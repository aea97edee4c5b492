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

// erf(x), max abs error 9e-8 over the reals.
GV_HD float gv_erff(float x) {
  const float a = fabsf(x);
  float r;
  if (a < 1.0f) {
    // erf(a) = a * p(2*a^2 - 1)
    const float t = GV_FMA(GV_MUL(a, a), 2.0f, -1.0f);
    float p = 1.230605449e-06f;
    p = GV_FMA(p, t, -1.766906826e-05f);
    p = GV_FMA(p, t, 2.175135451e-04f);
    p = GV_FMA(p, t, -2.285419498e-03f);
    p = GV_FMA(p, t, 1.985249668e-02f);
    p = GV_FMA(p, t, -1.405360997e-01f);
    p = GV_FMA(p, t, 9.654687643e-01f);
    r = GV_MUL(a, p);
  } else if (a < 4.0f) {
    // Three unit intervals, each a degree-9 polynomial in u = 2*(a - centre).
    float c0, c1, c2, c3, c4, c5, c6, c7, c8, c9, centre;
    if (a < 2.0f) {
      centre = 1.5f;
      c0 = 9.661051631e-01f; c1 = 5.946514383e-02f; c2 = -4.459885508e-02f;
      c3 = 1.734401286e-02f; c4 = -2.787466859e-03f; c5 = -4.646643938e-04f;
      c6 = 3.020868462e-04f; c7 = -3.679370275e-05f; c8 = -9.383547876e-06f;
      c9 = 3.037872602e-06f;
    } else if (a < 3.0f) {
      centre = 2.5f;
      c0 = 9.995930195e-01f; c1 = 1.089142170e-03f; c2 = -1.361434348e-03f;
      c3 = 1.043760800e-03f; c4 = -5.388446734e-04f; c5 = 1.911700965e-04f;
      c6 = -4.387873560e-05f; c7 = 4.229543720e-06f; c8 = 1.196742119e-06f;
      c9 = -4.803476372e-07f;
    } else {
      centre = 3.5f;
      c0 = 9.999992847e-01f; c1 = 2.699713605e-06f; c2 = -4.724084192e-06f;
      c3 = 5.286926353e-06f; c4 = -4.235686902e-06f; c5 = 2.566234798e-06f;
      c6 = -1.205385843e-06f; c7 = 4.543294381e-07f; c8 = -1.446854156e-07f;
      c9 = 3.033540352e-08f;
    }
    const float u = GV_MUL(GV_SUB(a, centre), 2.0f);
    float p = c9;
    p = GV_FMA(p, u, c8);
    p = GV_FMA(p, u, c7);
    p = GV_FMA(p, u, c6);
    p = GV_FMA(p, u, c5);
    p = GV_FMA(p, u, c4);
    p = GV_FMA(p, u, c3);
    p = GV_FMA(p, u, c2);
    p = GV_FMA(p, u, c1);
    p = GV_FMA(p, u, c0);
    r = p;
  } else {
    r = 1.0f;  // also NaN-free for +-inf; NaN input compares false above and lands here
  }
  if (a != a) return x;  // propagate NaN
  return x < 0.0f ? -r : r;
}

// erf-GELU exactly as the reference writes it (src/nvfp4_cutlass.cu:175-177):
// 0.5F * value * (1.0F + erff(value * 0.7071067811865475F)), left to right.
GV_HD float gv_gelu_erf(float value) {
  const float e = gv_erff(GV_MUL(value, 0.7071067811865475f));
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
