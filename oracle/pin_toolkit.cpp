// TEST INFRASTRUCTURE ONLY.  Exposes the host implementations of the CUDA
// toolkit conversion classes that the reference kernels call
// (__nv_fp8_e4m3 at src/nvfp4_cutlass.cu:312, __nv_fp4x2_e2m1 at :317-320,
// __float2bfloat16_rn at :245) so the oracle's hand-written encoders can be
// checked against them value by value.  Compiles with plain g++.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cstdint>
#include <cstring>

extern "C" {

uint8_t pin_encode_e4m3(float value) {
  const __nv_fp8_e4m3 encoded(value);
  return encoded.__x;
}

float pin_decode_e4m3(uint8_t code) {
  __nv_fp8_e4m3 encoded;
  encoded.__x = static_cast<__nv_fp8_storage_t>(code);
  return static_cast<float>(encoded);
}

// low nibble = first value, as the kernels store it
uint8_t pin_encode_e2m1x2(float first, float second) {
  return __nv_fp4x2_e2m1(float2{first, second}).__x;
}

uint16_t pin_float_to_bf16(float value) {
  const __nv_bfloat16 rounded = __float2bfloat16_rn(value);
  uint16_t bits;
  std::memcpy(&bits, &rounded, 2);
  return bits;
}

void pin_encode_e4m3_many(const float* values, uint8_t* out, long count) {
  for (long i = 0; i < count; ++i) out[i] = pin_encode_e4m3(values[i]);
}

void pin_encode_e2m1_many(const float* values, uint8_t* out, long count) {
  for (long i = 0; i < count; ++i) out[i] = pin_encode_e2m1x2(values[i], 0.0f) & 15;
}

void pin_float_to_bf16_many(const float* values, uint16_t* out, long count) {
  for (long i = 0; i < count; ++i) out[i] = pin_float_to_bf16(values[i]);
}

}  // extern "C"
