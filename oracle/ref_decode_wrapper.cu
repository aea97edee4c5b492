// TEST INFRASTRUCTURE ONLY.  Compiles the reference's own NVFP4 decode helpers
// (src/cuda/kernels/nvfp4_reference.cuh:2-16, `__device__ __host__` functions) for
// the host by including that file where it lies; nothing is copied.  REFERENCE_ROOT
// is given by oracle/Makefile.  Only the host side of the fragment is used.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include GV_REFERENCE_DECODE_HEADER

extern "C" {
float ref_decode_e2m1(unsigned value) { return decode_e2m1(value); }
float ref_decode_e4m3(unsigned value) { return decode_e4m3(value); }
}
