// Scratch of one expert runner: sizes, and the acquire/release sequence with the allocator
// injected, so that every partial-initialisation path can be exercised on the host without a GPU
// (the reference does the same for its FP8 resources, src/gpu/fp8_resources.hpp:9-12, tested by
// tests/test_fp8_resources.cpp:8-37).  Buffer sizes follow the reference's ExpertScratch
// (src/nvfp4_cutlass.cu:1680-1736) with scale regions padded to 128 rows per expert (:1699-1706).
#pragma once

#include <stddef.h>

namespace gv {

struct ScratchSizes {
  size_t routes;
  size_t tile_capacity;   // entries of the tile -> expert list
  size_t chunks;          // 1024-route chunks of the multi-block sort
  size_t int_count;       // ints of the plan block
  size_t bytes[7];        // input codes, input scales, w13 output, intermediate codes,
                          // intermediate scales, w2 output, plan ints
  bool zeroed[7];         // buffers that must start at zero
};

inline ScratchSizes scratch_sizes(int tokens) {
  constexpr size_t kRoutesPerToken = 8, kExpertCount = 128, kHiddenWidth = 2816, kInterWidth = 704;
  ScratchSizes s{};
  s.routes = static_cast<size_t>(tokens) * kRoutesPerToken;
  const size_t padded_rows = s.routes + kExpertCount * 127;
  s.tile_capacity = s.routes / 128 + kExpertCount + 1;
  s.chunks = (s.routes + 1023) / 1024;
  s.int_count = 3 * s.routes + 2 * (kExpertCount + 1) + 3 * (s.tile_capacity + 1) + s.chunks * kExpertCount + 1 + 64;
  s.bytes[0] = s.routes * (kHiddenWidth / 2);
  s.bytes[1] = padded_rows * (kHiddenWidth / 16);
  s.bytes[2] = s.routes * 2 * kInterWidth * 2;
  s.bytes[3] = s.routes * (kInterWidth / 2);
  s.bytes[4] = padded_rows * (kInterWidth / 16);
  s.bytes[5] = s.routes * kHiddenWidth * 2;
  s.bytes[6] = s.int_count * sizeof(int);
  const bool zeroed[7] = {true, true, false, true, true, false, true};
  for (int i = 0; i < 7; ++i) s.zeroed[i] = zeroed[i];
  return s;
}

// Runtime: static bool allocate(void**, size_t), static bool zero(void*, size_t),
// static void release(void*) noexcept.  allocate/zero return false on failure.
template <class Runtime>
struct ScratchMemory {
  void* buffers[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};

  // All seven buffers or none: on any failure everything taken so far is given back.
  bool acquire(const ScratchSizes& sizes) {
    for (int i = 0; i < 7; ++i) {
      if (!Runtime::allocate(&buffers[i], sizes.bytes[i])) {
        buffers[i] = nullptr;
        release();
        return false;
      }
    }
    for (int i = 0; i < 7; ++i) {
      if (sizes.zeroed[i] && !Runtime::zero(buffers[i], sizes.bytes[i])) {
        release();
        return false;
      }
    }
    return true;
  }

  void release() noexcept {
    for (int i = 6; i >= 0; --i) {
      if (buffers[i]) Runtime::release(buffers[i]);
      buffers[i] = nullptr;
    }
  }
};

}  // namespace gv
