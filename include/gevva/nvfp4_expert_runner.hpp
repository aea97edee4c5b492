// Header-only C++ face of the C ABI in gevva_moe.h with the name, methods and error
// behaviour of the reference class gevva::Nvfp4ExpertRunner
// (include/gevva/gpu.hpp:217-247), so that the reference's call sites
// (src/cuda/runtime/prefill.cuh:463-476, :1232-1245, src/cuda/runtime/verifier.cuh:326,
// :1020-1034, construction at src/decisions.cpp:139-143) compile against it unchanged.
//
// The constructor is a template on the model type: anything with
// `tensor(const std::string&)` returning an object whose `.data` is the device
// pointer works, which is what the reference's DeviceModel offers
// (src/nvfp4_cutlass.cu:1792-1802).
#pragma once

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>
#include <utility>

#include "../gevva_moe.h"

namespace gevva {

class Nvfp4ExpertRunner {
 public:
  template <class DeviceModelT>
  Nvfp4ExpertRunner(const DeviceModelT& experts, int layer, int maximum_tokens = 1,
                    Nvfp4ExpertRunner* shared_scratch = nullptr) {
    if (layer < 0 || layer >= 30) throw std::runtime_error("layer must be in [0, 29]");
    const std::string prefix = "layers." + std::to_string(layer) + ".";
    gevva_moe_weights weights{};
    weights.w13 = experts.tensor(prefix + "w13.weight").data;
    weights.w13_sf = experts.tensor(prefix + "w13.weight_scale").data;
    weights.w2 = experts.tensor(prefix + "w2.weight").data;
    weights.w2_sf = experts.tensor(prefix + "w2.weight_scale").data;
    weights.alpha1 = reinterpret_cast<const float*>(experts.tensor(prefix + "g1.alpha").data);
    weights.alpha2 = reinterpret_cast<const float*>(experts.tensor(prefix + "g2.alpha").data);
    weights.in_scale_q1 =
        reinterpret_cast<const float*>(experts.tensor(prefix + "g1.input_scale_quant").data);
    weights.in_scale_q2 =
        reinterpret_cast<const float*>(experts.tensor(prefix + "g2.input_scale_quant").data);
    check(gevva_moe_create(&handle_, &weights, maximum_tokens,
                           shared_scratch ? shared_scratch->handle_ : nullptr, nullptr),
          "Nvfp4ExpertRunner");
  }
  // Direct form for callers that already hold the eight device pointers.
  Nvfp4ExpertRunner(const gevva_moe_weights& weights, int maximum_tokens,
                    Nvfp4ExpertRunner* shared_scratch = nullptr) {
    check(gevva_moe_create(&handle_, &weights, maximum_tokens,
                           shared_scratch ? shared_scratch->handle_ : nullptr, nullptr),
          "Nvfp4ExpertRunner");
  }
  ~Nvfp4ExpertRunner() { gevva_moe_destroy(handle_); }
  Nvfp4ExpertRunner(const Nvfp4ExpertRunner&) = delete;
  Nvfp4ExpertRunner& operator=(const Nvfp4ExpertRunner&) = delete;
  Nvfp4ExpertRunner(Nvfp4ExpertRunner&& other) noexcept : handle_(other.handle_) {
    other.handle_ = nullptr;
  }
  Nvfp4ExpertRunner& operator=(Nvfp4ExpertRunner&& other) noexcept {
    if (this != &other) {
      gevva_moe_destroy(handle_);
      handle_ = other.handle_;
      other.handle_ = nullptr;
    }
    return *this;
  }

  void launch(const void* input, const int* expert_ids, const float* route_weights, void* output,
              cudaStream_t stream) const {
    check(gevva_moe_launch(handle_, input, expert_ids, route_weights, output, 1, stream), "launch");
  }
  void launch_batch(const void* input, const int* expert_ids, const float* route_weights,
                    void* output, int tokens, cudaStream_t stream) const {
    check(gevva_moe_launch(handle_, input, expert_ids, route_weights, output, tokens, stream),
          "launch_batch");
  }
  void launch_batch_unreduced(const void* input, const int* expert_ids, int tokens,
                              cudaStream_t stream) const {
    check(gevva_moe_launch(handle_, input, expert_ids, nullptr, nullptr, tokens, stream),
          "launch_batch_unreduced");
  }
  const void* routed_output() const { return gevva_moe_routed_output(handle_); }
  const int* inverse_routes() const { return gevva_moe_inverse_routes(handle_); }

 private:
  static void check(int status, const char* where) {
    if (status != GEVVA_MOE_OK)
      throw std::runtime_error(std::string(where) + ": " + gevva_moe_strerror(status));
  }
  gevva_moe* handle_ = nullptr;
};

// Stands where the reference launches route_128_top8_kernel<<<rows,128,0,stream>>>
// (src/cuda/runtime/prefill.cuh:420-422); same argument order as the kernel.
inline void route_128_top8(const void* logits, const void* expert_scale, float* weights, int* ids,
                           int rows, cudaStream_t stream, const float* activation_scales = nullptr,
                           const float* projection_weight_scale = nullptr, int ld = 128) {
  const int status = gevva_moe_route(logits, ld, expert_scale, weights, ids, rows,
                                     activation_scales, projection_weight_scale, stream);
  if (status != GEVVA_MOE_OK)
    throw std::runtime_error(std::string("route_128_top8: ") + gevva_moe_strerror(status));
}

}  // namespace gevva
