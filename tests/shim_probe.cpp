// Compile-and-run check of include/gevva/nvfp4_expert_runner.hpp against a stand-in for the
// reference's DeviceModel (an object whose tensor(name).data is a device pointer,
// src/nvfp4_cutlass.cu:1792-1802).  Without arguments it needs no GPU: it checks that the
// class has the reference's constructor and five methods (include/gevva/gpu.hpp:217-247) and
// that failures surface as std::runtime_error.  With "gpu" it runs one 16-token batch of zero
// weights through launch_batch and launch_batch_unreduced.  Built and run by test_cpp_shim.py.
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "gevva/nvfp4_expert_runner.hpp"

namespace {

struct Tensor {
  const void* data;
};

struct FakeDeviceModel {
  std::map<std::string, void*> tensors;
  std::vector<std::string> asked;
  Tensor tensor(const std::string& name) const {
    const_cast<FakeDeviceModel*>(this)->asked.push_back(name);
    const auto found = tensors.find(name);
    return Tensor{found == tensors.end() ? nullptr : found->second};
  }
};

// the reference's signatures, taken as member pointers: a mismatch fails to compile
using Runner = gevva::Nvfp4ExpertRunner;
void (Runner::*const kLaunch)(const void*, const int*, const float*, void*, cudaStream_t) const = &Runner::launch;
void (Runner::*const kLaunchBatch)(const void*, const int*, const float*, void*, int, cudaStream_t) const =
    &Runner::launch_batch;
void (Runner::*const kUnreduced)(const void*, const int*, int, cudaStream_t) const = &Runner::launch_batch_unreduced;
const void* (Runner::*const kRouted)() const = &Runner::routed_output;
const int* (Runner::*const kInverse)() const = &Runner::inverse_routes;

int fail(const char* what) {
  std::printf("FAIL: %s\n", what);
  return 1;
}

int host_checks() {
  (void)kLaunch; (void)kLaunchBatch; (void)kUnreduced; (void)kRouted; (void)kInverse;
  FakeDeviceModel empty;
  try {
    Runner runner(empty, 0, 16);
    return fail("null tensors were accepted");
  } catch (const std::runtime_error& error) {
    if (!std::strstr(error.what(), "Nvfp4ExpertRunner")) return fail("error text does not name the class");
  }
  if (empty.asked.size() != 8 || empty.asked[0] != "layers.0.w13.weight" ||
      empty.asked[7] != "layers.0.g2.input_scale_quant")
    return fail("the eight tensor names of layer 0 were not requested");
  try {
    Runner runner(empty, 30, 16);
    return fail("layer 30 was accepted");
  } catch (const std::runtime_error&) {
  }
  try {
    gevva::route_128_top8(nullptr, nullptr, nullptr, nullptr, 4, nullptr);
    return fail("null router arguments were accepted");
  } catch (const std::runtime_error&) {
  }
  std::printf("host checks ok\n");
  return 0;
}

int gpu_checks() {
  constexpr int kTokens = 16, kLayer = 7;
  FakeDeviceModel model;
  const std::string prefix = "layers." + std::to_string(kLayer) + ".";
  const std::pair<const char*, size_t> sizes[] = {
      {"w13.weight", 128ull * 1408 * 1408}, {"w13.weight_scale", 128ull * 1408 * 176},
      {"w2.weight", 128ull * 2816 * 352},   {"w2.weight_scale", 128ull * 2816 * 44},
      {"g1.alpha", 512},                    {"g2.alpha", 512},
      {"g1.input_scale_quant", 512},        {"g2.input_scale_quant", 512}};
  for (const auto& entry : sizes) {
    void* p = nullptr;
    if (cudaMalloc(&p, entry.second) != cudaSuccess || cudaMemset(p, 0, entry.second) != cudaSuccess)
      return fail("cudaMalloc");
    model.tensors[prefix + entry.first] = p;
  }
  Runner runner(model, kLayer, kTokens);
  Runner second(model, kLayer, kTokens, &runner);   // shares the first one's scratch
  try {
    Runner mismatch(model, kLayer, 2 * kTokens, &runner);
    return fail("shared scratch with another capacity was accepted");
  } catch (const std::runtime_error&) {
  }
  void *in = nullptr, *out = nullptr;
  int* ids = nullptr;
  float* weights = nullptr;
  cudaMalloc(&in, kTokens * 2816 * 2);
  cudaMalloc(&out, kTokens * 2816 * 2);
  cudaMalloc(reinterpret_cast<void**>(&ids), kTokens * 8 * sizeof(int));
  cudaMalloc(reinterpret_cast<void**>(&weights), kTokens * 8 * sizeof(float));
  cudaMemset(in, 0, kTokens * 2816 * 2);
  cudaMemset(out, 0xff, kTokens * 2816 * 2);
  cudaMemset(weights, 0, kTokens * 8 * sizeof(float));
  std::vector<int> host_ids(kTokens * 8);
  for (int i = 0; i < kTokens * 8; ++i) host_ids[i] = (i * 37) % 128;
  cudaMemcpy(ids, host_ids.data(), host_ids.size() * sizeof(int), cudaMemcpyHostToDevice);
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  runner.launch(in, ids, weights, out, stream);   // one token
  runner.launch_batch(in, ids, weights, out, kTokens, stream);
  second.launch_batch_unreduced(in, ids, kTokens, stream);   // last: its plan is what is read back below
  try {
    runner.launch_batch(in, ids, weights, out, kTokens + 1, stream);
    return fail("a batch beyond the capacity was accepted");
  } catch (const std::runtime_error&) {
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return fail("stream");
  std::vector<unsigned short> host_out(kTokens * 2816);
  cudaMemcpy(host_out.data(), out, host_out.size() * 2, cudaMemcpyDeviceToHost);
  for (unsigned short v : host_out)
    if ((v & 0x7fff) != 0) return fail("zero weights gave a non-zero output");
  std::vector<int> inverse(kTokens * 8);
  cudaMemcpy(inverse.data(), second.inverse_routes(), inverse.size() * sizeof(int), cudaMemcpyDeviceToHost);
  std::vector<int> seen(kTokens * 8, 0);
  for (int v : inverse) {
    if (v < 0 || v >= kTokens * 8 || seen[v]++) return fail("inverse_routes is not a permutation");
  }
  if (!second.routed_output()) return fail("routed_output is null");
  std::printf("gpu checks ok\n");
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  const int host = host_checks();
  if (host != 0 || argc < 2 || std::strcmp(argv[1], "gpu") != 0) return host;
  try {
    return gpu_checks();
  } catch (const std::exception& error) {
    std::printf("FAIL: %s\n", error.what());
    return 1;
  }
}
