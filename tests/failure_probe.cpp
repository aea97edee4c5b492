// Host-only checks of two failure paths, with no GPU involved (built and run by
// test_host_failure_paths.py):
//  1. the cross-rank barrier of the expert-parallel path (csrc/gv_ep_protocol.h, the code the
//     device kernel runs) driven by one thread per rank: complete barriers pass; when one rank
//     is withheld the others give up after their bounded wait and report a timeout; when the
//     late rank then arrives, later barriers pass again;
//  2. the scratch acquisition of a runner (csrc/gv_scratch.h) with an allocator that fails at
//     its k-th call, for every k: nothing is leaked and nothing is freed twice (the pattern of
//     the reference's tests/test_fp8_resources.cpp:8-37).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <set>
#include <thread>
#include <vector>

#include "../gevva_b200/csrc/gv_ep_protocol.h"
#include "../gevva_b200/csrc/gv_scratch.h"

namespace {

constexpr int kWorld = 4;

struct HostFlags {
  std::atomic<int> flags[kWorld][kWorld];  // [owner][slot]
  HostFlags() {
    for (auto& row : flags)
      for (auto& f : row) f.store(0);
  }
};

struct HostPort {
  HostFlags& memory;
  int rank;
  std::chrono::milliseconds limit;
  std::chrono::steady_clock::time_point start;
  void publish(int peer, int slot, int value) { memory.flags[peer][slot].store(value, std::memory_order_release); }
  int observe(int slot) { return memory.flags[rank][slot].load(std::memory_order_acquire); }
  void start_clock() { start = std::chrono::steady_clock::now(); }
  bool expired() { return std::chrono::steady_clock::now() - start > limit; }
  void pause() { std::this_thread::yield(); }
};

// One rank's barrier: what the 32 lanes of ep_barrier_kernel do side by side.
bool barrier(HostFlags& memory, int rank, int epoch, int limit_ms) {
  HostPort port{memory, rank, std::chrono::milliseconds(limit_ms), {}};
  for (int lane = 0; lane < kWorld; ++lane) gv::ep_barrier_announce(port, rank, lane, epoch);
  bool ok = true;
  for (int lane = 0; lane < kWorld; ++lane) ok = gv::ep_barrier_await(port, lane, epoch) && ok;
  return ok;
}

int fail(const char* what) {
  std::printf("FAIL: %s\n", what);
  return 1;
}

int barrier_checks() {
  HostFlags memory;
  // three complete barriers
  for (int epoch = 1; epoch <= 3; ++epoch) {
    bool ok[kWorld] = {};
    std::vector<std::thread> ranks;
    for (int r = 0; r < kWorld; ++r)
      ranks.emplace_back([&, r] { ok[r] = barrier(memory, r, epoch, 2000); });
    for (auto& t : ranks) t.join();
    for (bool v : ok)
      if (!v) return fail("a complete barrier timed out");
  }
  // rank 2 is withheld in barrier 4: the others must time out, each within its own limit
  {
    bool ok[kWorld] = {true, true, true, true};
    std::vector<std::thread> ranks;
    const auto begin = std::chrono::steady_clock::now();
    for (int r = 0; r < kWorld; ++r)
      if (r != 2) ranks.emplace_back([&, r] { ok[r] = barrier(memory, r, 4, 100); });
    for (auto& t : ranks) t.join();
    const auto took = std::chrono::steady_clock::now() - begin;
    if (ok[0] || ok[1] || ok[3]) return fail("a rank passed a barrier that one rank never joined");
    if (took > std::chrono::milliseconds(1500)) return fail("the bounded wait took far longer than its limit");
  }
  // the late rank arrives: it finds the others' flags already at 4 and passes at once
  if (!barrier(memory, 2, 4, 100)) return fail("the late rank did not pass once it arrived");
  // and the next barrier is complete again for everybody
  {
    bool ok[kWorld] = {};
    std::vector<std::thread> ranks;
    for (int r = 0; r < kWorld; ++r) ranks.emplace_back([&, r] { ok[r] = barrier(memory, r, 5, 2000); });
    for (auto& t : ranks) t.join();
    for (bool v : ok)
      if (!v) return fail("the barrier after a timeout did not recover");
  }
  std::printf("barrier checks ok\n");
  return 0;
}

struct FakeRuntime {
  static inline int calls = 0, fail_at = 0, double_frees = 0;
  static inline std::set<void*> live;
  static bool step() { return ++calls != fail_at; }
  static bool allocate(void** pointer, size_t bytes) {
    if (!step()) return false;
    *pointer = ::operator new(bytes ? 16 : 16);   // sizes are checked separately; a token block suffices
    live.insert(*pointer);
    return true;
  }
  static bool zero(void* pointer, size_t) { return step() && live.count(pointer) == 1; }
  static void release(void* pointer) noexcept {
    if (live.erase(pointer) != 1) ++double_frees;
    else ::operator delete(pointer);
  }
};

int scratch_checks() {
  const gv::ScratchSizes sizes = gv::scratch_sizes(4096);
  if (sizes.routes != 32768 || sizes.bytes[0] != 32768ull * 1408 || sizes.bytes[5] != 32768ull * 2816 * 2 ||
      sizes.bytes[1] != (32768ull + 128 * 127) * 176 || sizes.bytes[4] != (32768ull + 128 * 127) * 44)
    return fail("scratch sizes");
  // count the steps of a successful acquisition, then fail each of them in turn
  FakeRuntime::calls = 0;
  FakeRuntime::fail_at = 0;
  {
    gv::ScratchMemory<FakeRuntime> memory;
    if (!memory.acquire(sizes)) return fail("acquisition without injected failure");
    if (FakeRuntime::live.size() != 7) return fail("seven buffers expected");
    memory.release();
    if (!FakeRuntime::live.empty()) return fail("release left buffers behind");
    memory.release();   // idempotent
  }
  const int steps = FakeRuntime::calls;
  if (steps != 7 + 5) return fail("seven allocations and five clears expected");
  for (int k = 1; k <= steps; ++k) {
    FakeRuntime::calls = 0;
    FakeRuntime::fail_at = k;
    gv::ScratchMemory<FakeRuntime> memory;
    if (memory.acquire(sizes)) return fail("an injected failure went unnoticed");
    if (!FakeRuntime::live.empty()) return fail("a failed acquisition leaked a buffer");
    for (void* b : memory.buffers)
      if (b) return fail("a failed acquisition left a dangling pointer");
  }
  if (FakeRuntime::double_frees != 0) return fail("a buffer was freed twice");
  std::printf("scratch checks ok\n");
  return 0;
}

}  // namespace

int main() {
  const int a = barrier_checks();
  const int b = scratch_checks();
  return a | b;
}
