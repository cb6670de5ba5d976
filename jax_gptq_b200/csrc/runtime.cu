// Library-wide state: thread-local error text and per-device attribute cache.
#include "common.cuh"
#include <mutex>
#include <atomic>

namespace jgq {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

static std::atomic<unsigned long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
unsigned long long launches() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  // Immutable per-device cache; XLA may call in from one host thread per device.
  static int cache[64];
  static std::once_flag flags[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::call_once(flags[dev], [dev]() {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  });
  return cache[dev];
}

}  // namespace jgq

namespace jgq { unsigned long long launches(); }
extern "C" int jgq_version(void) { return 100; }
extern "C" uint64_t jgq_launch_count(void) { return (uint64_t)jgq::launches(); }
extern "C" const char* jgq_last_error(void) { return jgq::error_buffer(); }
