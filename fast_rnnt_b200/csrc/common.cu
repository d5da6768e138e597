// Host-side plumbing shared by every entry point: version, thread-local error text.
#include <stdarg.h>

#include <atomic>

#include "common.cuh"

namespace frnnt {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace frnnt

extern "C" int frnnt_version(void) { return 100; }
extern "C" const char *frnnt_last_error(void) { return frnnt::g_error; }
extern "C" int frnnt_with_cuda(void) { return 1; }
namespace frnnt { long long launches(); }
extern "C" long long frnnt_launch_count(void) { return frnnt::launches(); }
