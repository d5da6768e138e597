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

}  // namespace frnnt

extern "C" int frnnt_version(void) { return 100; }
extern "C" const char *frnnt_last_error(void) { return frnnt::g_error; }
extern "C" int frnnt_with_cuda(void) { return 1; }
namespace frnnt { long long launches(); }
extern "C" long long frnnt_launch_count(void) { return frnnt::launches(); }
