// Error reporting and device queries shared by every entry point of libb200moe.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace b200moe {
namespace {
thread_local char g_last_error[512] = "";
std::atomic<long long> g_launches{0};
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_last_error[0] = '\0'; }

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace b200moe

extern "C" int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

extern "C" int64_t b200moe_kernel_launch_count(void) {
  return b200moe::g_launches.load(std::memory_order_relaxed);
}

extern "C" const char* b200moe_last_error(void) { return b200moe::g_last_error; }
