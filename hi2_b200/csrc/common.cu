// Error text of the calling thread and the ABI version.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "common.cuh"

namespace hi2 {
namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
}  // namespace hi2

extern "C" int hi2_abi_version(void) { return 1; }
extern "C" const char* hi2_last_error(void) { return hi2::g_error; }
extern "C" long long hi2_launch_count(void) { return hi2::g_launches.load(std::memory_order_relaxed); }
