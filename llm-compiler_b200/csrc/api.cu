// ABI probe and error strings of libb200serve.so.
#include <atomic>

#include "b200_serve.h"

namespace b200 {
namespace {
// The launch mode belongs to the calling thread: CONSTANT_WEIGHTS and STABLE_KV_PREFIX are
// promises about what that thread's own launches may assume, and two engines driven from two
// threads must not inherit each other's. Captured launches keep the mode they were captured with.
thread_local int g_launch_mode = 0;
// Bound of the in-kernel mbarrier waits (polls); see b200_set_wait_limit.
std::atomic<unsigned> g_wait_limit{4000000u};
}
int launch_mode() { return g_launch_mode; }
unsigned wait_limit() { return g_wait_limit.load(std::memory_order_relaxed); }
namespace {
std::atomic<int> g_drop_loads{0};
}
int drop_loads() { return g_drop_loads.load(std::memory_order_relaxed); }
}  // namespace b200

extern "C" int64_t b200_debug_set_waits(int64_t poll_limit, int drop_loads) {
  if (poll_limit < 1 || poll_limit > 4000000000ll) return B200_ERR_BAD_ARGUMENT;
  b200::g_drop_loads.store(drop_loads != 0 ? 1 : 0, std::memory_order_relaxed);
  return b200::g_wait_limit.exchange(static_cast<unsigned>(poll_limit), std::memory_order_relaxed);
}

extern "C" int b200_abi_version(void) { return 104; }

extern "C" int b200_set_launch_mode(int flags) {
  if ((flags & ~(B200_LAUNCH_PROGRAMMATIC | B200_LAUNCH_CONSTANT_WEIGHTS |
                 B200_LAUNCH_STABLE_KV_PREFIX | B200_LAUNCH_LINEAR_WARP_LEVEL |
                 B200_LAUNCH_PREFILL_WARP_LEVEL)) != 0)
    return B200_ERR_BAD_ARGUMENT;
  const int previous = b200::g_launch_mode;
  b200::g_launch_mode = flags;
  return previous;
}

extern "C" int b200_get_launch_mode(void) { return b200::launch_mode(); }

extern "C" const char* b200_error_string(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_BAD_ARGUMENT: return "bad argument (null pointer, negative size or unknown enum)";
    case B200_ERR_UNSUPPORTED: return "unsupported dtype, head_dim or stride";
    case B200_ERR_ALIGNMENT: return "a pointer or stride breaks the 16-byte alignment rule";
    case B200_ERR_WORKSPACE: return "workspace missing or too small";
    case B200_ERR_LAUNCH: return "CUDA reported a launch error";
    case B200_ERR_TOO_LARGE: return "size beyond a documented maximum";
    default: return "unknown error code";
  }
}

#ifdef B200_TRACE
#include <cuda_runtime.h>
namespace b200 {
namespace {
constexpr int kMaxSetters = 16;
void (*g_setters[kMaxSetters])(unsigned long long*);
int g_setter_count = 0;
}  // namespace
void register_trace_setter(void (*setter)(unsigned long long*)) {
  if (g_setter_count < kMaxSetters) g_setters[g_setter_count++] = setter;
}
}  // namespace b200

// buffer: device memory of (1 + 8 * 65536) + (1 + 64 * 512) 64-bit words, zeroed by the caller; NULL detaches.
extern "C" int b200_trace_attach(void* buffer) {
  for (int i = 0; i < b200::g_setter_count; ++i)
    b200::g_setters[i](static_cast<unsigned long long*>(buffer));
  return cudaDeviceSynchronize() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
#endif
