// ABI probe and error strings of libb200serve.so.
#include <atomic>

#include "b200_serve.h"

namespace b200 {
namespace {
std::atomic<int> g_launch_mode{0};
}
int launch_mode() { return g_launch_mode.load(std::memory_order_relaxed); }
}  // namespace b200

extern "C" int b200_abi_version(void) { return 101; }

extern "C" int b200_set_launch_mode(int flags) {
  if ((flags & ~(B200_LAUNCH_PROGRAMMATIC | B200_LAUNCH_CONSTANT_WEIGHTS |
                 B200_LAUNCH_STABLE_KV_PREFIX | B200_LAUNCH_LINEAR_WARP_LEVEL |
                 B200_LAUNCH_PREFILL_WARP_LEVEL)) != 0)
    return B200_ERR_BAD_ARGUMENT;
  return b200::g_launch_mode.exchange(flags, std::memory_order_relaxed);
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
