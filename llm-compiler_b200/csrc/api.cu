// ABI probe and error strings of libb200serve.so.
#include "b200_serve.h"

extern "C" int b200_abi_version(void) { return 100; }

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
