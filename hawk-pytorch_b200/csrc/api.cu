// Library-level entry points of the C ABI (version and error text).
#include "common.cuh"

extern "C" int hawk_version(void) { return HAWK_B200_ABI_VERSION; }

extern "C" const char* hawk_strerror(int status) {
  switch (status) {
    case HAWK_OK: return "ok";
    case HAWK_ERR_NULL: return "a required pointer is NULL";
    case HAWK_ERR_SHAPE: return "a dimension or stride is out of range or not a supported multiple";
    case HAWK_ERR_DTYPE: return "unknown dtype";
    case HAWK_ERR_ALIGN: return "a pointer or stride is not aligned as required";
    case HAWK_ERR_WORKSPACE: return "workspace missing or too small";
    case HAWK_ERR_LAUNCH: return "CUDA refused a kernel launch";
    case HAWK_ERR_UNSUPPORTED: return "request not supported by this build";
    case HAWK_ERR_DEVICE: return "wrong device or driver entry point unavailable";
    case HAWK_ERR_TOO_LARGE: return "size exceeds the built-in scratch of the no-allocation entry point (B*D <= 262144)";
    default: return "unknown hawk_status";
  }
}
