// Library identity and status text.
#include "cq_common.cuh"

extern "C" int cq_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char* cq_status_string(int status) {
  switch (status) {
    case CQ_OK: return "ok";
    case CQ_ERR_BAD_ARG: return "bad argument (null pointer, extent, stride, alignment or enum)";
    case CQ_ERR_UNSUPPORTED: return "shape or option outside what the sm_100a kernels implement";
    case CQ_ERR_LAUNCH: return "CUDA reported an error at kernel launch";
    case CQ_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case CQ_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case CQ_ERR_TOO_LARGE: return "problem needs more scratch than this fixed-capacity entry point holds";
    default: return "unknown status";
  }
}
