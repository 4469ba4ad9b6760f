// Entry points of the tsb200 C ABI that are not tied to one kernel family.
#include <cuda.h>

#include "common.cuh"

extern "C" const char *tsb_status_string(int status) {
  switch (status) {
    case TSB_OK: return "ok";
    case TSB_ERR_DTYPE: return "unsupported dtype";
    case TSB_ERR_REDUCE: return "unsupported reduction";
    case TSB_ERR_ARG: return "invalid argument (null pointer or negative size)";
    case TSB_ERR_WORKSPACE: return "workspace missing or too small";
    case TSB_ERR_LAUNCH: return "CUDA launch failed";
    case TSB_ERR_TOO_LARGE: return "size exceeds a limit of this entry point";
    default: return "unknown status";
  }
}

extern "C" int64_t tsb_cuda_version(void) { return (int64_t)CUDA_VERSION; }
