// Version and status strings of the C ABI.
#include "common.cuh"
#include "mini_vllm_b200.h"

extern "C" int mvb_abi_version(void) { return 3; }

extern "C" const char* mvb_status_string(int status) {
  switch (status) {
    case MVB_OK: return "ok";
    case MVB_INVALID_ARGUMENT: return "invalid argument";
    case MVB_UNSUPPORTED_SHAPE: return "unsupported shape";
    case MVB_LAUNCH_FAILED: return "kernel launch failed";
    case MVB_TENSOR_MAP_FAILED: return "tensor map encoding failed";
    case MVB_MISALIGNED: return "pointer or stride not aligned";
    case MVB_NO_DRIVER_ENTRY: return "cuTensorMapEncodeTiled not available from the driver";
    case MVB_SCRATCH_TOO_SMALL: return "request needs more than the built-in 8 MiB decode scratch";
    default: return "unknown status";
  }
}
